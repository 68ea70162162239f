"""Minimal token-id generation server: rank 0 listens on a TCP port for JSON lines, every rank runs the engine.

    torchrun --nproc-per-node 8 examples/model_server.py --model Qwen/Qwen3-32B --backend triton_dist_gemm_ar --port 8765
    echo '{"input_ids": [[1, 2, 3]], "gen_len": 16}' | nc 127.0.0.1 8765

Request: ``{"input_ids": [[...], ...], "gen_len": n}`` (token ids; tokenisation is the client's job), ``{"cmd": "stop"}``
ends the server.  Reply: ``{"output_ids": [[...], ...], "ms_per_token": t}``.  Rank 0 broadcasts every request to the
other ranks (``broadcast_object_list``), all ranks call ``Engine.serve`` together.  Weights come from ``--checkpoint``
(a directory of safetensors files) or are random.  Counterpart of the reference's demo server
(python/triton_dist/mega_triton_kernel/test/models/model_server.py: rank-0 socket + broadcast of the request).
"""
import argparse
import json
import os
import socket
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import triton_distributed_b200 as tdb  # noqa: E402
from triton_distributed_b200.models import Engine, ModelConfig  # noqa: E402


def check_request(engine, req):
    """Validate a client's request on the host (every rank runs the same check on the broadcast copy, so all ranks
    agree): returns (ids, gen_len) or raises ValueError.  Nothing a client sends reaches a kernel unchecked."""
    if not isinstance(req, dict) or "input_ids" not in req:
        raise ValueError("request needs an 'input_ids' field")
    try:
        ids = torch.tensor(req["input_ids"], dtype=torch.int64)
        gen_len = int(req.get("gen_len", 16))
    except (TypeError, ValueError, RuntimeError) as e:
        raise ValueError(f"malformed request: {e}")
    engine.validate_request(ids, gen_len)
    return ids, gen_len


def handle(engine, req):
    try:
        ids, gen_len = check_request(engine, req)
    except ValueError as e:
        return {"error": str(e)}
    t0 = time.perf_counter()
    out = engine.serve(ids, gen_len)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    return {"output_ids": out.tolist(), "ms_per_token": 1e3 * dt / max(1, gen_len)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-dense")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--backend", default="torch")
    ap.add_argument("--max-length", type=int, default=4096)
    ap.add_argument("--port", type=int, default=8765)
    ap.add_argument("--max-requests", type=int, default=0, help="stop after this many requests (0 = until 'stop')")
    args = ap.parse_args()
    tdb.initialize_distributed(seed=0)
    rt = tdb.get_runtime()
    cfg = ModelConfig(model_name=args.model, max_length=args.max_length, rank=rt.rank, world_size=rt.world_size,
                      local_only=args.checkpoint is None, checkpoint_dir=args.checkpoint)
    engine = Engine(cfg)
    engine.backend = args.backend
    srv = None
    if rt.rank == 0:
        srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind(("127.0.0.1", args.port))
        srv.listen(4)
        print(f"serving {args.model} on 127.0.0.1:{args.port} with {rt.world_size} rank(s)", flush=True)
    served = 0
    while True:
        box, conn = [None], None
        if rt.rank == 0:
            conn, _ = srv.accept()
            line = conn.makefile("r").readline()
            try:
                box[0] = json.loads(line)
            except json.JSONDecodeError as e:
                box[0] = {"error": str(e)}
        if rt.world_size > 1:
            dist.broadcast_object_list(box, src=0, group=rt.cpu_group if getattr(rt, "cpu_group", None) else rt.group)
        req = box[0]
        if "error" in req or req.get("cmd") == "stop":
            if conn is not None:
                conn.sendall((json.dumps({"ok": req.get("cmd") == "stop", **req}) + "\n").encode())
                conn.close()
            if req.get("cmd") == "stop":
                break
            continue
        rep = handle(engine, req)
        if conn is not None:
            conn.sendall((json.dumps(rep) + "\n").encode())
            conn.close()
        served += 1
        if args.max_requests and served >= args.max_requests:
            break
    if srv is not None:
        srv.close()
    tdb.finalize_distributed()


if __name__ == "__main__":
    main()
