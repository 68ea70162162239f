"""Sweep of the decode GEMM's cluster form on one GPU: for every Qwen3-32B per-rank linear shape (TP given by --tp) and
token count, times every feasible (tile width, cluster size) pair, the launcher's own choice, the stream-K form and
torch.matmul, and prints one JSON line per problem with the winner in the form `ops/tuned_configs.py` takes (`--json-out FILE`
writes the winners as a table that `TDB200_TUNED_CONFIGS=FILE` loads in front of the built-in one).

  python benchmarks/tune_skinny.py --tp 8,4,2 --Ms 16,32,64,128

Device-timed with CUDA events around a CUDA graph of several calls; the weights rotate over copies that together exceed
L2, so every call streams its weights from HBM.
"""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triton_distributed_b200 import ops  # noqa: E402


def timeit(fn, iters=8, warmup=2, reps=6):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3 / reps)
    return statistics.median(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", default="8,4,2")
    ap.add_argument("--Ms", default="16,32,64,128")
    ap.add_argument("--max-nt", type=int, default=4)
    ap.add_argument("--json-out", default=None,
                    help="write the winners as a table file for the TDB200_TUNED_CONFIGS environment variable")
    args = ap.parse_args()
    seen = set()
    winners = []
    for tp in [int(t) for t in args.tp.split(",")]:
        H, I, Hq, Hkv, D = 5120, 25600 // tp, 64 // tp, max(1, 8 // tp), 128
        shapes = {"qkv": ((Hq + 2 * Hkv) * D, H), "o_proj": (H, Hq * D), "gate_up": (2 * I, H), "down": (H, I)}
        for name, (N, K) in shapes.items():
            if (N, K) in seen:
                continue
            seen.add((N, K))
            ncopy = max(2, min(8, -(-(300 << 20) // (N * K * 2))))
            ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(ncopy)]
            for M in [int(m) for m in args.Ms.split(",")]:
                x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
                out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
                i = [0]

                def call(**kw):
                    i[0] = (i[0] + 1) % ncopy
                    ops.skinny_gemm(x, ws[i[0]], out=out, **kw)

                def lib():
                    i[0] = (i[0] + 1) % ncopy
                    torch.matmul(x, ws[i[0]].t(), out=out)

                rec = {"tp": tp, "op": name, "M": M, "N": N, "K": K, "torch_us": round(timeit(lib), 2),
                       "auto_us": round(timeit(lambda: call(cluster=(0, 0))), 2),
                       "stream_k_us": round(timeit(lambda: call(splits=ops.gemm_ar.pick_stream_k_splits(M, N, K))), 2)}
                grid = {}
                for nt in range(1, args.max_nt + 1):
                    for s in range(1, 9):
                        try:
                            call(cluster=(nt, s))
                            torch.cuda.synchronize()
                        except RuntimeError:
                            continue
                        grid[f"{nt}x{s}"] = round(timeit(lambda: call(cluster=(nt, s))), 2)
                best = min(grid, key=grid.get) if grid else None
                rec["grid_us"] = grid
                if best is not None:
                    nt, s = (int(v) for v in best.split("x"))
                    rec["best"] = {"cluster_nt": nt, "cluster_s": s, "us": grid[best]}
                    rec["table_line"] = (f'("skinny_gemm", 1, {ops.gemm_ar._mpad(M)}, {N}, {K}): '
                                         f'{{"cluster_nt": {nt}, "cluster_s": {s}}},')
                    winners.append({"op": "skinny_gemm", "world": 1, "rows": ops.gemm_ar._mpad(M), "n": N, "k": K,
                                    "config": {"cluster_nt": nt, "cluster_s": s}})
                print(json.dumps(rec), flush=True)
            del ws
            torch.cuda.empty_cache()
    if args.json_out:
        with open(args.json_out, "w") as f:
            json.dump(winners, f, indent=1)


if __name__ == "__main__":
    main()
