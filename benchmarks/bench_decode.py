"""Decode latency of a Qwen3-architecture model with random weights (torchrun, TP = number of ranks):
torch eager / torch + CUDA graph (NCCL + cuBLAS) / fused GEMM+AR kernels + CUDA graph / decode megakernel.

  torchrun --nproc-per-node 8 benchmarks/bench_decode.py --model Qwen/Qwen3-32B --batch 1 --ctx 4096 [--layers 64]

Times `--steps` decode steps with CUDA events after warm-up, max over ranks; prints one JSON line per arm.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import triton_distributed_b200 as tdb  # noqa: E402
from triton_distributed_b200.mega import Qwen3Model  # noqa: E402
from triton_distributed_b200.models import DenseLLM, KV_Cache, ModelConfig  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Qwen/Qwen3-32B")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--arms", default="torch,torch_graph,gemm_ar_graph,mega",
                    help="also: mega_prefetch (megakernel with L2 prefetch tasks), prefill (see --prefill)")
    ap.add_argument("--prefill", type=int, default=2048, help="prompt length of the `prefill` arm (batch 1)")
    args = ap.parse_args()
    tdb.initialize_distributed(seed=0)
    rt = tdb.get_runtime()
    W, dev = rt.world_size, rt.device
    cfg = ModelConfig(model_name=args.model, max_length=args.ctx + args.steps + 8, rank=rt.rank, world_size=W,
                      num_layers_override=args.layers)
    model = DenseLLM(cfg)
    a = model.arch
    B = args.batch
    cache = KV_Cache(a.num_hidden_layers, B, cfg.max_length, max(1, a.num_key_value_heads // W), a.head_dim, device=dev)
    ids = torch.randint(0, a.vocab_size, (B, 1), device=dev)

    def timed(step_fn, reset):
        reset()
        for _ in range(3):
            step_fn()
        torch.cuda.synchronize()
        if W > 1:
            dist.barrier(group=rt.group)
        reset()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.steps):
            step_fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / args.steps], device=dev, dtype=torch.float64)
        if W > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.group)
        rt.check_status(sync=False)
        return float(t.item())

    def reset():
        cache.kv_offset.fill_(args.ctx)

    def emit(arm, ms):
        if rt.rank == 0:
            print(json.dumps({"arm": arm, "model": args.model, "layers": a.num_hidden_layers, "tp": W, "batch": B,
                              "ctx": args.ctx, "ms_per_step": ms}), flush=True)

    cache.rand_fill(args.ctx)
    logits = torch.empty(B, a.vocab_size, device=dev, dtype=torch.float32)

    def layer_step():
        pos = cache.kv_offset[:B].to(torch.int64).unsqueeze(1)
        logits.copy_(model.inference(ids, pos, cache))
        cache.inc_offset(1)

    def graphed(mode):
        model.init_ctx_for(mode, B)
        model.set_fwd(mode)
        reset()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                layer_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        rt.host_barrier()
        g = torch.cuda.CUDAGraph()
        reset()
        with torch.cuda.graph(g):
            layer_step()
        torch.cuda.synchronize()
        rt.host_barrier()
        return g

    arms = args.arms.split(",")
    if "torch" in arms:
        model.set_fwd("torch")
        emit("torch_eager", timed(layer_step, reset))
    if "torch_graph" in arms:
        g = graphed("torch")
        emit("torch_cuda_graph", timed(g.replay, reset))
        del g
    if "gemm_ar_graph" in arms:
        g = graphed("triton_dist_gemm_ar")
        emit("fused_gemm_ar_cuda_graph", timed(g.replay, reset))
        del g
    for arm_name, pre in (("mega", False), ("mega_prefetch", True)):
        if arm_name not in arms:
            continue
        mega = Qwen3Model(model, cache, B, prefetch=pre)

        def mega_step():
            logits.copy_(mega.mega_forward(ids))
            cache.inc_offset(1)

        emit("megakernel" + ("_prefetch" if pre else ""), timed(mega_step, reset))
        g = torch.cuda.CUDAGraph()
        reset()
        for _ in range(2):
            mega_step()
        torch.cuda.synchronize()
        rt.host_barrier()
        reset()
        with torch.cuda.graph(g):
            mega_step()
        torch.cuda.synchronize()
        rt.host_barrier()
        emit("megakernel" + ("_prefetch" if pre else "") + "_cuda_graph", timed(g.replay, reset))
        del mega, g
    if "prefill" in arms:
        # one prompt of --prefill tokens through the whole model: NCCL + cuBLAS layers against the overlapped layers
        P = args.prefill
        pcache = KV_Cache(a.num_hidden_layers, 1, P + 8, max(1, a.num_key_value_heads // W), a.head_dim, device=dev)
        pids = torch.randint(0, a.vocab_size, (1, P), device=dev)
        ppos = torch.arange(P, device=dev).unsqueeze(0)

        def prefill_step():
            pcache.kv_offset.zero_()
            model.inference(pids, ppos, pcache)

        # (the AG -> GEMM / GEMM -> RS backend shards the BATCH over the ranks, so a single prompt runs on the all-reduce one)
        for mode in ("torch", "triton_dist_AR"):
            if mode != "torch":
                model.init_ctx_for(mode, P)
            model.set_fwd(mode)
            ms = timed(prefill_step, lambda: None)
            if rt.rank == 0:
                print(json.dumps({"arm": f"prefill_{mode}", "model": args.model, "layers": a.num_hidden_layers, "tp": W,
                                  "tokens": P, "ms": ms}), flush=True)
        del pcache
    torch.cuda.synchronize()
    rt.host_barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
