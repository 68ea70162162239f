"""Tensor-parallel MoE ops on the DeepSeek-V3-shaped config (hidden 7168, 256 experts, top-8, expert intermediate
2048, 8192 tokens): the two fused launches against the same grouped GEMMs with stand-alone NCCL collectives.

  torchrun --nproc-per-node N benchmarks/bench_moe.py [--tokens 8192 --hidden 7168 --experts 256 --topk 8 --inter 2048]

Device-timed (CUDA events, max over ranks, L2 flushed between iterations).  One JSON line per op.
"""
import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import triton_distributed_b200 as tdb  # noqa: E402
from triton_distributed_b200 import ops  # noqa: E402
from triton_distributed_b200.utils import L2Flusher  # noqa: E402


def timed(fn, iters, warmup, fl, rt):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        fl.flush()
        if rt.world_size > 1:
            dist.barrier(group=rt.group)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    t = torch.tensor(ts, device="cuda", dtype=torch.float64)
    if rt.world_size > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.group)
    return statistics.median(t.tolist())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--n-chunks", default="1,2,4")
    ap.add_argument("--n-red", default="16,32,48", help="reducer CTA counts of the fused down projection to try")
    args = ap.parse_args()
    tdb.initialize_distributed(seed=0)
    rt = tdb.get_runtime()
    W, dev = rt.world_size, rt.device
    T, H, E, k = args.tokens, args.hidden, args.experts, args.topk
    il = args.inter // W
    tl = T // W
    fl = L2Flusher(dev)
    g = torch.Generator(device=dev).manual_seed(1)
    x_full = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    x = x_full[rt.rank * tl:(rt.rank + 1) * tl].contiguous()
    w13 = (torch.randn(E, 2 * il, H, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, il, device=dev) * 0.02).to(torch.bfloat16)
    ids, tw = ops.topk_router(torch.randn(T, E, device=dev, generator=g), k)
    agc = ops.create_ag_group_gemm_context(T, 2 * il, H, E, k)
    rsc = ops.create_moe_rs_context(max_token_num=T, hidden_dim=H, num_experts=E, topk=k)
    full = torch.empty(T, H, device=dev, dtype=torch.bfloat16)

    def emit(name, ms, flops, extra=None):
        if rt.rank == 0:
            rec = {"op": name, "world": W, "tokens": T, "hidden": H, "experts": E, "topk": k, "inter_local": il, "ms": ms,
                   "tflops_per_rank": flops / ms / 1e9}
            if extra:
                rec.update(extra)
            print(json.dumps(rec), flush=True)

    up_flops = 2.0 * T * k * H * 2 * il
    down_flops = 2.0 * T * k * il * H

    # ---- up projection: all-gather -> grouped GEMM
    def up_fused():
        return ops.ag_group_gemm(x, w13, agc, ids, sorted_output=True)

    def up_unfused():
        if W > 1:
            dist.all_gather_into_tensor(full, x, group=rt.group)
            src = full
        else:
            src = x
        srt = ops.sort_topk_ids_align_block_size(ids, E)
        return ops.group_gemm_gather(src, w13, srt, a_row_div=k), srt

    emit("moe_up_fused_ag_group_gemm", timed(up_fused, args.iters, args.warmup, fl, rt), up_flops)
    emit("moe_up_nccl_ag_then_group_gemm", timed(up_unfused, args.iters, args.warmup, fl, rt), up_flops)
    rt.check_status()
    hs, srt = up_fused()
    act = ops.silu_mul(hs)

    # ---- down projection: grouped GEMM -> top-k reduce -> reduce-scatter
    part_out = torch.empty(tl, H, device=dev, dtype=torch.bfloat16)

    def down_unfused():
        iota = torch.arange(srt.sorted_ids.numel(), dtype=torch.int32, device=dev)
        gids = torch.where(srt.sorted_ids >= 0, iota, srt.sorted_ids)
        s2 = ops.MoESort(gids, srt.pos_of, srt.tile_expert, srt.offsets, srt.meta, srt.counts, srt.k)
        y = ops.group_gemm_gather(act, w2, s2, a_row_div=1)
        red = ops.moe.reduce_topk(y, srt, tw, T)
        if W > 1:
            dist.reduce_scatter_tensor(part_out, red, group=rt.group)
            return part_out
        return red

    for nr in [int(v) for v in args.n_red.split(",")]:
        rsc.finalize()
        rsc = ops.create_moe_rs_context(max_token_num=T, hidden_dim=H, num_experts=E, topk=k, n_red_ctas=nr)
        for nc in [int(v) for v in args.n_chunks.split(",")]:
            emit("moe_down_fused_group_gemm_reduce_rs",
                 timed(lambda: ops.run_moe_reduce_rs(act, w2, ids, tw, rsc, n_chunks=nc, sort=srt), args.iters, args.warmup, fl, rt),
                 down_flops, {"n_chunks": nc, "n_red": nr})
            rt.check_status()
    emit("moe_down_group_gemm_then_topk_reduce_then_nccl_rs", timed(down_unfused, args.iters, args.warmup, fl, rt), down_flops)
    rt.check_status()
    torch.cuda.synchronize()
    rt.host_barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
