"""Per-op timing of the fused tensor-parallel GEMMs against their NCCL + cuBLAS baselines (torchrun, any N).

  torchrun --nproc-per-node N benchmarks/bench_tp_ops.py [--M 8192 --K 8192 --N 28672] [--iters 20]

Device-timed with CUDA events, L2 flushed between iterations, max over ranks.  Prints one JSON line per op.
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
from triton_distributed_b200.utils import L2Flusher, fused_roofline  # noqa: E402


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


def loop_ms(fn, iters, rt):
    """Back-to-back calls with no barrier or flush in between (how a layer stack issues them): ms per call, max over
    ranks."""
    torch.cuda.synchronize()
    if rt.world_size > 1:
        dist.barrier(group=rt.group)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda", dtype=torch.float64)
    if rt.world_size > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.group)
    return float(t.item())


def stall_summary(fn, ctx, rt, dev):
    """One call with the pair kernel's stall counters on; returns the summary of the slowest rank's view (rank 0's)."""
    ctx.stats = ops.new_stall_counters(dev)
    torch.cuda.synchronize()
    if rt.world_size > 1:
        dist.barrier(group=rt.group)
    fn()
    torch.cuda.synchronize()
    out = ops.summarize_stall_counters(ctx.stats)
    ctx.stats = None
    return {k: round(v, 4) if isinstance(v, float) else v for k, v in out.items()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, default=8192)
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--N", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--n-comm", default="0", help="comma list of comm-CTA counts for the AG-GEMM (0 = automatic)")
    ap.add_argument("--stats", type=int, default=1, help="also report the kernel's stall counters")
    ap.add_argument("--multimem", type=int, default=-1, help="AG push: 1 NVLS ring, 0 unicast, -1 the library's default")
    ap.add_argument("--only", default="", help="comma list of op names to run (default: all)")
    args = ap.parse_args()
    tdb.initialize_distributed(seed=0)
    rt = tdb.get_runtime()
    W, dev = rt.world_size, rt.device
    M, K, N = args.M, args.K, args.N
    m, n = M // W, N // W
    fl = L2Flusher(dev)
    a = torch.randn(m, K, device=dev, dtype=torch.bfloat16)
    w1 = (torch.randn(n, K, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(K, n, device=dev) * 0.02).to(torch.bfloat16)
    h = torch.empty(M, n, device=dev, dtype=torch.bfloat16)
    o = torch.empty(m, K, device=dev, dtype=torch.bfloat16)
    full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
    part = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
    w1t, w2t = w1.t(), w2.t()
    flops = 2.0 * M * K * n
    link_bytes = (W - 1) / W * M * K * 2

    only = set(v for v in args.only.split(",") if v)

    def want(name):
        return not only or name in only

    def emit(name, ms, extra=None):
        if rt.rank == 0:
            rec = {"op": name, "world": W, "M": M, "K": K, "N": N, "ms": ms}
            rec.update(fused_roofline(flops, link_bytes if W > 1 else 0.0, ms))
            if extra:
                rec.update(extra)
            print(json.dumps(rec), flush=True)

    # baselines
    def t_ag_gemm():
        if W > 1:
            dist.all_gather_into_tensor(full, a, group=rt.group)
            torch.matmul(full, w1t, out=h)
        else:
            torch.matmul(a, w1t, out=h)

    def t_gemm_rs():
        if W > 1:
            torch.matmul(h, w2t, out=part)
            dist.reduce_scatter_tensor(o, part, group=rt.group)
        else:
            torch.matmul(h, w2t, out=o)

    full.normal_()
    h.normal_()
    if want("torch_ag_gemm"):
        emit("torch_ag_gemm", timed(t_ag_gemm, args.iters, args.warmup, fl, rt))
    if want("torch_gemm_rs"):
        emit("torch_gemm_rs", timed(t_gemm_rs, args.iters, args.warmup, fl, rt))
    if want("torch_gemm_only_ag_shape"):
        emit("torch_gemm_only_ag_shape", timed(lambda: torch.matmul(full, w1t, out=h), args.iters, args.warmup, fl, rt))
    if want("own_gemm_only_ag_shape"):
        emit("own_gemm_only_ag_shape", timed(lambda: ops.gemm(full, w1, out=h), args.iters, args.warmup, fl, rt))
    if want("own_gemm_only_rs_shape"):
        emit("own_gemm_only_rs_shape", timed(lambda: ops.gemm(h, w2, out=part), args.iters, args.warmup, fl, rt))
    if want("torch_gemm_only_rs_shape"):
        emit("torch_gemm_only_rs_shape", timed(lambda: torch.matmul(h, w2t, out=part), args.iters, args.warmup, fl, rt))
    for nc in ([int(v) for v in args.n_comm.split(",")] if want("own_ag_gemm") else []):
        ag_ctx = ops.create_ag_gemm_context(max_M=M, K=K, dtype=torch.bfloat16, n_comm_ctas=nc,
                                            use_multimem=None if args.multimem < 0 else bool(args.multimem))
        f_ag = lambda: ops.ag_gemm(a, w1, ag_ctx, out=h)   # noqa: E731
        extra = {"n_comm": nc, "multimem": int(bool(ag_ctx.use_multimem))}
        ms = timed(f_ag, args.iters, args.warmup, fl, rt)
        extra["loop_ms"] = loop_ms(f_ag, args.iters, rt)
        if args.stats and W > 1:
            extra["stalls"] = stall_summary(f_ag, ag_ctx, rt, dev)
        emit("own_ag_gemm", ms, extra)
        rt.check_status()
        ag_ctx.finalize()
    if want("own_gemm_rs"):
        rs_ctx = ops.create_gemm_rs_context(max_M=M, N=K)
        f_rs = lambda: ops.gemm_rs(h, w2, rs_ctx, out=o)   # noqa: E731
        ms = timed(f_rs, args.iters, args.warmup, fl, rt)
        extra = {"loop_ms": loop_ms(f_rs, args.iters, rt)}
        if args.stats and W > 1:
            extra["stalls"] = stall_summary(f_rs, rs_ctx, rt, dev)
        emit("own_gemm_rs", ms, extra)
        rt.check_status()
        if want("own_pair_loop") and W > 1:
            ag_ctx = ops.create_ag_gemm_context(max_M=M, K=K, dtype=torch.bfloat16)

            def both():
                ops.ag_gemm(a, w1, ag_ctx, out=h)
                ops.gemm_rs(h, w2, rs_ctx, out=o)
            for _ in range(3):
                both()
            emit("own_pair_loop", loop_ms(both, args.iters, rt))
            rt.check_status()
    # ---------------------------------------------------------------- block-scaled fp8 variant of the same shapes
    if want("own_fp8") or want("own_gemm_fp8_only") or want("own_ag_gemm_fp8") or want("own_gemm_rs_fp8"):
        aq, a_s = ops.quantize_act_1x128(a)
        w1q, w1s = ops.quantize_weight_128x128(w1)
        w2q, w2s = ops.quantize_weight_128x128(w2)
        fullq, full_s = ops.quantize_act_1x128(full)
        hq, h_s = ops.quantize_act_1x128(h)
        emit("own_gemm_fp8_only_ag_shape", timed(lambda: ops.gemm_fp8_blockscaled(fullq, full_s, w1q, w1s, out=h),
                                                 args.iters, args.warmup, fl, rt))
        emit("own_gemm_fp8_only_rs_shape", timed(lambda: ops.gemm_fp8_blockscaled(hq, h_s, w2q, w2s, out=part),
                                                 args.iters, args.warmup, fl, rt))
        if W > 1:
            link8 = {"link_bytes_fp8": (W - 1) / W * M * (K + K // 128 * 4)}
            agc = ops.create_ag_gemm_fp8_context(max_M=M, K=K)
            f_ag8 = lambda: ops.ag_gemm_fp8(aq, a_s, w1q, w1s, agc, out=h)   # noqa: E731
            ms = timed(f_ag8, args.iters, args.warmup, fl, rt)
            extra = dict(link8, loop_ms=loop_ms(f_ag8, args.iters, rt))
            if args.stats:
                extra["stalls"] = stall_summary(f_ag8, agc, rt, dev)
            emit("own_ag_gemm_fp8", ms, extra)
            rt.check_status()
            rsc = ops.create_gemm_rs_fp8_context(max_M=M, N=K)
            f_rs8 = lambda: ops.gemm_rs_fp8(hq, h_s, w2q, w2s, rsc, out=o)   # noqa: E731
            ms = timed(f_rs8, args.iters, args.warmup, fl, rt)
            extra = {"loop_ms": loop_ms(f_rs8, args.iters, rt)}
            if args.stats:
                extra["stalls"] = stall_summary(f_rs8, rsc, rt, dev)
            emit("own_gemm_rs_fp8", ms, extra)
            rt.check_status()
    tdb.finalize_distributed()


if __name__ == "__main__":
    main()
