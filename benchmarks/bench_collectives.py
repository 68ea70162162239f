"""Latency of the decode-time collectives against NCCL (torchrun, any N), one JSON line per measurement:

  allreduce   bf16 messages 16 KB ... 64 MB: one-shot push, two-shot push, NVLS one-shot, NVLS two-shot, NCCL
  gemm_ar     row-parallel GEMM + all-reduce, M in {1, 8, 32, 128}, K = 25600 / W, N = 5120: fused kernel (GEMV for
              M <= 8, tcgen05 weight-streaming kernel above) against cuBLAS + NCCL
  ep          expert-parallel dispatch + combine, hidden 7168, 256 experts, top-8, fp8 dispatch: 128 and 4096 tokens
              per rank, against two NCCL all_to_all_single calls moving the same rows in bf16

Device-timed inside CUDA graphs where the op allows it (the way decode uses them), median, max over ranks.
"""
import argparse
import json
import os

# the prefill-size EP exchange alone needs about 1 GB of receive buffers per rank: take a roomier symmetric heap than
# the 4 GiB default (180 GB of HBM per GPU)
os.environ.setdefault("TDB200_SYMM_HEAP_BYTES", str(16 << 30))
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import triton_distributed_b200 as tdb  # noqa: E402
from triton_distributed_b200 import ops  # noqa: E402
from triton_distributed_b200.ops.allreduce import AllReduceMethod  # noqa: E402


def timed(fn, rt, iters=20, warmup=5, graph=True, reps=4):
    """Median device time of one call in microseconds, max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = None
    if graph:
        rt.host_barrier()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                fn()
        torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if rt.world_size > 1:
            dist.barrier(group=rt.group)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        if g is not None:
            g.replay()
        else:
            fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3 / (reps if g is not None else 1))
    t = torch.tensor([statistics.median(ts)], device="cuda", dtype=torch.float64)
    if rt.world_size > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.group)
    rt.check_status(sync=False)
    return float(t.item())


def emit(rt, **kw):
    if rt.rank == 0:
        print(json.dumps(kw), flush=True)


def bench_allreduce(rt, sizes):
    ctx = ops.create_allreduce_ctx(max(sizes))
    methods = [AllReduceMethod.OneShot, AllReduceMethod.TwoShot]
    if rt.has_multicast:
        methods += [AllReduceMethod.OneShot_Multimem, AllReduceMethod.TwoShot_Multimem]
    for nbytes in sizes:
        x = torch.randn(nbytes // 2, device=rt.device).to(torch.bfloat16)
        out = torch.empty_like(x)
        rec = {"bench": "allreduce", "world": rt.world_size, "bytes": nbytes}
        for m in methods:
            if m == AllReduceMethod.OneShot and nbytes > (4 << 20):
                continue   # one-shot push moves W x the message; pointless for large ones
            rec[m.name + "_us"] = round(timed(lambda: ops.all_reduce(x, m, ctx, output=out), rt), 2)
        y = x.clone()
        rec["nccl_us"] = round(timed(lambda: dist.all_reduce(y, group=rt.group), rt), 2)
        best = min(v for k, v in rec.items() if k.endswith("_us") and k != "nccl_us")
        rec["best_vs_nccl"] = round(rec["nccl_us"] / best, 3)
        emit(rt, **rec)
    ctx.finalize()


def bench_gemm_ar(rt, Ms, k_local=0):
    W = rt.world_size
    K, N = (k_local or 25600 // W), 5120
    w = (torch.randn(N, K, device=rt.device) * 0.02).to(torch.bfloat16)
    wt = w.t()
    gctx = ops.create_gemm_ar_context(max_M=max(Ms), N=N)
    vctx = ops.create_gemv_ar_context(N)
    actx = ops.create_allreduce_ctx(max(4 * max(Ms) * N * 2, 1 << 20))
    for M in Ms:
        x = torch.randn(M, K, device=rt.device, dtype=torch.bfloat16)
        out = torch.empty(M, N, device=rt.device, dtype=torch.bfloat16)
        rec = {"bench": "gemm_ar", "world": W, "M": M, "K_local": K, "N": N}
        if M <= ops.GEMV_FAST_M and ops.gemv_supported(M, K):
            rec["fused_us"] = round(timed(lambda: ops.gemv_fused(x, w, out=out, ar_ctx=vctx), rt), 2)
            rec["kernel"] = "gemv"
        else:
            rec["fused_us"] = round(timed(lambda: ops.gemm_allreduce_op(gctx, x, w, output=out), rt), 2)
            rec["kernel"] = "tcgen05 swap-AB"
            rec["splits"] = ops.gemm_ar.pick_gemm_ar_splits(M, N, K)

        if M >= 32:
            # the unfused pair of own kernels: tcgen05 GEMM (128-row tiles, lib entry, not the decode dispatch) + own all-reduce
            part = torch.empty(M, N, device=rt.device, dtype=torch.bfloat16)
            lib = tdb._native.load(True)

            def two():
                lib.gemm_bf16(x, w, part, 128, 0, None)
                ops.all_reduce(part, ctx=actx, output=out)

            rec["own_gemm_then_ar_us"] = round(timed(two, rt), 2)

        def ref():
            torch.matmul(x, wt, out=out)
            dist.all_reduce(out, group=rt.group)

        rec["cublas_nccl_us"] = round(timed(ref, rt), 2)
        rec["speedup"] = round(rec["cublas_nccl_us"] / rec["fused_us"], 3)
        emit(rt, **rec)
    gctx.finalize()
    vctx.finalize()
    actx.finalize()


def bench_ep(rt, tokens_list):
    W = rt.world_size
    H, E, K = 7168, 256, 8
    if E % W:
        return
    for T in tokens_list:
        ctx = ops.create_all_to_all_context(max_m=T, hidden=H, num_tot_experts=E, topk=K, quant=True, layout="ll" if T <= 256 else "packed")
        x = torch.randn(T, H, device=rt.device).to(torch.bfloat16)
        tw, ids = torch.softmax(torch.randn(T, E, device=rt.device), -1).topk(K, dim=-1)
        tw = (tw / tw.sum(-1, keepdim=True)).float()

        def own():
            recv = ops.ep_dispatch(ctx, x, ids)
            return ops.ep_combine(ctx, recv.x_sorted, recv, tw)

        # device time of a step as a serving loop issues it: captured in a CUDA graph (no host launch gaps); the eager
        # number (host launches included) is printed beside it
        rec = {"bench": "ep_dispatch_combine", "world": W, "tokens_per_rank": T, "hidden": H, "experts": E, "topk": K,
               "own_eager_us": round(timed(own, rt, graph=False, iters=10, warmup=3), 2)}
        rec["own_us"] = round(timed(own, rt, graph=True, iters=10, warmup=2, reps=4), 2)
        # NCCL baseline: the same (token, slot) rows in bf16, equal splits, there and back
        rows = T * K // W * W
        send = torch.randn(rows, H, device=rt.device).to(torch.bfloat16)
        recvb = torch.empty_like(send)

        def ref():
            dist.all_to_all_single(recvb, send, group=rt.group)
            dist.all_to_all_single(send, recvb, group=rt.group)

        rec["nccl_two_a2a_eager_us"] = round(timed(ref, rt, graph=False, iters=10, warmup=3), 2)
        rec["nccl_two_a2a_us"] = round(timed(ref, rt, graph=True, iters=10, warmup=2, reps=4), 2)
        rec["speedup"] = round(rec["nccl_two_a2a_us"] / rec["own_us"], 3)
        emit(rt, **rec)
        ctx.finalize()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="allreduce,gemm_ar,ep")
    ap.add_argument("--sizes", default="16384,65536,262144,1048576,4194304,16777216,67108864")
    ap.add_argument("--Ms", default="1,8,32,128")
    ap.add_argument("--ep-tokens", default="128,4096")
    ap.add_argument("--gemm-ar-k", type=int, default=0, help="local K of the GEMM-AR sweep (default 25600 / world)")
    args = ap.parse_args()
    tdb.initialize_distributed(seed=0)
    rt = tdb.get_runtime()
    what = args.what.split(",")
    if "allreduce" in what and rt.world_size > 1:
        bench_allreduce(rt, [int(s) for s in args.sizes.split(",")])
    if "gemm_ar" in what and rt.world_size > 1:
        bench_gemm_ar(rt, [int(m) for m in args.Ms.split(",")], args.gemm_ar_k)
    if "ep" in what and rt.world_size > 1:
        bench_ep(rt, [int(t) for t in args.ep_tokens.split(",")])
    torch.cuda.synchronize()
    rt.host_barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
