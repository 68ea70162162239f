"""Multi-GPU checks (torchrun, one rank per GPU): heap + device API, collectives, fused AG-GEMM / GEMM-RS.

Every check compares against torch.distributed (NCCL) + torch fp32 math on the same data.  Exits non-zero on the
first failing rank.  Optional args: --quick (small sizes only), --nvls 0|1.
"""
import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import triton_distributed_b200 as tdb  # noqa: E402
from triton_distributed_b200 import _native, ops  # noqa: E402


def log(rt, *a):
    if rt.rank == 0:
        print(*a, flush=True)


def check_primitives(rt):
    lib = _native.load(True)
    W, n = rt.world_size, 300
    data = rt.symm_tensor((W * n,), torch.int32)
    scratch = rt.symm_tensor((2 * n,), torch.int32)
    sig = rt.symm_tensor((32,), torch.int32)
    bar = rt.symm_tensor((16,), torch.int32)
    torch.cuda.synchronize()
    rt.host_barrier()
    for epoch in (1, 2, 3):
        lib.primitives_test(rt.heap, data, scratch, sig, bar, n, epoch, 5.0)
        torch.cuda.synchronize()
        rt.check_status()
        prev = (rt.rank + W - 1) % W
        pp = (prev + W - 1) % W
        ar = torch.arange(n, device="cuda", dtype=torch.int32)
        assert torch.equal(data[prev * n:(prev + 1) * n], ar + (prev + 1) * 1000), "putmem_signal_block"
        assert torch.equal(scratch[:n], ar + (pp + 1) * 1000), "getmem_warp"
        assert sig[0].item() == epoch
        for r in range(W):
            assert sig[8 + r].item() == epoch * 100 + r, "thread put"
        rt.host_barrier()   # a faster peer must not start the next epoch's puts while this rank still checks
    # peer views and the multicast view
    t = rt.symm_tensor((16,), torch.float32)
    t.fill_(float(rt.rank + 1))
    torch.cuda.synchronize()
    rt.barrier_all_on_stream()
    torch.cuda.synchronize()
    for r in range(W):
        assert rt.peer_view(t, r)[0].item() == float(r + 1), "peer view"
    rt.barrier_all_on_stream()
    torch.cuda.synchronize()
    log(rt, f"OK primitives (heap mode {rt.heap.mode}, multicast {rt.has_multicast})")


def check_allreduce(rt, quick):
    W = rt.world_size
    ctx = ops.create_allreduce_ctx(64 << 20)
    methods = [ops.AllReduceMethod.OneShot, ops.AllReduceMethod.TwoShot]
    if rt.has_multicast:
        methods += [ops.AllReduceMethod.OneShot_Multimem, ops.AllReduceMethod.TwoShot_Multimem]
    sizes = [8, 1000, 8192, 65536 + 8, 1 << 20] + ([] if quick else [4 << 20, (16 << 20) + 24])
    for dtype in (torch.bfloat16, torch.float32, torch.float16):
        for n in sizes:
            x = (torch.randn(n, device="cuda") * 0.01 * (rt.rank + 1)).to(dtype)
            ref = x.clone()
            dist.all_reduce(ref, group=rt.group)
            for m in methods:
                if n * x.element_size() > (4 << 20) and m == ops.AllReduceMethod.OneShot:
                    continue
                out = ops.all_reduce(x, method=m, ctx=ctx)
                torch.cuda.synchronize()
                rt.check_status()
                tol = 2e-2 if dtype != torch.float32 else 1e-4
                err = (out.float() - ref.float()).abs().max().item()
                assert err <= tol * max(1.0, ref.float().abs().max().item()), f"all_reduce {m} {dtype} n={n}: err {err}"
    # back-to-back calls without host sync (buffer parity / epoch logic), plus auto method
    x = torch.randn(4096, device="cuda", dtype=torch.bfloat16)
    outs = [ops.all_reduce(x * (i + 1), ctx=ctx) for i in range(8)]
    ref = x.clone().float()
    dist.all_reduce(ref, group=rt.group)
    torch.cuda.synchronize()
    for i, o in enumerate(outs):
        assert (o.float() - ref * (i + 1)).abs().max().item() < 0.05 * (i + 1) * W, "back-to-back all_reduce"
    log(rt, "OK all_reduce", [m.name for m in methods])


def check_rs_ag(rt):
    W = rt.world_size
    M, N = 64 * W, 512
    ctx = ops.create_reduce_scater_2d_ctx(M, N, dtype=torch.bfloat16)
    for use_nvls in ([True, False] if rt.has_multicast else [False]):
        ctx.use_nvls = use_nvls
        x = (torch.randn(M, N, device="cuda") * 0.1 * (rt.rank + 1)).to(torch.bfloat16)
        out = ops.reduce_scatter_2d_op(x, ctx)
        ref = torch.empty(M // W, N, device="cuda", dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(ref, x, group=rt.group)
        torch.cuda.synchronize()
        rt.check_status()
        assert (out.float() - ref.float()).abs().max().item() < 0.05 * W, f"reduce_scatter nvls={use_nvls}"
    agc = ops.create_fast_allgather_context()
    for mode in [ops.AllGatherMethod.All2All_IntraNode, ops.AllGatherMethod.All2All_Pull] + (
            [ops.AllGatherMethod.NVLS] if rt.has_multicast else []):
        for n in (16, 4096, 1 << 18):
            buf = rt.symm_tensor((W, n), torch.float32)
            mine = torch.randn(n, device="cuda")
            buf[rt.rank].copy_(mine)
            ref = torch.empty(W, n, device="cuda")
            dist.all_gather_into_tensor(ref, mine, group=rt.group)
            ops.fast_allgather(buf, agc, mode)
            torch.cuda.synchronize()
            rt.check_status()
            assert torch.equal(buf, ref), f"fast_allgather {mode} n={n}"
            rt.host_barrier()
            rt.symm_free(buf)
    for n in (2, 64, 4096):
        x = torch.randn(n, device="cuda")
        ref = torch.empty(W, n, device="cuda")
        dist.all_gather_into_tensor(ref, x, group=rt.group)
        for _ in range(3):
            out = ops.all_gather_ll(x, agc)
        torch.cuda.synchronize()
        rt.check_status()
        assert torch.equal(out, ref), f"all_gather_ll n={n}"
    log(rt, "OK reduce_scatter / all_gather")


def check_fused_gemms(rt, quick):
    W = rt.world_size
    # (2560, 1024, 256): on two ranks 80 pair tiles, more than one wave, so the tail runs as half-width tiles
    shapes = [(128, 256, 256), (300, 520, 264), (1024, 1024, 512), (2560, 1024, 256)] + (
        [] if quick else [(1024, 3584, 8192)])
    for (m, N, K) in shapes:   # m = rows per rank
        for use_mc in ([True, False] if rt.has_multicast else [False]):
            ctx = ops.create_ag_gemm_context(max_M=m * W, K=K, dtype=torch.bfloat16, use_multimem=use_mc)
            for it in range(5):
                # iterations 3 and 4 repeat on the single-CTA kernel where the automatic choice is the CTA-pair kernel
                ctx.kernel_form = "auto" if it < 3 else "single"
                a = (torch.randn(m, K, device="cuda") * (0.5 + 0.1 * rt.rank)).to(torch.bfloat16)
                b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
                strag = (it % W, 0.02) if it == 1 else None
                out = ops.ag_gemm(a, b, ctx, straggler_option=strag)
                full = torch.empty(m * W, K, device="cuda", dtype=torch.bfloat16)
                dist.all_gather_into_tensor(full, a, group=rt.group)
                ref = full.float() @ b.float().t()
                torch.cuda.synchronize()
                rt.check_status()
                err = (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
                assert err < 2e-2, f"ag_gemm m={m} N={N} K={K} mc={use_mc} it={it}: rel err {err}"
                torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=3e-2)
            ctx.finalize()
    for (m, N, K) in shapes:   # m = rows per rank of the output
        ctx = ops.create_gemm_rs_context(max_M=m * W, N=N)
        for it in range(5):
            ctx.kernel_form = "auto" if it < 3 else "single"
            a = (torch.randn(m * W, K, device="cuda") * 0.1 * (rt.rank + 1)).to(torch.bfloat16)
            b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
            out = ops.gemm_rs(a, b, ctx)
            part = a.float() @ b.float().t()
            dist.all_reduce(part, group=rt.group)
            ref = part[rt.rank * m:(rt.rank + 1) * m]
            torch.cuda.synchronize()
            rt.check_status()
            err = (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
            assert err < 3e-2, f"gemm_rs m={m} N={N} K={K} it={it}: rel err {err}"
        ctx.finalize()
    log(rt, "OK ag_gemm / gemm_rs")


def check_fp8_fused(rt):
    """Block-scaled fp8 AG-GEMM / GEMM-RS (one launch each) against the fp32 restatement over NCCL-gathered operands."""
    W = rt.world_size
    for (m, N, K) in [(128, 256, 256), (300, 520, 384), (1024, 1024, 1024), (2560, 512, 512)]:   # m = rows per rank
        ctx = ops.create_ag_gemm_fp8_context(max_M=m * W, K=K)
        b = torch.randn(N, K, device="cuda") * 0.05
        bq, bs = ops.quantize_weight_128x128(b)
        for it in range(3):
            a = (torch.randn(m, K, device="cuda") * (0.5 + rt.rank + it)).to(torch.bfloat16)
            aq, a_s = ops.quantize_act_1x128(a)
            out = ops.ag_gemm_fp8(aq, a_s, bq, bs, ctx)
            ref = ops.ag_gemm_fp8_reference(aq, a_s, bq, bs, rt.group)
            torch.cuda.synchronize()
            rt.check_status()
            torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().mean().item() + 1e-3)
        ctx.finalize()
    for (m, N, K) in [(128, 256, 256), (300, 520, 384), (1024, 1024, 1024), (2560, 512, 512)]:   # m = output rows per rank
        ctx = ops.create_gemm_rs_fp8_context(max_M=m * W, N=N)
        for it in range(3):
            a = (torch.randn(m * W, K, device="cuda") * (0.5 + 0.3 * rt.rank)).to(torch.bfloat16)
            b = torch.randn(N, K, device="cuda") * 0.05
            aq, a_s = ops.quantize_act_1x128(a)
            bq, bs = ops.quantize_weight_128x128(b)
            out = ops.gemm_rs_fp8(aq, a_s, bq, bs, ctx)
            part = ops.gemm_fp8_blockscaled_reference(aq, a_s, bq, bs)
            dist.all_reduce(part, group=rt.group)
            ref = part[rt.rank * m:(rt.rank + 1) * m]
            torch.cuda.synchronize()
            rt.check_status()
            # partial tiles travel as bf16: one rounding per source rank on top of the output rounding
            torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2 * ref.abs().mean().item() + 1e-3)
        ctx.finalize()
    log(rt, "OK fp8 ag_gemm / gemm_rs")


def check_gemm_ar(rt):
    W = rt.world_size
    for (N, K) in [(5120, 3200), (1280, 640), (520, 264)]:
        for use_mc in ([True, False] if rt.has_multicast else [False]):
            ctx = ops.create_gemm_ar_context(max_M=128, N=N, use_multimem=use_mc)
            for M in (1, 8, 32, 128, 77):
                for it in range(2):
                    a = (torch.randn(M, K, device="cuda") * 0.1 * (rt.rank + 1)).to(torch.bfloat16)
                    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
                    out = ops.gemm_allreduce_op(ctx, a, b)
                    ref = a.float() @ b.float().t()
                    dist.all_reduce(ref, group=rt.group)
                    torch.cuda.synchronize()
                    rt.check_status()
                    err = (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
                    assert err < 3e-2, f"gemm_ar M={M} N={N} K={K} mc={use_mc} it={it}: rel err {err}"
            ctx.finalize()
    log(rt, "OK gemm_allreduce")


def check_gemv_ar(rt):
    """Fused decode GEMV: RMSNorm / SiLU*up prologue, all-reduce + in-place residual epilogue, both reduce paths."""
    for (N, K) in [(5120, 3200), (5120, 1024), (264, 520)]:
        for use_mc in ([True, False] if rt.has_multicast else [False]):
            ctx = ops.create_gemv_ar_context(N, use_multimem=use_mc)
            for M in (1, 3, 8, 16):
                for it, mode in enumerate(("plain", "silu", "norm", "plain")):
                    torch.manual_seed(1000 * M + it)   # same residual stream on every rank
                    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
                    torch.manual_seed(77 + rt.rank + 10 * it)
                    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
                    x = torch.randn(M, 2 * K if mode == "silu" else K, device="cuda", dtype=torch.bfloat16)
                    kw = {"silu_mul": True} if mode == "silu" else {}
                    if mode == "norm":
                        kw["norm_weight"] = (1.0 + 0.1 * torch.randn(K, device="cuda")).to(torch.bfloat16)
                    ref = ops.gemv_reference(x, w, residual=res, group=rt.group, all_reduce=True, **kw).float()
                    buf = res.clone()
                    ops.gemv_fused(x, w, out=buf, residual=buf, ar_ctx=ctx, **kw)
                    torch.cuda.synchronize()
                    rt.check_status()
                    err = (buf.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
                    assert err < 3e-2, f"gemv_ar {mode} M={M} N={N} K={K} mc={use_mc}: rel err {err}"
            ctx.finalize()
    log(rt, "OK gemv_allreduce")


def check_dist_decode(rt):
    from triton_distributed_b200.parallel import SpGQAFlashDecodeAttention

    W = rt.world_size
    B, Hq, Hkv, D, page = 3, 16, 2, 128, 16
    layer = SpGQAFlashDecodeAttention(rt.rank, 0, W, 1, Hq, Hkv, D, D, page_size=page, max_allowed_batch=B)
    g = torch.Generator(device="cuda").manual_seed(7)   # same data on every rank
    lens_global = [1000, 37, 4096 + 5]
    max_len = max(lens_global)
    k_full = torch.randn(B, max_len, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    v_full = torch.randn(B, max_len, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16, generator=g)
    # shard the KV over ranks: rank r owns a contiguous slice of every sequence
    per = [(n + W - 1) // W for n in lens_global]
    local_lens = [max(0, min(p, n - rt.rank * p)) for p, n in zip(per, lens_global)]
    pages_per_seq = (max(per) + page - 1) // page
    k_cache = torch.zeros(B * pages_per_seq, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    bt = torch.arange(B * pages_per_seq, dtype=torch.int32, device="cuda").reshape(B, pages_per_seq)
    for b in range(B):
        n0 = rt.rank * per[b]
        ln = local_lens[b]
        if ln > 0:
            k_cache.view(B, pages_per_seq * page, Hkv, D)[b, :ln] = k_full[b, n0:n0 + ln]
            v_cache.view(B, pages_per_seq * page, Hkv, D)[b, :ln] = v_full[b, n0:n0 + ln]
    global_kv_lens = torch.zeros(W, B, dtype=torch.int32, device="cuda")
    for r in range(W):
        for b in range(B):
            global_kv_lens[r, b] = max(0, min(per[b], lens_global[b] - r * per[b]))
    # oracle: plain attention over the full KV
    kf = k_full.float().repeat_interleave(Hq // Hkv, dim=2)
    vf = v_full.float().repeat_interleave(Hq // Hkv, dim=2)
    refs = []
    for b in range(B):
        n = lens_global[b]
        s = torch.einsum("hd,khd->hk", q[b].float(), kf[b, :n]) / (D ** 0.5)
        refs.append(torch.einsum("hk,khd->hd", torch.softmax(s, -1), vf[b, :n]))
    # the one-launch form (split-KV + exchange + merge in one kernel) and the two-launch form, alternating on the same
    # staging buffers and epoch counter
    for it in range(6):
        layer.one_launch = it % 3 != 2
        out = layer.forward(q, k_cache, v_cache, global_kv_lens, bt)
        torch.cuda.synchronize()
        rt.check_status()
        assert layer.last_launches == (1 if layer.one_launch else 2), layer.last_launches
        for b in range(B):
            err = (out[b].float() - refs[b]).abs().max().item()
            assert err < 3e-2, f"dist flash decode (launches={layer.last_launches}) it={it} b={b}: err {err}"
    layer.one_launch = None          # automatic choice
    out = layer.forward(q, k_cache, v_cache, global_kv_lens, bt)
    torch.cuda.synchronize()
    rt.check_status()
    assert layer.last_launches in (1, 2)
    for b in range(B):
        assert (out[b].float() - refs[b]).abs().max().item() < 3e-2
    log(rt, "OK distributed flash-decode")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    tdb.initialize_distributed(seed=42)
    rt = tdb.get_runtime()
    t0 = time.time()
    checks = {"primitives": lambda: check_primitives(rt), "allreduce": lambda: check_allreduce(rt, args.quick),
              "rs_ag": lambda: check_rs_ag(rt), "fused": lambda: check_fused_gemms(rt, args.quick),
              "fp8": lambda: check_fp8_fused(rt), "gemm_ar": lambda: check_gemm_ar(rt), "gemv_ar": lambda: check_gemv_ar(rt),
              "dist_decode": lambda: check_dist_decode(rt)}
    for name, fn in checks.items():
        if args.only and name not in args.only.split(","):
            continue
        fn()
        torch.cuda.synchronize()
        rt.host_barrier()
    log(rt, f"ALL OK in {time.time() - t0:.1f}s")
    torch.cuda.synchronize()
    rt.host_barrier()
    sys.stdout.flush()
    os._exit(0)   # skip interpreter teardown: nothing left to check, and it must not delay the launcher


if __name__ == "__main__":
    main()
