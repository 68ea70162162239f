"""tcgen05 GEMM against an fp32 torch reference (single GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(M, N, K, block_n=0, seed=0):
    from triton_distributed_b200.ops import gemm

    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, generator=g)
    b = (torch.randn(N, K, device="cuda", dtype=torch.float32, generator=g) * 0.05).to(torch.bfloat16)
    out = gemm(a, b, block_n=block_n)
    ref = a.float() @ b.float().t()
    torch.cuda.synchronize()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < 2e-2, f"M={M} N={N} K={K} block_n={block_n}: max err {err} (scale {scale})"
    # element-wise: the only error a correct kernel makes is the bf16 rounding of the output (2^-9 relative); one
    # dropped or doubled 64-wide k-block moves an element by about 0.05 * 8 = 0.4, far outside this band
    torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("shape", [(128, 256, 64), (128, 256, 256), (256, 512, 1024), (1024, 1024, 2048)])
def test_gemm_aligned(shape):
    _check(*shape)


@pytest.mark.parametrize("shape", [(100, 200, 72), (4091, 264, 520), (1, 5120, 3200), (257, 136, 8)])
def test_gemm_ragged(shape):
    _check(*shape)


@pytest.mark.parametrize("block_n", [128, 256])
def test_gemm_block_n(block_n):
    _check(512, 768, 512, block_n=block_n)


@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 512), (384, 512, 256), (1000, 520, 264),
                                   (4096, 4096, 512), (8192, 2048, 1024)])
def test_gemm_cta_pair(shape):
    # 256 x 256 tiles over two SMs (cta_group::2); 384 and 1000 rows leave the second CTA of a pair without rows
    _check(*shape, block_n=512)


def test_gemm_large_k():
    # the benchmark's K: 128 k-blocks per tile, the smem ring wraps 21 times per tile
    _check(512, 512, 8192, block_n=512)
    _check(256, 384, 8192)


@pytest.mark.parametrize("shape", [(2048, 2560, 512),    # 80 pair tiles on 74 pairs: 6 tail tiles run as 12 halves
                                   (2048, 2460, 256),    # last tile column is 156 wide: second half has 28 columns
                                   (2048, 2360, 256),    # last tile column is 56 wide: its second half is empty
                                   (2304, 2560, 320)])   # 90 tiles: 16 tail tiles as 32 halves
def test_gemm_cta_pair_split_tail(shape):
    _check(*shape, block_n=512)


def test_gemm_stall_counters():
    from triton_distributed_b200.ops import STALL_COUNTERS, gemm, new_stall_counters, summarize_stall_counters

    a = torch.randn(2048, 1024, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(2560, 1024, device="cuda") * 0.05).to(torch.bfloat16)
    st = new_stall_counters(a.device)
    out = gemm(a, b, block_n=512, stats=st)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), a.float() @ b.float().t(), rtol=1e-2, atol=2e-2)
    summ = summarize_stall_counters(st)
    assert summ["ctas"] == 148 and summ["cta_total_cycles_max"] > 0
    assert all(0.0 <= summ[f"{n}_mean_frac"] <= 1.0 for n in STALL_COUNTERS[:-1])


def test_gemm_many_tiles_per_cta():
    # more tiles than CTAs: exercises the smem ring and both TMEM accumulator buffers across tiles
    _check(4096, 4096, 512)


def test_gemm_strided_views():
    from triton_distributed_b200.ops import gemm

    a_full = torch.randn(300, 1024, device="cuda", dtype=torch.bfloat16)
    b_full = (torch.randn(400, 1024, device="cuda") * 0.05).to(torch.bfloat16)
    a, b = a_full[:, :512], b_full[:, 512:]
    out = gemm(a, b)
    ref = a.float() @ b.float().t()
    assert (out.float() - ref).abs().max().item() / ref.abs().max().item() < 2e-2


@pytest.mark.parametrize("shape", [(1, 5120, 3200), (8, 1280, 5120), (32, 6400, 5120), (128, 5120, 3200), (200, 520, 264),
                                   (16, 18992, 5120), (3, 136, 64)])
def test_skinny_gemm_split_k(shape):
    from triton_distributed_b200.ops import skinny_gemm

    M, N, K = shape
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    for splits in (0, 1, 3):
        for _ in range(2):   # twice: the kernel must leave its scratch clean
            out = skinny_gemm(a, b, splits=splits)
        torch.cuda.synchronize()
        err = (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
        assert err < 2e-2, f"skinny {shape} splits={splits}: rel err {err}"


def test_skinny_gemm_stream_k_scratch_covers_the_token_pad():
    """65 tokens are padded to 128 in the column-major accumulation buffer of the stream-K form: the scratch must be
    sized by the pad (150 column tiles here, so the cluster form does not apply and every tile is split)."""
    from triton_distributed_b200.ops import gemm_ar, skinny_gemm

    M, N, K = 65, 19200, 1024
    assert gemm_ar.split_scratch_elems(M, N) == 19200 * 128
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    for splits in (0, 3):
        for _ in range(2):
            out = skinny_gemm(a, b, splits=splits)
        torch.cuda.synchronize()
        err = (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
        assert err < 2e-2, f"splits={splits}: rel err {err}"


@pytest.mark.parametrize("shape,cluster", [
    ((16, 2560, 5120), (1, 6)), ((16, 2560, 5120), (2, 8)), ((16, 2560, 5120), (3, 4)), ((16, 2560, 5120), (4, 3)),
    ((128, 5120, 2048), (1, 3)), ((128, 5120, 2048), (2, 5)), ((128, 5120, 2048), (3, 2)),
    ((64, 520, 264), (1, 1)), ((64, 520, 264), (2, 2)), ((33, 520, 264), (3, 1)), ((200, 1280, 1024), (1, 4)),
])
def test_skinny_gemm_cluster_forms(shape, cluster):
    """Every tile width / cluster size of the cluster form against the fp32 reference (column edge: N = 520)."""
    from triton_distributed_b200.ops import skinny_gemm

    M, N, K = shape
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    try:
        out = skinny_gemm(a, b, cluster=cluster)
    except RuntimeError as e:
        pytest.skip(f"cluster form {cluster} cannot run here: {e}")
    out = skinny_gemm(a, b, cluster=cluster)
    torch.cuda.synchronize()
    err = (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
    assert err < 2e-2, f"cluster form {cluster} on {shape}: rel err {err}"


@pytest.mark.parametrize("M", [1, 2, 3, 4, 8, 12, 16])
@pytest.mark.parametrize("mode", ["plain", "norm", "silu", "norm_residual"])
def test_gemv_fused(M, mode):
    # decode GEMV with fused RMSNorm / SiLU*up prologue and residual epilogue against the fp32 reference
    from triton_distributed_b200 import ops

    torch.manual_seed(M)
    for (N, K) in [(1280, 5120), (5120, 1024), (6400, 5120), (5120, 3200), (136, 64), (1003, 264)]:
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        kw = {}
        if mode == "silu":
            x = torch.randn(M, 2 * K, device="cuda", dtype=torch.bfloat16)
            kw["silu_mul"] = True
        else:
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        if mode.startswith("norm"):
            kw["norm_weight"] = (1.0 + 0.1 * torch.randn(K, device="cuda")).to(torch.bfloat16)
            kw["eps"] = 1e-6
        res = None
        if mode == "norm_residual":
            res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        ref = ops.gemv_reference(x, w, residual=res, **kw).float()
        out = ops.gemv_fused(x, w, residual=res, **kw)
        torch.cuda.synchronize()
        err = (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
        assert err < 2e-2, f"gemv {mode} M={M} N={N} K={K}: rel err {err}"
        if res is not None:
            # in place: out aliases the residual
            buf = res.clone()
            ops.gemv_fused(x, w, out=buf, residual=buf, **kw)
            torch.cuda.synchronize()
            err = (buf.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
            assert err < 2e-2, f"gemv in-place {mode} M={M} N={N} K={K}: rel err {err}"
