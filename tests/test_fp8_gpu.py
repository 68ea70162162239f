"""Native block-scaled fp8 GEMM (tcgen05 kind::f8f6f4 with per-128-K promotion) against the fp32 PyTorch restatement
of the same accumulation order, on one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed):
    from triton_distributed_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(seed)
    # rows and weight blocks with very different magnitudes: wrong or swapped scales cannot hide
    x = torch.randn(M, K, device="cuda", generator=g) * (0.25 + 4.0 * torch.rand(M, 1, device="cuda", generator=g))
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05 * (0.5 + torch.rand(N, 1, device="cuda", generator=g))
    w[:, : K // 2] *= 3.0
    xq, xs = ops.quantize_act_1x128(x.to(torch.bfloat16))
    wq, ws = ops.quantize_weight_128x128(w)
    return x, w, xq, xs, wq, ws


def _reference(xq, xs, wq, ws, rows=512):
    from triton_distributed_b200 import ops

    outs = [ops.gemm_fp8_blockscaled_reference(xq[i:i + rows], xs[i:i + rows], wq, ws) for i in range(0, xq.shape[0], rows)]
    return torch.cat(outs, 0)


@pytest.mark.parametrize("shape", [(256, 256, 128), (256, 512, 1024), (512, 768, 2048), (300, 520, 384), (1, 136, 256),
                                   (1000, 264, 512), (1024, 2048, 8192), (4096, 2304, 512)])
def test_gemm_fp8_blockscaled_native(shape):
    from triton_distributed_b200 import ops

    M, N, K = shape
    x, w, xq, xs, wq, ws = _operands(M, N, K, seed=M + N)
    out = ops.gemm_fp8_blockscaled(xq, xs, wq, ws)
    torch.cuda.synchronize()
    assert out.dtype == torch.bfloat16 and out.shape == (M, N)
    ref = _reference(xq, xs, wq, ws)
    # same operands, same block order: only fp32 summation order inside a block and the bf16 output rounding differ
    torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().mean().item() + 1e-3)
    # and the quantised product tracks the unquantised one (e4m3: ~2^-4 relative per element, averaged over K)
    exact = x.to(torch.bfloat16).float() @ w.float().t()
    assert (out.float() - exact).abs().max().item() < 0.08 * exact.abs().max().item()


def test_gemm_fp8_twice_and_stall_counters():
    from triton_distributed_b200 import ops

    x, w, xq, xs, wq, ws = _operands(2048, 2560, 1024, seed=3)
    ref = _reference(xq, xs, wq, ws)
    st = ops.new_stall_counters("cuda")
    for _ in range(2):
        out = ops.gemm_fp8_blockscaled(xq, xs, wq, ws, stats=st)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().mean().item() + 1e-3)
    assert ops.summarize_stall_counters(st)["ctas"] > 0


def test_fp8_quantiser_kernel_matches_torch():
    from triton_distributed_b200 import ops
    from triton_distributed_b200.ops import fp8

    x = (torch.randn(333, 1024, device="cuda") * 3).to(torch.bfloat16)
    q, s = ops.quantize_act_1x128(x)
    xb = x.float().reshape(333, 8, 128)
    s_ref = xb.abs().amax(-1).clamp_min(1e-10) / fp8.FP8_MAX
    torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
    deq = ops.dequantize_act_1x128(q, s, torch.float32)
    assert (deq - x.float()).abs().max().item() <= x.float().abs().max().item() / 16 + 1e-6
