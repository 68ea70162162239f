"""Block-scaled fp8 operands (1 x 128 activations, 128 x 128 weights): round trip and GEMM numerics on CPU."""
import torch

from dist_utils import run_cpu_ranks
from triton_distributed_b200 import ops


def test_quantise_round_trip_and_scale_shapes():
    torch.manual_seed(0)
    x = torch.randn(37, 256) * 3
    w = torch.randn(200, 256) * 0.02
    xq, xs = ops.quantize_act_1x128(x)
    wq, ws = ops.quantize_weight_128x128(w)
    assert xq.dtype == torch.float8_e4m3fn and xs.shape == (37, 2) and ws.shape == (2, 2) and wq.shape == w.shape
    # e4m3 keeps three mantissa bits: relative error of a block is bounded by 2^-4 of its largest value
    assert (ops.dequantize_act_1x128(xq, xs, torch.float32) - x).abs().max() <= x.abs().max() / 16 + 1e-6
    assert (ops.dequantize_weight_128x128(wq, ws, torch.float32) - w).abs().max() <= w.abs().max() / 16 + 1e-6


def test_blockscaled_gemm_matches_its_reference_and_the_unquantised_product():
    torch.manual_seed(1)
    x = torch.randn(64, 512)
    w = torch.randn(192, 512) * 0.05
    xq, xs = ops.quantize_act_1x128(x)
    wq, ws = ops.quantize_weight_128x128(w)
    ref = ops.gemm_fp8_blockscaled_reference(xq, xs, wq, ws)
    out = ops.gemm_fp8_blockscaled(xq, xs, wq, ws, out_dtype=torch.float32)
    assert (out - ref).abs().max().item() < 1e-3 * ref.abs().max().item()
    exact = x @ w.t()
    assert (ref - exact).abs().max().item() < 0.06 * exact.abs().max().item()


def _ag_fp8(rank, world):
    torch.manual_seed(7)
    x = torch.randn(world * 16, 256)
    w = torch.randn(world * 24, 256) * 0.05
    xq, xs = ops.quantize_act_1x128(x[rank * 16:(rank + 1) * 16])
    wq, ws = ops.quantize_weight_128x128(w[rank * 24:(rank + 1) * 24])
    out = ops.ag_gemm_fp8(xq, xs, wq, ws)
    exact = x @ w[rank * 24:(rank + 1) * 24].t()
    assert out.shape == exact.shape
    assert (out.float() - exact).abs().max().item() < 0.08 * exact.abs().max().item()


def test_ag_gemm_fp8_two_ranks():
    run_cpu_ranks(_ag_fp8, 2)
