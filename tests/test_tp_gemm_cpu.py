"""AG-GEMM and GEMM-RS through the public API on two CPU ranks (gloo), fp32, against a single-process matmul."""
import torch

from dist_utils import run_cpu_ranks


def _ag_gemm(rank, world):
    from triton_distributed_b200.ops import ag_gemm, create_ag_gemm_context

    s = 7
    As = []
    for r in range(world):
        g = torch.Generator().manual_seed(s + r)
        As.append(torch.randn(128, 256, generator=g))
    g = torch.Generator().manual_seed(100 + rank)
    B = torch.randn(256, 256, generator=g) / 16.0          # this rank's column block, stored [N_local, K]
    ctx = create_ag_gemm_context(tensor_A=As[rank], tensor_B=B, max_M=128 * world)
    out = ag_gemm(As[rank], B, ctx)
    ref = torch.cat(As, 0) @ B.t()
    assert out.shape == (128 * world, 256)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)


def _gemm_rs(rank, world):
    from triton_distributed_b200.ops import create_gemm_rs_context, gemm_rs

    s = 11
    Xs, Ws = [], []
    for r in range(world):
        g = torch.Generator().manual_seed(s + r)
        Xs.append(torch.randn(256, 128, generator=g))
        Ws.append(torch.randn(512, 128, generator=g) / (128 ** 0.5))
    ctx = create_gemm_rs_context(max_M=256, N=512, output_dtype=torch.float32)
    out = gemm_rs(Xs[rank], Ws[rank], ctx)
    full = sum(x @ w.t() for x, w in zip(Xs, Ws))
    m = 256 // world
    assert out.shape == (m, 512)
    torch.testing.assert_close(out, full[rank * m:(rank + 1) * m], rtol=1e-4, atol=1e-4)


def test_ag_gemm_two_cpu_ranks():
    run_cpu_ranks(_ag_gemm, 2)


def test_gemm_rs_two_cpu_ranks():
    run_cpu_ranks(_gemm_rs, 2)
