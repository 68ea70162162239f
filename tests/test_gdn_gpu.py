"""Gated delta rule CUDA kernel against the fp32 token recurrence."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,cu", [(257, None), (400, [0, 90, 91, 400])])
def test_gdn_kernel_matches_recurrence(T, cu):
    from test_gdn_cpu import _inputs
    from triton_distributed_b200 import ops

    H, K, V = 4, 128, 128
    q, k, v, g, beta = _inputs(T, H, K, V, seed=3, dtype=torch.bfloat16, device="cuda")
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32, device="cuda")
    n = 1 if cu is None else len(cu) - 1
    h0 = (torch.randn(n, H, K, V, device="cuda") * 0.05)
    scale = K ** -0.5
    gc, o, A, ht = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, True, cu_t)
    o_r, s_r = ops.gated_delta_rule_recurrent(q, k, v, g, beta, scale, h0, cu_t)
    torch.cuda.synchronize()
    assert A is None and gc.shape == (1, T, H)
    err_o = (o.float() - o_r).abs().max().item() / (o_r.abs().max().item() + 1e-6)
    err_s = (ht - s_r).abs().max().item() / (s_r.abs().max().item() + 1e-6)
    assert err_o < 2e-2 and err_s < 1e-3, (err_o, err_s)
