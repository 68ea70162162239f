"""Gated delta rule CUDA kernel against the fp32 token recurrence."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("impl", ["chunk", "recurrent"])
@pytest.mark.parametrize("T,cu", [(257, None), (400, [0, 90, 91, 400])])
def test_gdn_kernel_matches_recurrence(T, cu, impl):
    from test_gdn_cpu import _inputs
    from triton_distributed_b200 import ops

    H, K, V = 4, 128, 128
    q, k, v, g, beta = _inputs(T, H, K, V, seed=3, dtype=torch.bfloat16, device="cuda")
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32, device="cuda")
    n = 1 if cu is None else len(cu) - 1
    h0 = (torch.randn(n, H, K, V, device="cuda") * 0.05)
    scale = K ** -0.5
    gc, o, A, ht = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, True, cu_t, impl=impl)
    o_r, s_r = ops.gated_delta_rule_recurrent(q, k, v, g, beta, scale, h0, cu_t)
    torch.cuda.synchronize()
    assert A is None and gc.shape == (1, T, H)
    err_o = (o.float() - o_r).abs().max().item() / (o_r.abs().max().item() + 1e-6)
    err_s = (ht - s_r).abs().max().item() / (s_r.abs().max().item() + 1e-6)
    # the chunked form feeds bf16 copies of the state and of the WY factors to the tensor cores (as the reference does)
    assert err_o < 2e-2 and err_s < (2e-2 if impl == "chunk" else 1e-3), (impl, err_o, err_s)


@pytest.mark.parametrize("V", [64, 256])
def test_gdn_chunk_kernels_match_torch_chunked_form(V):
    """Every output of the chunk-parallel kernels (chunk-local cumulative decay, WY matrices A, outputs, final state)
    against the same algorithm in fp32 PyTorch, with ragged sequences (tail chunks of 1 and 27 tokens)."""
    from test_gdn_cpu import _inputs
    from triton_distributed_b200 import ops
    from triton_distributed_b200.ops.gdn import gated_delta_rule_chunked

    T, H, K = 64 * 3 + 1 + 91, 3, 128
    cu = torch.tensor([0, 193, 284], dtype=torch.int32, device="cuda")
    q, k, v, g, beta = _inputs(T, H, K, V, seed=5, dtype=torch.bfloat16, device="cuda")
    scale = K ** -0.5
    gc, o, A, ht = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, None, True, cu, return_A=True, impl="chunk")
    gc_r, o_r, A_r, ht_r = gated_delta_rule_chunked(q, k, v, g, beta, scale, None, cu)
    torch.cuda.synchronize()
    torch.testing.assert_close(gc, gc_r, rtol=1e-4, atol=1e-4)
    assert (A - A_r).abs().max().item() < 2e-2 * max(1.0, A_r.abs().max().item())
    assert (o.float() - o_r).abs().max().item() < 2e-2 * (o_r.abs().max().item() + 1e-6)
    assert (ht - ht_r).abs().max().item() < 2e-2 * (ht_r.abs().max().item() + 1e-6)
