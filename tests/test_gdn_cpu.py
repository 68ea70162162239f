"""Gated delta rule: the chunk-parallel form against the token-by-token recurrence (CPU, fp32)."""
import torch
import torch.nn.functional as F

from triton_distributed_b200 import ops


def _inputs(T, H, K, V, seed=0, dtype=torch.float32, device="cpu"):
    g_ = torch.Generator().manual_seed(seed)
    q = torch.randn(1, T, H, K, generator=g_)
    k = F.normalize(torch.randn(1, T, H, K, generator=g_), dim=-1)
    v = torch.randn(1, T, H, V, generator=g_)
    beta = torch.rand(1, T, H, generator=g_)
    g = F.logsigmoid(torch.rand(1, T, H, generator=g_))
    return [t.to(device=device, dtype=dtype) for t in (q, k, v)] + [g.to(device), beta.to(device=device, dtype=dtype)]


def test_chunked_matches_recurrent_varlen_with_initial_state():
    T, H, K, V = 300, 3, 32, 16
    q, k, v, g, beta = _inputs(T, H, K, V)
    cu = torch.tensor([0, 64, 171, 300], dtype=torch.int32)
    h0 = torch.randn(3, H, K, V) * 0.1
    o_r, s_r = ops.gated_delta_rule_recurrent(q, k, v, g, beta, 0.3, h0, cu)
    gc, o_c, A, s_c = ops.gated_delta_rule_chunked(q, k, v, g, beta, 0.3, h0, cu)
    assert (o_r - o_c).abs().max().item() < 1e-4
    assert (s_r - s_c).abs().max().item() < 1e-4
    assert A.shape == (1, T, H, 64) and gc.shape == (1, T, H)
    # the cumulative decay restarts at every chunk of every sequence
    assert torch.allclose(gc[0, 64], g[0, 64]) and torch.allclose(gc[0, 128], g[0, 128])


def test_public_entry_point_on_cpu():
    T, H, K, V = 130, 2, 16, 8
    q, k, v, g, beta = _inputs(T, H, K, V, seed=1)
    gc, o, A, ht = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, 0.25, None, True, None, return_A=True)
    o_r, s_r = ops.gated_delta_rule_recurrent(q, k, v, g, beta, 0.25)
    assert (o.float() - o_r).abs().max().item() < 1e-4 and (ht - s_r).abs().max().item() < 1e-4 and A is not None
    idx = ops.prepare_chunk_indices(torch.tensor([0, 70, 130]), 64)
    assert idx.tolist() == [[0, 0], [0, 1], [1, 0]]
