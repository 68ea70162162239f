"""Memory-bound kernels against their torch fp32 references (single GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_rmsnorm_and_fused_residual():
    from triton_distributed_b200.ops import rmsnorm
    from triton_distributed_b200.ops.elementwise import rmsnorm_reference

    for T, H in [(7, 5120), (64, 1024), (3, 128)]:
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(H, device="cuda", dtype=torch.bfloat16)
        torch.testing.assert_close(rmsnorm(x, w, 1e-6).float(), rmsnorm_reference(x, w, 1e-6).float(), rtol=2e-2, atol=2e-2)
        res = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        res2 = res.clone()
        y = rmsnorm(x, w, 1e-6, residual=res2)
        s = (x.float() + res.float()).to(torch.bfloat16)
        torch.testing.assert_close(res2.float(), s.float(), rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(y.float(), rmsnorm_reference(s, w, 1e-6).float(), rtol=2e-2, atol=2e-2)


def test_silu_mul_and_add():
    from triton_distributed_b200.ops import residual_add, silu_mul
    from triton_distributed_b200.ops.elementwise import silu_mul_reference

    x = torch.randn(33, 2 * 3200, device="cuda", dtype=torch.bfloat16)
    torch.testing.assert_close(silu_mul(x).float(), silu_mul_reference(x).float(), rtol=2e-2, atol=2e-2)
    a = torch.randn(17, 5120, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(17, 5120, device="cuda", dtype=torch.bfloat16)
    torch.testing.assert_close(residual_add(a, b).float(), (a.float() + b.float()), rtol=1e-2, atol=1e-2)


def test_qk_norm_rope_kv():
    from triton_distributed_b200.ops import qk_norm_rope_kv
    from triton_distributed_b200.ops.elementwise import qk_norm_rope_kv_reference

    T, Hq, Hkv, D = 9, 8, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    qw = torch.randn(D, device="cuda", dtype=torch.bfloat16)
    kw = torch.randn(D, device="cuda", dtype=torch.bfloat16)
    pos = torch.tensor([0, 1, 5, 100, 4095, 7, 8, 9, 33000], device="cuda")
    slots = torch.tensor([3, 0, 8, 1, 2, -1, 5, 6, 7], device="cuda")
    kc = torch.zeros(16, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc2, vc2 = kc.clone(), vc.clone()
    q = qk_norm_rope_kv(qkv, qw, kw, pos, slots, kc, vc, Hq, Hkv, D, 1e-6, 1e6)
    q_ref = qk_norm_rope_kv_reference(qkv, qw, kw, pos, slots, kc2, vc2, Hq, Hkv, D, 1e-6, 1e6)
    torch.testing.assert_close(q.float(), q_ref.float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(kc.float(), kc2.float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(vc.float(), vc2.float(), rtol=0, atol=0)


def test_embedding_argmax_abs_sum():
    from triton_distributed_b200.ops import abs_sum, argmax, embedding

    table = torch.randn(1000, 256, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 1000, (4, 5), device="cuda")
    assert torch.equal(embedding(ids, table), table[ids])
    logits = torch.randn(6, 151936, device="cuda", dtype=torch.float32)
    assert torch.equal(argmax(logits), logits.argmax(-1))
    x = torch.randn(1000, 512, device="cuda", dtype=torch.bfloat16)
    torch.testing.assert_close(abs_sum(x)[0], x.float().abs().sum(), rtol=1e-3, atol=1e-1)
