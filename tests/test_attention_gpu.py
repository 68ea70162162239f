"""Attention kernels against the fp32 torch reference (single GPU)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _paged_cache(B, max_len, Hkv, D, page, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pages_per_seq = (max_len + page - 1) // page
    n_pages = B * pages_per_seq
    k = torch.randn(n_pages, page, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    v = torch.randn(n_pages, page, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    perm = torch.randperm(n_pages, device="cuda", generator=g).to(torch.int32)
    bt = perm.reshape(B, pages_per_seq).contiguous()
    return k, v, bt


@pytest.mark.parametrize("cfg", [(4, 8, 1, 128, 1, [1, 63, 64, 700]), (2, 32, 8, 128, 16, [4096, 1000]),
                                 (3, 16, 4, 64, 64, [129, 5, 2048]), (1, 40, 2, 128, 256, [3000])])
def test_decode_split_kv(cfg):
    from triton_distributed_b200.ops import attention_reference, gqa_fwd_batch_decode

    B, Hq, Hkv, D, page, lens = cfg
    k, v, bt = _paged_cache(B, max(lens), Hkv, D, page)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
    ref, ref_lse = attention_reference(q, k, v, bt, cu, kv_lens, None, False, None, 0.0, True)
    for splits in (-1, 1, 3):
        out, lse = gqa_fwd_batch_decode(q, k, v, None, None, kv_lens, bt, kv_split=splits, return_lse=True)
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(lse, ref_lse.t().contiguous(), rtol=1e-2, atol=1e-2)


def test_decode_softcap():
    from triton_distributed_b200.ops import attention_reference, gqa_fwd_batch_decode

    B, Hq, Hkv, D = 2, 8, 2, 128
    k, v, bt = _paged_cache(B, 500, Hkv, D, 32)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16) * 3
    kv_lens = torch.tensor([500, 77], dtype=torch.int32, device="cuda")
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
    ref = attention_reference(q, k, v, bt, cu, kv_lens, None, False, None, 20.0)
    out = gqa_fwd_batch_decode(q, k, v, None, None, kv_lens, bt, soft_cap=20.0)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("cfg", [(2, 8, 2, 128, 16, [100, 257], [100, 257]), (1, 4, 4, 64, 64, [64], [200]),
                                 (3, 16, 2, 128, 1, [1, 70, 130], [5, 70, 300])])
def test_prefill_causal(cfg):
    from triton_distributed_b200.ops import attention_reference, flash_attn_varlen

    B, Hq, Hkv, D, page, qlens, kvlens = cfg
    k, v, bt = _paged_cache(B, max(kvlens), Hkv, D, page, seed=1)
    T = sum(qlens)
    q = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device="cuda")
    kv_lens = torch.tensor(kvlens, dtype=torch.int32, device="cuda")
    ref, ref_lse = attention_reference(q, k, v, bt, cu, kv_lens, None, True, None, 0.0, True)
    out, lse = flash_attn_varlen(q, k, v, bt, cu, kv_lens, max(qlens), causal=True, return_lse=True)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, ref_lse, rtol=1e-2, atol=1e-2)
    # non-causal with explicit positions
    ref2 = attention_reference(q, k, v, bt, cu, kv_lens, None, False)
    out2 = flash_attn_varlen(q, k, v, bt, cu, kv_lens, max(qlens), causal=False)
    torch.testing.assert_close(out2.float(), ref2.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("impl", ["sm100", "mma"])
@pytest.mark.parametrize("cfg", [(2, 8, 2, 16, [300, 129], [300, 500], None),
                                 (1, 16, 8, 64, [1024], [1024], None),
                                 (2, 4, 1, 128, [128, 200], [384, 700], [256, 100])])
def test_prefill_both_kernels(cfg, impl):
    """The tcgen05 prefill kernel (KV packed into dense K / V^T, S and PV in TMEM) and the mma.sync kernel against the
    fp32 reference: ragged batches, paged caches with shuffled pages, explicit query positions (context-parallel chunks),
    causal and not."""
    from triton_distributed_b200.ops import attention_reference, flash_attn_varlen
    from triton_distributed_b200.ops.attention import check_attention_errors

    B, Hq, Hkv, page, qlens, kvlens, pos0 = cfg
    D = 128
    k, v, bt = _paged_cache(B, max(kvlens), Hkv, D, page, seed=2)
    q = torch.randn(sum(qlens), Hq, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device="cuda")
    kv_lens = torch.tensor(kvlens, dtype=torch.int32, device="cuda")
    qp = None if pos0 is None else torch.tensor(pos0, dtype=torch.int32, device="cuda")
    for causal in (True, False):
        ref, ref_lse = attention_reference(q, k, v, bt, cu, kv_lens, qp, causal, None, 0.0, True)
        out, lse = flash_attn_varlen(q, k, v, bt, cu, kv_lens, max(qlens), q_pos0=qp, causal=causal, return_lse=True, impl=impl)
        torch.cuda.synchronize()
        check_attention_errors()
        torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(lse, ref_lse, rtol=1e-2, atol=1e-2)
