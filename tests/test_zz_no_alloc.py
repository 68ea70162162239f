"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the library run under another component's memory manager (a serving plug-in, a custom op of a
framework that owns the device memory, a bare C program with a fixed buffer set) and may not allocate; for them
the split-KV workspace is a fixed array inside the library.  This test drives that entry point with ctypes,
exactly as such a caller would, and checks it against the regular entry point (which takes a workspace tensor)
and against an fp32 PyTorch restatement of the attention on consecutive calls - the second one re-uses the array with the first call's leftovers in it.

The file name makes pytest collect it last, so a run that stops at the first failure has already run the rest.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from triton_distributed_b200 import _native

    _native.load(True)   # resolves the torch libraries the shared object links against
    lib = ctypes.CDLL(str(_native.lib_path()))
    lib.tdb_decode_attn_noalloc.restype = ctypes.c_int
    lib.tdb_decode_attn_noalloc.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 7 + [ctypes.c_float] * 2 + [ctypes.c_void_p]
    lib.tdb_decode_attn_noalloc_capacity.restype = ctypes.c_int64
    lib.tdb_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _case(B, Hq, Hkv, D, page, lens, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pages_per_seq = (max(lens) + page - 1) // page
    n_pages = B * pages_per_seq
    k = torch.randn(n_pages, page, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    v = torch.randn(n_pages, page, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    bt = torch.randperm(n_pages, device="cuda", generator=g).to(torch.int32).reshape(B, pages_per_seq).contiguous()
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16, generator=g)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    return q, k, v, bt, kv_lens


def _oracle(q, k, v, bt, kv_lens):
    """Plain fp32 softmax attention over the paged cache, one sequence at a time."""
    B, Hq, D = q.shape
    page, Hkv = k.shape[1], k.shape[2]
    out = torch.empty(B, Hq, D, dtype=torch.float32, device=q.device)
    for b in range(B):
        n = int(kv_lens[b])
        pages = bt[b, :(n + page - 1) // page].long()
        kk = k[pages].reshape(-1, Hkv, D)[:n].float().repeat_interleave(Hq // Hkv, dim=1)   # [n, Hq, D]
        vv = v[pages].reshape(-1, Hkv, D)[:n].float().repeat_interleave(Hq // Hkv, dim=1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), kk) / math.sqrt(D)
        out[b] = torch.einsum("hn,nhd->hd", torch.softmax(s, dim=-1), vv)
    return out


def _call(lib, q, k, v, bt, kv_lens, splits, out):
    B, Hq, D = q.shape
    return lib.tdb_decode_attn_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), bt.data_ptr(), kv_lens.data_ptr(),
                                       out.data_ptr(), B, Hq, k.shape[2], D, k.shape[1], bt.shape[1], splits,
                                       1.0 / math.sqrt(D), 0.0, torch.cuda.current_stream().cuda_stream)


def test_no_alloc_decode_matches_regular_entry_point_twice():
    from triton_distributed_b200.ops import gqa_fwd_batch_decode

    lib = _lib()
    assert lib.tdb_decode_attn_noalloc_capacity() == 1 << 20
    # two different problems back to back: the second call finds the first call's partials in the array
    for it, (B, Hq, Hkv, D, page, lens, splits) in enumerate([(4, 16, 2, 128, 16, [1000, 64, 1, 333], 4),
                                                              (2, 8, 8, 64, 32, [257, 4096], 7),
                                                              (4, 16, 2, 128, 16, [999, 65, 2, 334], 4)]):
        q, k, v, bt, kv_lens = _case(B, Hq, Hkv, D, page, lens, it)
        out = torch.empty_like(q)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        allocs_before = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        rc = _call(lib, q, k, v, bt, kv_lens, splits, out)
        assert rc == 0, lib.tdb_noalloc_last_error().decode()
        torch.cuda.synchronize()
        if it == 2:
            # same kernels as the first call, so no module load can hide behind the numbers: the call itself
            # took no device memory, neither from the driver nor from torch's allocator
            assert torch.cuda.mem_get_info()[0] == free_before
            assert torch.cuda.memory_stats().get("allocation.all.allocated", 0) == allocs_before
        ref = gqa_fwd_batch_decode(q, k, v, None, None, kv_lens, bt, kv_split=splits)
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
        # and against a plain fp32 restatement of the op, so both entry points cannot be wrong together
        torch.testing.assert_close(out.float(), _oracle(q, k, v, bt, kv_lens), rtol=2e-2, atol=2e-2)


def test_no_alloc_rejects_oversized_request():
    lib = _lib()
    q, k, v, bt, kv_lens = _case(2, 8, 8, 128, 16, [64, 64], 5)
    B, Hq, D = 4096, 64, 128   # 4096 * 64 * 8 * 129 floats: far beyond the built-in array; nothing is launched
    rc = lib.tdb_decode_attn_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), bt.data_ptr(), kv_lens.data_ptr(),
                                     q.data_ptr(), B, Hq, 8, D, 16, 4, 8, 0.1, 0.0, None)
    assert rc == -2
    assert b"exceeds" in lib.tdb_noalloc_last_error()
