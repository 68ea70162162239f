"""Sequence-parallel attention, Ulysses all-to-all and the pipeline transport on CPU ranks (gloo): the host-side
logic (zig-zag chunking, block tables, row orderings, buffer hand-over) against single-process references."""
import math

import torch

from dist_utils import run_cpu_ranks


def _attn_ref(q, k, v, causal=True):
    # q [S, Hq, D], k/v [S, Hkv, D]
    Hq, Hkv = q.shape[1], k.shape[1]
    k = k.repeat_interleave(Hq // Hkv, dim=1)
    v = v.repeat_interleave(Hq // Hkv, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), k.float()) / math.sqrt(q.shape[-1])
    if causal:
        S = q.shape[0]
        s = s.masked_fill(~torch.ones(S, S).tril().bool(), float("-inf"))
    return torch.einsum("hqk,khd->qhd", s.softmax(-1), v.float())


def _sp_attention(rank, world):
    import triton_distributed_b200 as tdb
    from triton_distributed_b200.parallel import (create_sp_ag_attention_context_intra_node, fused_sp_ag_attn_intra_node)

    tdb.initialize_distributed(seed=0)
    B, S, Hq, Hkv, D = 2, 64, 4, 2, 16
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, S, Hq, D, generator=g)
    k = torch.randn(B, S, Hkv, D, generator=g)
    v = torch.randn(B, S, Hkv, D, generator=g)
    for zig in (True, False):
        n_chunks = 2 * world if zig else world
        c = S // n_chunks
        mine = [rank, 2 * world - 1 - rank] if zig else [rank]

        def shard(x):
            return torch.cat([x[b, ch * c:(ch + 1) * c] for b in range(B) for ch in mine], 0)

        ctx = create_sp_ag_attention_context_intra_node(B, Hq, Hkv, S, D, input_dtype=torch.float32)
        local = len(mine) * c
        cu_q = torch.arange(0, (B + 1) * local, local, dtype=torch.int32)
        cu_k = torch.arange(0, (B + 1) * S, S, dtype=torch.int32)
        out = fused_sp_ag_attn_intra_node(ctx, shard(q), shard(k), shard(v), None, cu_q, cu_k, local, S,
                                          is_causal=True, enable_zig_zag=zig)
        ref = torch.cat([_attn_ref(q[b], k[b], v[b])[ch * c:(ch + 1) * c] for b in range(B) for ch in mine], 0)
        assert (out.float() - ref).abs().max().item() < 1e-4, f"sp attention zig_zag={zig}"
    # sequences of different lengths in one packed batch (page size = gcd of the chunk lengths)
    lens = [96, 32, 64]
    qs = [torch.randn(n, Hq, D, generator=g) for n in lens]
    ks = [torch.randn(n, Hkv, D, generator=g) for n in lens]
    vs = [torch.randn(n, Hkv, D, generator=g) for n in lens]
    for zig in (True, False):
        n_chunks = 2 * world if zig else world
        mine = [rank, 2 * world - 1 - rank] if zig else [rank]

        def shard(xs):
            return torch.cat([x[ch * (n // n_chunks):(ch + 1) * (n // n_chunks)] for x, n in zip(xs, lens) for ch in mine], 0)

        ctx = create_sp_ag_attention_context_intra_node(1, Hq, Hkv, sum(lens), D, input_dtype=torch.float32)
        loc = [len(mine) * (n // n_chunks) for n in lens]
        cu_q = torch.tensor([0] + list(torch.tensor(loc).cumsum(0)), dtype=torch.int32)
        cu_k = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
        out = fused_sp_ag_attn_intra_node(ctx, shard(qs), shard(ks), shard(vs), None, cu_q, cu_k, max(loc), max(lens),
                                          is_causal=True, enable_zig_zag=zig)
        ref = torch.cat([_attn_ref(qs[b], ks[b], vs[b])[ch * (n // n_chunks):(ch + 1) * (n // n_chunks)]
                         for b, n in enumerate(lens) for ch in mine], 0)
        assert (out.float() - ref).abs().max().item() < 1e-4, f"sp attention var-len zig_zag={zig}"
    tdb.finalize_distributed()


def test_sp_allgather_attention_two_ranks():
    run_cpu_ranks(_sp_attention, 2)


def _ulysses(rank, world):
    import triton_distributed_b200 as tdb
    from triton_distributed_b200.parallel import SpUlysessOAll2AllGemmKernel, SpUlysessQKVGemmAll2AllKernel

    tdb.initialize_distributed(seed=0)
    S, H, heads, D = 16, 32, 4, 8
    s_local = S // world
    g = torch.Generator().manual_seed(11)
    x = torch.randn(S, H, generator=g)
    w_qkv = torch.randn(3 * heads * D, H, generator=g) * 0.1
    w_o = torch.randn(H, heads * D, generator=g) * 0.1
    pre = SpUlysessQKVGemmAll2AllKernel(num_head=heads, head_dim=D, max_seqlen=S, output_dtype=torch.float32)
    post = SpUlysessOAll2AllGemmKernel(num_head=heads, head_dim=D, max_seqlen=S, output_dtype=torch.float32)
    qkv = pre.forward(x[rank * s_local:(rank + 1) * s_local], w_qkv)          # [S, 3, heads / W, D]
    hl = heads // world
    ref_qkv = (x @ w_qkv.t()).reshape(S, 3, heads, D)[:, :, rank * hl:(rank + 1) * hl]
    assert (qkv - ref_qkv).abs().max().item() < 1e-4, "ulysses pre-attention all-to-all"
    # a stand-in for attention that keeps the layout: use q as the attention output
    attn = qkv[:, 0].contiguous()                                              # [S, heads / W, D]
    out = post.forward(attn, w_o)                                              # [s_local, H]
    full_attn = (x @ w_qkv.t()).reshape(S, 3, heads, D)[:, 0].reshape(S, heads * D)
    ref_out = (full_attn @ w_o.t())[rank * s_local:(rank + 1) * s_local]
    assert (out - ref_out).abs().max().item() < 1e-3, "ulysses post-attention all-to-all + O projection"
    tdb.finalize_distributed()


def test_ulysses_two_ranks():
    run_cpu_ranks(_ulysses, 2)


def _pp(rank, world):
    import triton_distributed_b200 as tdb
    from triton_distributed_b200.parallel import CommOp

    tdb.initialize_distributed(seed=0)
    op = CommOp(max_tokens=8, hidden=4, num_buffers=2, dtype=torch.float32)
    for step in range(4):
        buf = step % 2
        if rank == 0:
            op.send(torch.full((5, 4), float(step)), 1, buf)
            op.wait_signal(buf)
        else:
            view = op.read(0, 5, buf)
            op.wait_signal(buf)
            assert torch.all(view == step), (step, view)
            op.set_signal(buf)
    tdb.finalize_distributed()


def test_pp_transport_two_ranks():
    run_cpu_ranks(_pp, 2)
