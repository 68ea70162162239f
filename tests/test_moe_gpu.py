"""MoE kernels (router, sort, grouped GEMM, top-k reduce) against torch references on one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import triton_distributed_b200 as tdb

    tdb.initialize_distributed(seed=0)
    return tdb.get_runtime()


@pytest.mark.parametrize("cfg", [(37, 8, 2), (512, 128, 8), (1000, 256, 8), (5, 64, 6)])
def test_topk_router(cfg):
    from triton_distributed_b200.ops import topk_router, topk_router_reference

    T, E, k = cfg
    logits = torch.randn(T, E, device="cuda")
    ids, w = topk_router(logits, k, True)
    rids, rw = topk_router_reference(logits, k, True)
    assert torch.equal(ids.sort(-1).values, rids.sort(-1).values)
    torch.testing.assert_close(w.sum(-1), torch.ones(T, device="cuda"), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(w.gather(1, ids.long().argsort(-1)), rw.gather(1, rids.long().argsort(-1)), rtol=1e-4, atol=1e-5)


def test_align_sort_invariants():
    from triton_distributed_b200.ops import sort_topk_ids_align_block_size

    T, E, k = 777, 32, 4
    ids = torch.randint(0, E + 1, (T, k), device="cuda", dtype=torch.int32)   # E = dropped
    s = sort_topk_ids_align_block_size(ids, E)
    flat = ids.reshape(-1)
    total, tiles = s.meta.tolist()
    assert total % 128 == 0 and tiles == total // 128
    counts = torch.bincount(flat[flat < E].long(), minlength=E)
    assert torch.equal(s.counts.long(), counts)
    sid = s.sorted_ids[:total]
    real = sid[sid >= 0].long()
    assert real.numel() == int((flat < E).sum()) and real.unique().numel() == real.numel()
    te = s.tile_expert[:tiles].long()
    for t in range(tiles):
        rows = sid[t * 128:(t + 1) * 128]
        rows = rows[rows >= 0].long()
        assert (flat[rows] == te[t]).all()
    assert (s.tile_expert[tiles:] == -1).all()
    pos = s.pos_of[:T * k].long()
    ok = flat < E
    assert torch.equal(s.sorted_ids[pos[ok]].long(), torch.nonzero(ok).squeeze(1))
    assert (pos[~ok] == -1).all()


@pytest.mark.parametrize("cfg", [(300, 16, 2, 256, 512), (2048, 32, 8, 1024, 768), (64, 8, 8, 7168, 256)])
def test_moe_mlp_single_rank(rt, cfg):
    from triton_distributed_b200 import ops

    T, E, k, H, I = cfg
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w1 = (torch.randn(E, 2 * I, H, device="cuda") * 0.03).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, device="cuda") * 0.03).to(torch.bfloat16)
    ids, tw = ops.topk_router(torch.randn(T, E, device="cuda"), k)
    agc = ops.create_ag_group_gemm_context(T, 2 * I, H, E, k)
    rsc = ops.create_moe_rs_context(max_token_num=T, hidden_dim=H, num_experts=E, topk=k)
    # API layout: (token, slot) order
    h = ops.ag_group_gemm(x, w1, agc, ids)
    ref_h = ops.group_gemm_reference(x, w1, ids)
    torch.testing.assert_close(h.float(), ref_h.float(), rtol=3e-2, atol=3e-2)
    act = ops.silu_mul(h)
    out = ops.run_moe_reduce_rs(act, w2, ids, tw, rsc)
    ref = ops.moe_reduce_reference(act, w2, ids, tw)
    torch.testing.assert_close(out.float(), ref.float(), rtol=3e-2, atol=3e-2)
    # fused layout: stay expert-sorted between the two grouped GEMMs
    hs, srt = ops.ag_group_gemm(x, w1, agc, ids, sorted_output=True)
    out2 = ops.run_moe_reduce_rs(ops.silu_mul(hs), w2, ids, tw, rsc, sort=srt)
    torch.testing.assert_close(out2.float(), ref.float(), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("cfg", [(512, 16, 4, 4, 1), (1024, 64, 8, 8, 3), (96, 8, 2, 2, 0)])
def test_staged_sort_and_device_tile_schedule(rt, cfg):
    """The staged sort keeps every expert's rows together, ordered by ring distance; the device-side tile schedule
    equals the host C++ reference on the same layout."""
    from triton_distributed_b200 import ops

    T, E, k, W, rank = cfg
    ids, _ = ops.topk_router(torch.randn(T, E, device="cuda"), k)
    tpr = T // W
    srt = ops.sort_topk_ids_staged(ids, E, tpr, rank, W)
    flat = ids.reshape(-1).long()
    sid = srt.sorted_ids.long()
    offs = srt.offsets.long().tolist()
    cnt = srt.counts.long().tolist()
    assert sorted(sid[sid >= 0].tolist()) == list(range(T * k))
    for e in range(E):
        rows = sid[offs[e]:offs[e] + cnt[e]]
        assert (flat[rows] == e).all() and (sid[offs[e] + cnt[e]:offs[e + 1]] == -1).all()
        stage = ((rows // k) // tpr - rank) % W
        assert (stage[1:] >= stage[:-1]).all(), "rows of an expert must be ordered by arrival stage"
    assert torch.equal(srt.sorted_ids[srt.pos_of.long()].long(), torch.arange(T * k, device="cuda"))
    order, stage = ops.tile_schedule(srt, tpr, rank, W)
    ref_order, ref_stage = ops.tile_arrival_order(srt, tpr, rank, W)
    assert torch.equal(stage.cpu(), ref_stage) and torch.equal(order.cpu(), ref_order)


@pytest.mark.parametrize("cfg", [(300, 16, 2, 256, 512), (1024, 8, 4, 7168, 256), (77, 4, 1, 64, 136)])
def test_group_gemm_with_in_kernel_gather(rt, cfg):
    from triton_distributed_b200 import ops

    T, E, k, H, N = cfg
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(E, N, H, device="cuda") * 0.03).to(torch.bfloat16)
    ids, tw = ops.topk_router(torch.randn(T, E, device="cuda"), k)
    srt = ops.sort_topk_ids_align_block_size(ids, E)
    ref = ops.group_gemm_reference(x, w, ids).float()                       # (token, slot) order
    y = ops.group_gemm_gather(x, w, srt, a_row_div=k, scatter_out=True)
    torch.testing.assert_close(y.float(), ref, rtol=3e-2, atol=3e-2)
    ys = ops.group_gemm_gather(x, w, srt, a_row_div=k, scatter_out=False, row_weight=tw)
    sid = srt.sorted_ids.long()
    ok = sid >= 0
    torch.testing.assert_close(ys[ok].float(), ref[sid[ok]] * tw.reshape(-1)[sid[ok]].unsqueeze(-1), rtol=3e-2, atol=3e-2)
    assert (ys[: int(srt.meta[0])][~ok[: int(srt.meta[0])]] == 0).all()     # padding rows of visited tiles are zeros
