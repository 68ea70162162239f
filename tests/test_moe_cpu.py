"""MoE layers on CPU ranks (gloo, fp32): TP-MoE sharded forward and EP dispatch/combine against dense math."""
import torch

from dist_utils import run_cpu_ranks


def _tp_moe(rank, world):
    from triton_distributed_b200.parallel import TP_MoE
    from triton_distributed_b200.runtime import get_runtime

    rt = get_runtime()
    g = torch.Generator().manual_seed(5)
    T, H, I, E, k = 16, 32, 64, 8, 2
    router, gate, up, down = (torch.randn(E, H, generator=g), torch.randn(E, I, H, generator=g) * 0.1,
                              torch.randn(E, I, H, generator=g) * 0.1, torch.randn(E, H, I, generator=g) * 0.1)
    x = torch.randn(T, H, generator=g)
    moe = TP_MoE(rank, world, rt.group)
    moe._init_parameters(router, gate, up, down, k, True, device="cpu")
    moe._init_ctx(T)
    ref = moe.torch_fwd(x)
    tl = T // world
    out = moe.dist_triton_fwd(x[rank * tl:(rank + 1) * tl])
    torch.testing.assert_close(out, ref[rank * tl:(rank + 1) * tl], rtol=1e-4, atol=1e-4)
    out_ar = moe.dist_triton_AR_fwd(x)
    torch.testing.assert_close(out_ar, ref, rtol=1e-4, atol=1e-4)
    # dense oracle: every expert on every token, masked by the routing
    p = torch.softmax(x @ router.t(), -1)
    w, ids = torch.topk(p, k, -1)
    w = w / w.sum(-1, keepdim=True)
    dense = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            h = torch.nn.functional.silu(gate[e] @ x[t]) * (up[e] @ x[t])
            dense[t] += w[t, j] * (down[e] @ h)
    torch.testing.assert_close(ref, dense, rtol=1e-4, atol=1e-4)


def _ep(rank, world):
    from triton_distributed_b200 import ops

    g = torch.Generator().manual_seed(9 + rank)
    T, H, E, k = 12, 128, 8, 3
    x = torch.randn(T, H, generator=g)
    ids = torch.stack([torch.randperm(E + 1, generator=g)[:k] for _ in range(T)]).to(torch.int32)   # E = dropped
    w = torch.rand(T, k, generator=g)
    ctx = ops.create_all_to_all_context(T, H, num_tot_experts=E, topk=k, quant=False)
    recv = ops.ep_dispatch(ctx, x, ids)
    # "expert": multiply by (global expert id + 1)
    epr = E // world
    y = torch.zeros_like(recv.x_sorted)
    for t, e in enumerate(recv.sort.tile_expert.tolist()):
        if e >= 0:
            y[t * 128:(t + 1) * 128] = recv.x_sorted[t * 128:(t + 1) * 128] * float(rank * epr + e + 1)
    out = ops.ep_combine(ctx, y, recv, w)
    ref = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            if e < E:
                ref[t] += w[t, j] * x[t] * (e + 1)
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)


def test_tp_moe_two_cpu_ranks():
    run_cpu_ranks(_tp_moe, 2)


def test_ep_dispatch_combine_two_cpu_ranks():
    run_cpu_ranks(_ep, 2)


def test_fp8_quant_reference_roundtrip():
    from triton_distributed_b200.ops import fp8_dequant, fp8_quant

    x = (torch.randn(5, 256) * 3).to(torch.bfloat16)
    q, s = fp8_quant(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (5, 2)
    back = fp8_dequant(q, s)
    assert (back.float() - x.float()).abs().max() <= 0.07 * x.float().abs().max()


def test_tile_arrival_order_matches_a_python_oracle():
    # C++ host reference of the AG -> grouped-GEMM tile order against a direct restatement
    import torch

    from triton_distributed_b200 import ops

    torch.manual_seed(3)
    W, tpr, k, E, blk = 4, 24, 2, 5, 16
    ids = torch.randint(0, E, (W * tpr, k))
    srt = ops.sort_topk_ids_align_block_size(ids, E, blk)
    for rank in range(W):
        order, stage = ops.tile_arrival_order(srt, tpr, rank, W, blk)
        sid = srt.sorted_ids.tolist()
        tiles = (len(sid) + blk - 1) // blk
        exp_stage = []
        for t in range(tiles):
            d = [((i // k) // tpr - rank) % W for i in sid[t * blk:(t + 1) * blk] if i >= 0]
            exp_stage.append(max(d) if d else -1)
        assert stage.tolist() == exp_stage
        o = order.tolist()
        assert sorted(o) == list(range(tiles))
        keys = [W if exp_stage[t] < 0 else exp_stage[t] for t in o]
        assert keys == sorted(keys), "tiles must be visited by arrival stage"
        for a, b in zip(o, o[1:]):
            if exp_stage[a] == exp_stage[b]:
                assert a < b, "expert order is kept inside a stage"
