"""Multi-GPU MoE checks (torchrun): TP-MoE modes against the torch path, EP dispatch/combine (both layouts, with and
without fp8) against a dense oracle, all_to_all_single_2d against NCCL."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import triton_distributed_b200 as tdb  # noqa: E402
from triton_distributed_b200 import ops  # noqa: E402
from triton_distributed_b200.parallel import EP_MoE, TP_MoE  # noqa: E402


def log(rt, *a):
    if rt.rank == 0:
        print(*a, flush=True)


def check_tp_moe(rt):
    W = rt.world_size
    T, H, I, E, k = 64 * W, 512, 256 * W, 16, 4
    g = torch.Generator(device="cuda").manual_seed(11)
    mk = lambda *s: (torch.randn(*s, device="cuda", generator=g) * 0.05).to(torch.bfloat16)   # noqa: E731
    router, gate, up, down = mk(E, H), mk(E, I, H), mk(E, I, H), mk(E, H, I)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    moe = TP_MoE(rt.rank, W, rt.group)
    moe._init_parameters(router, gate, up, down, k)
    moe._init_ctx(T)
    ref = moe.torch_fwd(x)
    tl = T // W
    for it in range(3):
        out = moe.dist_triton_fwd(x[rt.rank * tl:(rt.rank + 1) * tl].contiguous())
        torch.cuda.synchronize()
        rt.check_status()
        err = (out.float() - ref[rt.rank * tl:(rt.rank + 1) * tl].float()).abs().max().item()
        assert err < 0.05 * ref.float().abs().max().item() + 0.02, f"TP-MoE ag_rs err {err}"
        out2 = moe.dist_triton_AR_fwd(x)
        torch.cuda.synchronize()
        rt.check_status()
        err2 = (out2.float() - ref.float()).abs().max().item()
        assert err2 < 0.05 * ref.float().abs().max().item() + 0.02, f"TP-MoE AR err {err2}"
    log(rt, "OK TP-MoE (AG+grouped GEMM, grouped GEMM+RS / AR)")


def check_tp_moe_ops(rt):
    """The two fused launches against their fp32 restatements over NCCL-gathered inputs, with several chunk counts,
    ragged token counts per expert and back-to-back calls (epoch parity of the workspaces, flags and counters)."""
    W = rt.world_size
    for (tl, H, I, E, k) in [(64, 512, 256, 16, 4), (200, 1024, 384, 8, 2), (256, 768, 128, 32, 8)]:
        T = tl * W
        g = torch.Generator(device="cuda").manual_seed(31)                      # same weights / routing on every rank
        w1 = (torch.randn(E, I, H, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
        w2 = (torch.randn(E, H, I, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
        agc = ops.create_ag_group_gemm_context(T, I, H, E, k)
        rsc = ops.create_moe_rs_context(max_token_num=T, hidden_dim=H, num_experts=E, topk=k)
        for it in range(4):
            ids, tw = ops.topk_router(torch.randn(T, E, device="cuda", generator=g), k)
            x_full = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
            x = x_full[rt.rank * tl:(rt.rank + 1) * tl].contiguous()
            # all-gather -> grouped GEMM, (token, slot) order and sorted layout
            ref_h = ops.group_gemm_reference(x_full, w1, ids).float()
            h = ops.ag_group_gemm(x, w1, agc, ids)
            torch.cuda.synchronize()
            rt.check_status()
            torch.testing.assert_close(h.float(), ref_h, rtol=3e-2, atol=3e-2)
            hs, srt = ops.ag_group_gemm(x, w1, agc, ids, sorted_output=True)
            torch.cuda.synchronize()
            rt.check_status()
            sid = srt.sorted_ids.long()
            torch.testing.assert_close(hs[sid >= 0].float(), ref_h[sid[sid >= 0]], rtol=3e-2, atol=3e-2)
            # grouped GEMM -> top-k reduce -> reduce-scatter / all-reduce: every rank holds its own slice of the
            # intermediate dimension, so the partial products differ per rank and the sum over ranks is the result
            act = (torch.randn(T * k, I, device="cuda") * (0.2 + 0.1 * rt.rank)).to(torch.bfloat16)
            part = ops.moe_reduce_reference(act, w2, ids, tw).float()
            dist.all_reduce(part, group=rt.group)
            n_chunks = (1, 2, 4, 3)[it]
            out = ops.run_moe_reduce_rs(act, w2, ids, tw, rsc, n_chunks=n_chunks)
            torch.cuda.synchronize()
            rt.check_status()
            torch.testing.assert_close(out.float(), part[rt.rank * tl:(rt.rank + 1) * tl], rtol=5e-2, atol=5e-2)
            out_ar = ops.run_moe_reduce_ar(act, w2, ids, tw, rsc, n_chunks=n_chunks)
            torch.cuda.synchronize()
            rt.check_status()
            torch.testing.assert_close(out_ar.float(), part, rtol=5e-2, atol=5e-2)
        agc.finalize()
        rsc.finalize()
    log(rt, "OK fused TP-MoE ops (AG -> grouped GEMM, grouped GEMM -> top-k reduce -> RS / AR)")


def check_ep(rt):
    W = rt.world_size
    H, I, E, k, T = 1024, 256, 8 * W, 4, 96
    for layout in ("ll", "packed"):
        for quant in (False, True):
            moe = EP_MoE(H, I, E, k, T, quant=quant, layout=layout, seed=21)
            g = torch.Generator(device="cuda").manual_seed(100 + rt.rank)
            for it in range(3):
                x = torch.randn(T - 7 * it, H, device="cuda", generator=g).to(torch.bfloat16)
                out = moe(x)
                torch.cuda.synchronize()
                rt.check_status()
                # oracle: rebuild all experts from the same generator stream and run them densely on the local tokens
                g2 = torch.Generator(device="cuda").manual_seed(21)
                router = (torch.randn(E, H, device="cuda", generator=g2) * 0.02).to(torch.bfloat16)
                ids, w = moe.route(x)
                ref = torch.zeros(x.shape[0], H, device="cuda")
                xin = x
                if quant:
                    q, s = ops.fp8_quant(x)
                    xin = ops.fp8_dequant(q, s)
                for e in range(E):
                    a = (torch.randn(2 * I, H, device="cuda", generator=g2) * 0.02).to(torch.bfloat16)
                    b = (torch.randn(H, I, device="cuda", generator=g2) * 0.02).to(torch.bfloat16)
                    sel = (ids == e)
                    tok = sel.any(-1).nonzero(as_tuple=True)[0]
                    if tok.numel() == 0:
                        continue
                    h = xin[tok].float() @ a.float().t()
                    h = (torch.nn.functional.silu(h[:, :I]) * h[:, I:]).to(torch.bfloat16).float()
                    y = (h @ b.float().t()).to(torch.bfloat16).float()
                    ref[tok] += y * (w * sel)[tok].sum(-1, keepdim=True)
                err = (out.float() - ref).abs().max().item()
                assert err < 0.05 * ref.abs().max().item() + 1e-3, f"EP {layout} quant={quant} it={it}: err {err}"
            moe.a2a.finalize()
    log(rt, "OK EP dispatch / combine (ll + packed, bf16 + fp8)")


def check_a2a_single(rt):
    W = rt.world_size
    ctx = ops.create_all_to_all_single_2d_context(4096, 256)
    for it in range(3):
        g = torch.Generator().manual_seed(5 + it)
        splits = torch.randint(0, 300, (W, W), generator=g)          # same matrix on every rank
        ins = splits[rt.rank].tolist()
        outs = splits[:, rt.rank].tolist()
        x = torch.randn(sum(ins), 256, device="cuda").to(torch.bfloat16)
        got = ops.all_to_all_single_2d(ctx, x, outs, ins)
        ref = torch.empty(sum(outs), 256, device="cuda", dtype=torch.bfloat16)
        dist.all_to_all_single(ref, x, outs, ins, group=rt.group)
        torch.cuda.synchronize()
        rt.check_status()
        assert torch.equal(got, ref), "all_to_all_single_2d"
    log(rt, "OK all_to_all_single_2d")


def main():
    tdb.initialize_distributed(seed=5)
    rt = tdb.get_runtime()
    check_tp_moe(rt)
    check_tp_moe_ops(rt)
    check_ep(rt)
    check_a2a_single(rt)
    log(rt, "MOE OK")
    torch.cuda.synchronize()
    rt.host_barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
