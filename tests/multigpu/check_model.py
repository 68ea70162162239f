"""Multi-GPU model check (torchrun): every overlapped backend of the dense model against its torch (NCCL + cuBLAS)
backend, with and without CUDA graphs, on a small Qwen3-shaped model."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import triton_distributed_b200 as tdb  # noqa: E402
from triton_distributed_b200.models import ArchConfig, Engine, ModelConfig, PRESETS  # noqa: E402


def compare_generation(ref_logits, ref_toks, logits, toks, rel=0.15, abs_=0.05, min_ok_frac=1.0):
    """Greedy decoding of two numerically different backends can part ways at a near-tie, after which their logits are
    not comparable.  Compare, step by step, only the sequences whose token history is still identical; returns the
    largest in-tolerance error and the number of (step, sequence) pairs compared.  ``min_ok_frac`` < 1 tolerates a few
    pairs outside the band: a mixture-of-experts router is discontinuous, a near-tie between two experts can flip with
    the GEMM's rounding and changes that token's output by far more than rounding."""
    worst, n, bad = 0.0, 0, 0
    for i, (a, b) in enumerate(zip(ref_logits, logits)):
        same = (ref_toks[:, :i] == toks[:, :i]).all(dim=1) if i > 0 else torch.ones(a.shape[0], dtype=torch.bool, device=a.device)
        if not bool(same.any()):
            break
        err = (a[same] - b[same]).abs().amax(dim=1)
        tol = rel * a[same].abs().max().item() + abs_
        ok = err < tol
        bad += int((~ok).sum())
        n += int(same.sum())
        if bool(ok.any()):
            worst = max(worst, err[ok].max().item())
    assert n > 0 and (n - bad) >= min_ok_frac * n, f"{bad} of {n} (step, sequence) pairs with identical history are out of tolerance"
    return worst, n


def main():
    tdb.initialize_distributed(seed=3)
    rt = tdb.get_runtime()
    W = rt.world_size
    PRESETS["check"] = ArchConfig("check", 1024, 2048, 3, 16, 8, 128, 4096)
    # the per-rank shapes of "check" on eight ranks (2 query heads, 1 KV head, 256 intermediate columns per rank and a
    # batch of 16), whatever the world size is: narrow shards take other kernel paths than wide ones
    PRESETS["check-narrow"] = ArchConfig("check-narrow", 1024, 256 * W, 3, 2 * W, W, 128, 4096)
    for name, B in (("check", 2 * W), ("check-narrow", 16)):
        check_backends(rt, ModelConfig(model_name=name, max_length=256, rank=rt.rank, world_size=W), B)
    cfg = ModelConfig(model_name="check", max_length=256, rank=rt.rank, world_size=W)
    check_megakernel(rt, cfg)
    if rt.rank == 0:
        print("MODEL OK", flush=True)
    torch.cuda.synchronize()
    rt.host_barrier()
    sys.stdout.flush()
    os._exit(0)   # skip interpreter teardown: nothing left to check, and it must not delay the launcher


def check_backends(rt, cfg, B):
    ids = torch.randint(0, 4096, (B, 33), device=rt.device, generator=torch.Generator(device=rt.device).manual_seed(1))
    ref = None
    for backend, graph in [("torch", False), ("triton_dist_AR", False), ("triton_dist_AR", True), ("triton_dist_gemm_ar", True),
                           ("triton_dist", False), ("triton_dist", True)]:
        eng = Engine(cfg)
        eng.backend = backend
        eng.no_graph = not graph
        eng.keep_logits = True
        toks = eng.serve(ids, 8)
        torch.cuda.synchronize()
        rt.check_status()
        if ref is None:
            ref = (eng.step_logits, toks)
        err, n = compare_generation(ref[0], ref[1], eng.step_logits, toks)
        if rt.rank == 0:
            print(f"{cfg.model_name} B={B} backend {backend:22s} graph={graph} max|dlogits|={err:.4f} over {n} (step, sequence) "
                  f"pairs with identical history, decode {eng.last_decode_ms:.3f} ms/step", flush=True)
        assert n >= 2 * B, "too few comparable steps"
        rt.host_barrier()


def check_megakernel(rt, cfg):
    """decode megakernel (fused GEMM+AR tasks across ranks) against the layer-wise model"""
    W = rt.world_size
    from triton_distributed_b200.mega import Qwen3Model
    from triton_distributed_b200.models import DenseLLM, KV_Cache
    model = DenseLLM(cfg)
    model.set_fwd("triton_dist_AR")
    model.init_ctx_for("triton_dist_AR", 64)
    a = model.arch
    for Bm in (1, 16, 48):
        prompt = torch.randint(0, 4096, (Bm, 21), device=rt.device, generator=torch.Generator(device=rt.device).manual_seed(2))
        pos = torch.arange(21, device=rt.device).unsqueeze(0).expand(Bm, 21).contiguous()
        caches = [KV_Cache(a.num_hidden_layers, Bm, 256, max(1, a.num_key_value_heads // W), a.head_dim, device=rt.device)
                  for _ in range(2)]
        for c in caches:
            model.inference(prompt, pos, c)
            c.inc_offset(21)
        mega = Qwen3Model(model, caches[1], Bm, prefetch=(Bm == 16))
        tok = prompt[:, :1].contiguous()
        for step in range(4):
            ref_l = model.inference(tok, caches[0].kv_offset.to(torch.int64).unsqueeze(1), caches[0])
            got = mega.mega_forward(tok)
            torch.cuda.synchronize()
            rt.check_status()
            err = (got - ref_l).abs().max().item()
            assert err < 0.1 * ref_l.abs().max().item() + 0.05, f"megakernel B={Bm} step {step}: {err}"
            for c in caches:
                c.inc_offset(1)
            tok = ref_l.argmax(-1).reshape(Bm, 1)
        rt.host_barrier()
    if rt.rank == 0:
        print("megakernel matches the layer-wise decode on", W, "ranks", flush=True)
    check_mega_aux_tasks(rt)


def check_mega_aux_tasks(rt):
    """Stand-alone all-reduce, rank-barrier and prefetch tasks of the megakernel across ranks, with and without NVLS."""
    import torch.distributed as dist
    from triton_distributed_b200.mega import ModelBuilder

    W, dev = rt.world_size, rt.device
    B, K, N = 7, 256, 2048 + 128
    g = torch.Generator(device=dev).manual_seed(11 + rt.rank)
    x = torch.randn(B, K, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    for use_mc in (True, False):
        part = torch.zeros(B, N, device=dev, dtype=torch.bfloat16)
        out = torch.zeros(B, N, device=dev, dtype=torch.bfloat16)
        b = ModelBuilder(B, use_multimem=use_mc)
        b.make_prefetch(w)
        b.make_linear(x, w, part)                       # local partial product, no fused all-reduce
        b.make_barrier_all_intra_node()
        b.make_allreduce(part, out, chunk_cols=512)
        b.compile()
        for it in range(3):
            b.run()
            torch.cuda.synchronize()
            rt.check_status()
            ref = part.float().clone()
            dist.all_reduce(ref, group=rt.group)
            err = (out.float() - ref).abs().max().item()
            assert err < 2e-2 * ref.abs().max().item() + 1e-3, f"mega all-reduce task (nvls={use_mc}) it={it}: {err}"
        rt.host_barrier()
    if rt.rank == 0:
        print("megakernel all-reduce / barrier / prefetch tasks OK on", W, "ranks", flush=True)


if __name__ == "__main__":
    main()
