"""Decode megakernel on one GPU: a whole decode step in one launch against the layer-by-layer model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import triton_distributed_b200 as tdb

    tdb.initialize_distributed(seed=0)
    return tdb.get_runtime()


@pytest.mark.parametrize("batch", [1, 3, 20, 64])
def test_megakernel_matches_layerwise_decode(rt, batch):
    from triton_distributed_b200.mega import Qwen3Model
    from triton_distributed_b200.models import DenseLLM, KV_Cache, ModelConfig

    cfg = ModelConfig(model_name="tiny-dense", max_length=128, rank=rt.rank, world_size=rt.world_size)
    model = DenseLLM(cfg)
    model.set_fwd("triton_dist_AR")
    model.init_ctx_for("triton_dist_AR", 64)
    a = model.arch
    prompt = torch.randint(0, 1000, (batch, 9), device=rt.device)
    pos = torch.arange(9, device=rt.device).unsqueeze(0).expand(batch, 9).contiguous()
    caches = [KV_Cache(a.num_hidden_layers, batch, 128, a.num_key_value_heads, a.head_dim, device=rt.device) for _ in range(2)]
    for c in caches:
        model.inference(prompt, pos, c)
        c.inc_offset(9)
    mega = Qwen3Model(model, caches[1], batch, enable_profiling=(batch == 3), prefetch=(batch in (1, 20)))
    tok = torch.randint(0, 1000, (batch, 1), device=rt.device)
    for step in range(3):
        ref = model.inference(tok, caches[0].kv_offset.to(torch.int64).unsqueeze(1), caches[0])
        got = mega.mega_forward(tok)
        torch.cuda.synchronize()
        rt.check_status()
        err = (got - ref).abs().max().item()
        assert err < 0.1 * ref.abs().max().item() + 0.05, f"batch {batch} step {step}: max |dlogits| {err}"
        for c in caches:
            c.inc_offset(1)
        tok = ref.argmax(-1).reshape(batch, 1)
    # KV caches written by the megakernel equal the layer-wise ones
    torch.testing.assert_close(caches[1].k_cache[:, :, :12].float(), caches[0].k_cache[:, :, :12].float(), rtol=3e-2, atol=3e-2)
    if batch == 3:
        act = mega.builder.get_sm_activity()
        assert len(act) > 0 and all(0 <= v <= 1.0001 for v in act.values())
        assert sum(mega.builder.tasks_per_sm()) > 0


def test_builder_prefetch_barrier_allreduce_lm_head_tasks(rt, tmp_path):
    """The auxiliary task types on their own: L2 prefetch (no visible effect, must not disturb anything), rank barrier,
    stand-alone all-reduce (one rank: the sum is the input) and the LM-head linear, against PyTorch."""
    from triton_distributed_b200.mega import ModelBuilder

    B, K, N = 5, 512, 1024 + 256
    dev = rt.device
    g = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn(B, K, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    big = torch.randn(3 * 1024 * 1024 + 8, device=dev, generator=g).to(torch.bfloat16)    # 6 MB + a ragged tail
    logits = torch.zeros(B, N, device=dev, dtype=torch.bfloat16)
    summed = torch.zeros(B, N, device=dev, dtype=torch.bfloat16)
    b = ModelBuilder(B, enable_profiling=True)
    st_p = b.make_prefetch(big)
    st_l = b.make_lm_head(x, w, logits)
    st_b = b.make_barrier_all_intra_node()
    st_a = b.make_allreduce(logits, summed, chunk_cols=512)
    assert len({st_p, st_l, st_b, st_a}) == 4
    b.compile()
    for _ in range(2):
        b.run()
        torch.cuda.synchronize()
        rt.check_status()
    ref = (x.float() @ w.float().t())
    torch.testing.assert_close(logits.float(), ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(summed.float() / rt.world_size, logits.float(), rtol=1e-2, atol=1e-2)
    names = {e["name"] for e in b.dump_trace(str(tmp_path / "trace.json"))["traceEvents"]}
    assert {"prefetch_l2", "barrier_all", "all_reduce", "linear"} <= names, names
