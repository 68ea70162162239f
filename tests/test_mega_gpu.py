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
    mega = Qwen3Model(model, caches[1], batch, enable_profiling=(batch == 3))
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
