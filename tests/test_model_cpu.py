"""Dense model, safetensors loader and TP sharding on CPU ranks (gloo, fp32): TP=2 logits equal TP=1 logits."""
import json
import os
import tempfile

import torch

from dist_utils import run_cpu_ranks


def _write_checkpoint(d):
    from triton_distributed_b200.models import save_file

    g = torch.Generator().manual_seed(3)
    H, I, L, Hq, Hkv, D, V = 64, 128, 2, 4, 2, 16, 97
    cfg = {"model_type": "qwen3", "hidden_size": H, "intermediate_size": I, "num_hidden_layers": L,
           "num_attention_heads": Hq, "num_key_value_heads": Hkv, "head_dim": D, "vocab_size": V,
           "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": False}
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    r = lambda *s: torch.randn(*s, generator=g) * 0.05   # noqa: E731
    t0 = {"model.embed_tokens.weight": r(V, H), "model.norm.weight": 1 + r(H), "lm_head.weight": r(V, H)}
    t1 = {}
    for i in range(L):
        p = f"model.layers.{i}."
        t = t0 if i == 0 else t1
        t[p + "input_layernorm.weight"] = 1 + r(H)
        t[p + "post_attention_layernorm.weight"] = 1 + r(H)
        t[p + "self_attn.q_proj.weight"] = r(Hq * D, H)
        t[p + "self_attn.k_proj.weight"] = r(Hkv * D, H)
        t[p + "self_attn.v_proj.weight"] = r(Hkv * D, H)
        t[p + "self_attn.o_proj.weight"] = r(H, Hq * D)
        t[p + "self_attn.q_norm.weight"] = 1 + r(D)
        t[p + "self_attn.k_norm.weight"] = 1 + r(D)
        t[p + "mlp.gate_proj.weight"] = r(I, H)
        t[p + "mlp.up_proj.weight"] = r(I, H)
        t[p + "mlp.down_proj.weight"] = r(H, I)
    save_file(t0, os.path.join(d, "model-00001-of-00002.safetensors"))
    save_file(t1, os.path.join(d, "model-00002-of-00002.safetensors"))
    wm = {k: "model-00001-of-00002.safetensors" for k in t0}
    wm.update({k: "model-00002-of-00002.safetensors" for k in t1})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": wm}, f)


def _run(rank, world, ckpt, out_dir):
    from triton_distributed_b200.models import Engine, ModelConfig

    cfg = ModelConfig(model_name="ckpt", max_length=32, dtype=torch.float32, rank=rank, world_size=world,
                      checkpoint_dir=ckpt)
    ids = torch.tensor([[5, 9, 2, 77, 31], [1, 2, 3, 4, 5]])
    res = {}
    for backend in ("torch", "triton_dist", "triton_dist_AR", "triton_dist_gemm_ar"):
        eng = Engine(cfg)
        eng.backend = backend
        eng.no_graph = True
        toks = eng.serve(ids, 4)
        res[backend] = (toks, eng._logits.clone())
    if rank == 0:
        torch.save(res, os.path.join(out_dir, f"w{world}.pt"))


def test_tp2_matches_tp1_on_cpu():
    with tempfile.TemporaryDirectory() as d:
        _write_checkpoint(d)
        run_cpu_ranks(_run, 1, (d, d))
        run_cpu_ranks(_run, 2, (d, d))
        r1 = torch.load(os.path.join(d, "w1.pt"))
        r2 = torch.load(os.path.join(d, "w2.pt"))
        ref_toks, ref_logits = r1["torch"]
        for backend, (toks, logits) in list(r1.items()) + list(r2.items()):
            assert torch.equal(toks, ref_toks), backend
            torch.testing.assert_close(logits, ref_logits, rtol=1e-4, atol=1e-4)


def test_safetensors_roundtrip_and_slices():
    from triton_distributed_b200.models import SafetensorsFile, save_file

    with tempfile.TemporaryDirectory() as d:
        a = torch.randn(12, 10)
        b = torch.randn(7).to(torch.bfloat16)
        save_file({"a": a, "b": b}, os.path.join(d, "x.safetensors"), metadata={"format": "pt"})
        f = SafetensorsFile(os.path.join(d, "x.safetensors"))
        assert torch.equal(f.get("a"), a) and torch.equal(f.get("b"), b)
        assert torch.equal(f.get("a", rows=(3, 9)), a[3:9])
        assert torch.equal(f.get("a", cols=(2, 5)), a[:, 2:5])
        assert torch.equal(f.get("a", rows=(6, 12), cols=(5, 10)), a[6:12, 5:10])
        f.close()
        # files written here are readable by the upstream safetensors package when it is installed
        try:
            from safetensors.torch import load_file
            ld = load_file(os.path.join(d, "x.safetensors"))
            assert torch.equal(ld["a"], a) and torch.equal(ld["b"], b)
        except ImportError:
            pass


def _run_sampling(rank, world, ckpt, out_dir):
    """temperature > 0 on two ranks: every rank must return the same ids (same generator seed + broadcast)."""
    import torch.distributed as dist

    from triton_distributed_b200.models import Engine, ModelConfig

    cfg = ModelConfig(model_name="ckpt", max_length=32, dtype=torch.float32, rank=rank, world_size=world,
                      checkpoint_dir=ckpt)
    eng = Engine(cfg, temperature=0.9, top_p=0.95, seed=17)
    eng.backend = "triton_dist_AR"
    eng.no_graph = True
    toks = eng.serve(torch.tensor([[5, 9, 2, 77, 31], [1, 2, 3, 4, 5]]), 6)
    gathered = [torch.empty_like(toks) for _ in range(world)]
    dist.all_gather(gathered, toks)
    for t in gathered:
        assert torch.equal(t, gathered[0]), (rank, t, gathered[0])
    # a second request re-uses the engine: the contexts of the first one are kept, not re-created
    key = eng._ctx_key
    toks2 = eng.serve(torch.tensor([[7, 7, 7], [8, 8, 8]]), 3)
    assert eng._ctx_key == key and toks2.shape == (2, 3)


def test_sampling_is_identical_on_all_ranks():
    with tempfile.TemporaryDirectory() as d:
        _write_checkpoint(d)
        run_cpu_ranks(_run_sampling, 2, (d, d))


def _run_reject(rank, world, ckpt, out_dir):
    import pytest

    from triton_distributed_b200.models import Engine, ModelConfig

    cfg = ModelConfig(model_name="ckpt", max_length=16, dtype=torch.float32, rank=rank, world_size=world,
                      checkpoint_dir=ckpt)
    eng = Engine(cfg)
    eng.no_graph = True
    ok = torch.tensor([[1, 2, 3, 4]])
    with pytest.raises(ValueError, match="max_length"):
        eng.serve(ok, 13)                                   # 4 + 13 > 16 cache rows per sequence
    with pytest.raises(ValueError, match="token ids"):
        eng.serve(torch.tensor([[1, 2, 97]]), 2)            # vocabulary is 97
    with pytest.raises(ValueError, match="token ids"):
        eng.serve(torch.tensor([[-1, 2, 3]]), 2)
    with pytest.raises(ValueError, match="gen_len"):
        eng.serve(ok, 0)
    with pytest.raises(ValueError):
        eng.serve(torch.zeros(0, 4, dtype=torch.int64), 2)
    assert eng.kv_cache is None                             # nothing was allocated or launched for any of them
    assert eng.serve(ok, 12).shape == (1, 12)               # exactly full is fine


def test_engine_rejects_requests_that_do_not_fit():
    with tempfile.TemporaryDirectory() as d:
        _write_checkpoint(d)
        run_cpu_ranks(_run_reject, 1, (d, d))


def test_model_server_checks_requests_on_the_host():
    import importlib.util

    spec = importlib.util.spec_from_file_location("model_server", os.path.join(os.path.dirname(__file__), "..", "examples",
                                                                               "model_server.py"))
    ms = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ms)

    class FakeEngine:
        def __init__(self):
            self.served = 0

        def validate_request(self, ids, gen_len):
            if ids.shape[1] + gen_len > 8:
                raise ValueError("prompt + gen_len exceeds max_length")

        def serve(self, ids, gen_len):
            self.served += 1
            return ids[:, :1].repeat(1, gen_len)

    e = FakeEngine()
    assert "error" in ms.handle(e, {"input_ids": [[1, 2, 3]], "gen_len": 100})
    assert "error" in ms.handle(e, {"gen_len": 1})
    assert "error" in ms.handle(e, {"input_ids": [[1, 2], [3]], "gen_len": 1})
    assert "error" in ms.handle(e, {"input_ids": "abc", "gen_len": 1})
    assert e.served == 0
    assert ms.handle(e, {"input_ids": [[1, 2, 3]], "gen_len": 2})["output_ids"] == [[1, 1]]
