"""Models, KV caches, weight loading and the serving engine (the reference's ``triton_dist.models``)."""
from .config import ArchConfig, ModelConfig, PRESETS  # noqa: F401
from .kv_cache import KV_Cache, PagedKVCache  # noqa: F401
from .safetensors_io import SafetensorsFile, ShardedCheckpoint, save_file  # noqa: F401
from .dense import DenseLLM, DenseLLMLayer  # noqa: F401
from .engine import Engine  # noqa: F401
from .qwen_moe import Qwen3MoE, Qwen3MoELayer  # noqa: F401


class AutoLLM:
    """``AutoLLM.from_pretrained(ModelConfig)`` picks the model class (python/triton_dist/models/__init__.py:33-59)."""

    @staticmethod
    def from_pretrained(model_config: ModelConfig, group=None):
        arch = model_config.arch()
        if arch.is_moe:
            from .qwen_moe import Qwen3MoE
            return Qwen3MoE(model_config, group)
        return DenseLLM(model_config, group)


def smoke_decode():
    """One prefill + two decode steps of a tiny Qwen3-shaped model on the current device."""
    import torch

    from ..runtime import get_runtime

    rt = get_runtime()
    cfg = ModelConfig(model_name="tiny-dense", max_length=64, rank=rt.rank, world_size=rt.world_size)
    eng = Engine(cfg)
    eng.backend = "triton_dist_gemm_ar"
    ids = torch.randint(0, 1000, (2, 8), device=rt.device)
    out = eng.serve(ids, 3)
    assert out.shape == (2, 3)
