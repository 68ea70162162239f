"""Model configuration: run-time options (``ModelConfig``, as python/triton_dist/models/config.py:31-37) and the
architecture hyper-parameters (``ArchConfig``) of the supported families, built in so that random-init benchmarks
need no download; ``ArchConfig.from_hf_json`` reads a Hugging Face ``config.json`` instead."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class ArchConfig:
    name: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    qk_norm: bool = True
    tie_word_embeddings: bool = False
    # MoE (0 experts = dense)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @staticmethod
    def from_hf_json(path: str) -> "ArchConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            c = json.load(f)
        heads = c["num_attention_heads"]
        mt = c.get("model_type", "")
        return ArchConfig(
            name=c.get("_name_or_path", mt), hidden_size=c["hidden_size"], intermediate_size=c.get("intermediate_size", 0),
            num_hidden_layers=c["num_hidden_layers"], num_attention_heads=heads,
            num_key_value_heads=c.get("num_key_value_heads", heads), head_dim=c.get("head_dim", c["hidden_size"] // heads),
            vocab_size=c["vocab_size"], rms_norm_eps=c.get("rms_norm_eps", 1e-6), rope_theta=c.get("rope_theta", 1e4),
            qk_norm=mt.startswith("qwen3"), tie_word_embeddings=c.get("tie_word_embeddings", False),
            num_experts=c.get("num_experts", 0), num_experts_per_tok=c.get("num_experts_per_tok", 0),
            moe_intermediate_size=c.get("moe_intermediate_size", 0), norm_topk_prob=c.get("norm_topk_prob", True))


PRESETS = {
    "Qwen/Qwen3-0.6B": ArchConfig("Qwen/Qwen3-0.6B", 1024, 3072, 28, 16, 8, 128, 151936, tie_word_embeddings=True),
    "Qwen/Qwen3-8B": ArchConfig("Qwen/Qwen3-8B", 4096, 12288, 36, 32, 8, 128, 151936),
    "Qwen/Qwen3-14B": ArchConfig("Qwen/Qwen3-14B", 5120, 17408, 40, 40, 8, 128, 151936),
    "Qwen/Qwen3-32B": ArchConfig("Qwen/Qwen3-32B", 5120, 25600, 64, 64, 8, 128, 151936),
    "meta-llama/Meta-Llama-3-70B": ArchConfig("meta-llama/Meta-Llama-3-70B", 8192, 28672, 80, 64, 8, 128, 128256,
                                              rms_norm_eps=1e-5, rope_theta=5e5, qk_norm=False),
    "ByteDance-Seed/Seed-OSS-36B-Instruct": ArchConfig("ByteDance-Seed/Seed-OSS-36B-Instruct", 5120, 27648, 64, 80, 8, 128,
                                                       155136, rope_theta=1e7, qk_norm=False),
    "Qwen/Qwen3-30B-A3B": ArchConfig("Qwen/Qwen3-30B-A3B", 2048, 6144, 48, 32, 4, 128, 151936, num_experts=128,
                                     num_experts_per_tok=8, moe_intermediate_size=768),
    "Qwen/Qwen3-235B-A22B": ArchConfig("Qwen/Qwen3-235B-A22B", 4096, 12288, 94, 64, 4, 128, 151936, num_experts=128,
                                       num_experts_per_tok=8, moe_intermediate_size=1536),
    # what one rank of Qwen3-32B holds under TP=8, as a single-GPU model: lets one GPU profile the per-rank kernels
    "Qwen/Qwen3-32B-tp8-shard": ArchConfig("Qwen/Qwen3-32B-tp8-shard", 5120, 3200, 64, 8, 1, 128, 18992),
    # small shapes for tests and the smoke check
    "tiny-dense": ArchConfig("tiny-dense", 256, 512, 2, 8, 2, 64, 1024),
    "tiny-moe": ArchConfig("tiny-moe", 256, 512, 2, 8, 2, 64, 1024, num_experts=8, num_experts_per_tok=2,
                           moe_intermediate_size=128),
}


@dataclass
class ModelConfig:
    model_name: str = "Qwen/Qwen3-32B"
    max_length: int = 4096
    dtype: torch.dtype = torch.bfloat16
    rank: int = 0
    world_size: int = 1
    local_only: bool = True          # there is no network: never try to download
    checkpoint_dir: Optional[str] = None   # directory with *.safetensors (+ index json); None = random init
    num_layers_override: Optional[int] = None
    seed: int = 0

    def arch(self) -> ArchConfig:
        if self.checkpoint_dir and os.path.exists(os.path.join(self.checkpoint_dir, "config.json")):
            a = ArchConfig.from_hf_json(self.checkpoint_dir)
        elif self.model_name in PRESETS:
            a = PRESETS[self.model_name]
        else:
            raise KeyError(f"unknown model {self.model_name}; known: {sorted(PRESETS)}")
        if self.num_layers_override is not None:
            import dataclasses
            a = dataclasses.replace(a, num_hidden_layers=self.num_layers_override)
        return a
