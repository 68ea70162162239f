"""Qwen3-MoE (sparse MLP blocks, tensor-parallel experts) on the layers of this package.

API of the reference: ``Qwen3MoE`` (python/triton_dist/models/qwen_moe.py:50-206), modes torch / triton_dist.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..parallel.tp_attn import TP_Attn
from ..parallel.tp_moe import TP_MoE
from ..runtime import get_runtime
from .config import ModelConfig
from .dense import DenseLLM, DenseLLMLayer


class Qwen3MoELayer(DenseLLMLayer):
    def __init__(self, layer_idx: int, rank: int, world_size: int, group):
        self.layer_idx = layer_idx
        self.attn = TP_Attn(rank, world_size, group)
        self.mlp = TP_MoE(rank, world_size, group)
        self.input_norm_w = self.post_norm_w = None
        self.eps = 1e-6


class Qwen3MoE(DenseLLM):
    def __init__(self, model_config: ModelConfig, group=None):
        self.rt = get_runtime()
        self.model_config = model_config
        self.arch = model_config.arch()
        self.rank, self.world_size = self.rt.rank, self.rt.world_size
        self.group = group if group is not None else self.rt.group
        self.dtype, self.device = model_config.dtype, self.rt.device
        self.mode = "torch"
        self.layers = [Qwen3MoELayer(i, self.rank, self.world_size, self.group) for i in range(self.arch.num_hidden_layers)]
        self.init_parameters()
        self.set_fwd("torch")

    def init_parameters(self):
        a, dev, dt = self.arch, self.device, self.dtype
        if self.model_config.checkpoint_dir:
            self._load_checkpoint()
            return
        g = torch.Generator(device=dev).manual_seed(self.model_config.seed)
        self.embed_tokens = (torch.randn(a.vocab_size, a.hidden_size, device=dev, generator=g) * 0.02).to(dt)
        self.lm_head = (torch.randn(a.vocab_size, a.hidden_size, device=dev, generator=g) * 0.02).to(dt)
        self.final_norm_w = torch.ones(a.hidden_size, device=dev, dtype=dt)
        for i, l in enumerate(self.layers):
            l.eps = a.rms_norm_eps
            l.input_norm_w = torch.ones(a.hidden_size, device=dev, dtype=dt)
            l.post_norm_w = torch.ones(a.hidden_size, device=dev, dtype=dt)
            l.attn.init_random(a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim, a.qk_norm,
                               a.rope_theta, a.rms_norm_eps, dt, dev, seed=self.model_config.seed + 2 * i)
            l.mlp.init_random(a.hidden_size, a.moe_intermediate_size, a.num_experts, a.num_experts_per_tok, dt, dev,
                              seed=self.model_config.seed + 2 * i + 1)
            l.mlp.norm_topk = a.norm_topk_prob

    def _load_checkpoint(self):
        from .safetensors_io import ShardedCheckpoint

        a, dev, dt, W, r = self.arch, self.device, self.dtype, self.world_size, self.rank
        ck = ShardedCheckpoint(self.model_config.checkpoint_dir)
        get = lambda n: ck.get(n).to(dev).to(dt)   # noqa: E731
        self.embed_tokens = get("model.embed_tokens.weight")
        self.lm_head = get("lm_head.weight") if "lm_head.weight" in ck else self.embed_tokens
        self.final_norm_w = get("model.norm.weight")
        D, Hq, Hkv = a.head_dim, a.num_attention_heads, a.num_key_value_heads
        for i, l in enumerate(self.layers):
            p = f"model.layers.{i}."
            l.eps = a.rms_norm_eps
            l.input_norm_w = get(p + "input_layernorm.weight")
            l.post_norm_w = get(p + "post_attention_layernorm.weight")
            l.attn._init_parameters(wq=ck.get(p + "self_attn.q_proj.weight"), wk=ck.get(p + "self_attn.k_proj.weight"),
                                    wv=ck.get(p + "self_attn.v_proj.weight"), wo=ck.get(p + "self_attn.o_proj.weight"),
                                    q_norm=ck.get(p + "self_attn.q_norm.weight") if (p + "self_attn.q_norm.weight") in ck else None,
                                    k_norm=ck.get(p + "self_attn.k_norm.weight") if (p + "self_attn.k_norm.weight") in ck else None,
                                    hidden=a.hidden_size, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                                    rope_theta=a.rope_theta, eps=a.rms_norm_eps, device=dev)
            l.attn.wqkv, l.attn.wo = l.attn.wqkv.to(dt), l.attn.wo.to(dt)
            gate = torch.stack([ck.get(p + f"mlp.experts.{e}.gate_proj.weight") for e in range(a.num_experts)])
            up = torch.stack([ck.get(p + f"mlp.experts.{e}.up_proj.weight") for e in range(a.num_experts)])
            down = torch.stack([ck.get(p + f"mlp.experts.{e}.down_proj.weight") for e in range(a.num_experts)])
            l.mlp._init_parameters(ck.get(p + "mlp.gate.weight").to(dt), gate.to(dt), up.to(dt), down.to(dt),
                                   a.num_experts_per_tok, a.norm_topk_prob, dev)
        ck.close()

    def init_triton_dist_ctx(self, max_M: int = 4096):
        l0 = self.layers[0]
        l0.attn._init_ctx(max_M)
        l0.mlp._init_ctx(max_M)
        for l in self.layers[1:]:
            l.attn.ag_ctx, l.attn.rs_ctx = l0.attn.ag_ctx, l0.attn.rs_ctx
            l.mlp.ag_ctx, l.mlp.rs_ctx, l.mlp.ll_ctx = l0.mlp.ag_ctx, l0.mlp.rs_ctx, l0.mlp.ll_ctx
        self.ag_ll_ctx = ops.create_fast_allgather_context(max_ll_bytes=max(64 * 1024, 2 * max_M * self.arch.hidden_size
                                                                            // max(self.world_size, 1)))

    def init_triton_dist_AR_ctx(self, max_M: int = 4096):
        l0 = self.layers[0]
        l0.attn._init_AR_ctx(max_M)
        l0.mlp._init_ctx(max_M)
        for l in self.layers[1:]:
            l.attn.ar_ctx = l0.attn.ar_ctx
            l.mlp.ag_ctx, l.mlp.rs_ctx, l.mlp.ll_ctx = l0.mlp.ag_ctx, l0.mlp.rs_ctx, l0.mlp.ll_ctx

    def init_triton_dist_gemm_ar_ctx(self, max_M: int = 256):
        l0 = self.layers[0]
        l0.attn._init_gemm_ar_ctx(max_M)
        l0.mlp._init_ctx(max_M)
        for l in self.layers[1:]:
            l.attn.gemm_ar_ctx = l0.attn.gemm_ar_ctx
            l.mlp.ag_ctx, l.mlp.rs_ctx, l.mlp.ll_ctx = l0.mlp.ag_ctx, l0.mlp.rs_ctx, l0.mlp.ll_ctx
