"""Qwen3 (dense) decode step as one megakernel launch.

API of the reference: ``Qwen3Model`` (python/triton_dist/mega_triton_kernel/models/qwen3.py:51-202): decode only
(one token per sequence), embedding and sampling outside the kernel, LM head optionally inside.  The model is built
from an existing :class:`~triton_distributed_b200.models.DenseLLM` (its sharded weights) and a dense ``KV_Cache``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..models.dense import DenseLLM
from ..models.kv_cache import KV_Cache
from .model_builder import ModelBuilder


class Qwen3Model:
    def __init__(self, model: DenseLLM, kv_cache: KV_Cache, batch: int, lm_head_inside: bool = True,
                 enable_profiling: bool = False, policy: str = "round_robin", prefetch: bool = False):
        """``prefetch``: schedule L2 prefetch tasks for the weights of the operator after next wherever the step would
        otherwise leave HBM idle (during the attention of short contexts and the two all-reduces of a layer)."""
        self.model, self.kv_cache, self.batch = model, kv_cache, batch
        a = model.arch
        W = model.world_size
        dev, dt = model.device, model.dtype
        H, D = a.hidden_size, a.head_dim
        l0 = model.layers[0]
        Hq, Hkv = l0.attn.q_heads, l0.attn.kv_heads
        I = l0.mlp.inter_local
        B = batch
        z = lambda *s: torch.zeros(*s, dtype=dt, device=dev)   # noqa: E731
        self.resid, self.n_out, self.qkv = z(B, H), z(B, H), z(B, (Hq + 2 * Hkv) * D)
        self.q, self.attn_out, self.o_out = z(B, Hq, D), z(B, Hq * D), z(B, H)
        self.gate_up, self.act, self.down_out = z(B, 2 * I), z(B, I), z(B, H)
        self.final, self.logits = z(B, H), z(B, a.vocab_size)
        self.kv_lens = torch.zeros(B, dtype=torch.int32, device=dev)
        b = ModelBuilder(B, enable_profiling=enable_profiling, policy=policy)
        self.builder = b
        prev_out = None
        for li, l in enumerate(model.layers):
            k_cache, v_cache = kv_cache.layer(li)
            if li == 0:
                b.make_rms_norm(self.resid, l.input_norm_w, self.n_out, l.eps)
            else:
                b.make_rms_norm(prev_out, l.input_norm_w, self.n_out, l.eps, residual=self.resid)
            b.make_qkv_proj(self.n_out, l.attn.wqkv, self.qkv)
            b.make_qk_norm_rope_update_kvcache(self.qkv, l.attn.q_norm_w, l.attn.k_norm_w, self.q, k_cache, v_cache,
                                               kv_cache.kv_offset, Hq, Hkv, D, l.attn.eps, l.attn.rope_theta)
            if prefetch:
                b.make_prefetch(l.attn.wo, after=self.qkv)
            b.make_flash_decode(self.q, k_cache, v_cache, self.kv_lens, self.attn_out.view(B, Hq, D), Hq, Hkv, D, l.attn.scale)
            if prefetch:
                b.make_prefetch(l.mlp.gate_up_proj, after=self.attn_out)
            b.make_o_proj(self.attn_out, l.attn.wo, self.o_out, all_reduce=True)
            b.make_rms_norm(self.o_out, l.post_norm_w, self.n_out, l.eps, residual=self.resid)
            b.make_fc1(self.n_out, l.mlp.gate_up_proj, self.gate_up)
            b.make_silu_mul_up(self.gate_up, self.act)
            if prefetch and li + 1 < len(model.layers):
                b.make_prefetch(model.layers[li + 1].attn.wqkv, after=self.act)
            b.make_fc2(self.act, l.mlp.down_proj, self.down_out, all_reduce=True)
            prev_out = self.down_out
        b.make_rms_norm(prev_out, model.final_norm_w, self.final, a.rms_norm_eps, residual=self.resid)
        self.lm_head_inside = lm_head_inside
        if lm_head_inside:
            b.make_lm_head(self.final, model.lm_head, self.logits)
        b.compile()

    @torch.no_grad()
    def mega_forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        """input_ids [B, 1] -> fp32 logits [B, vocab]; the caller advances ``kv_cache.kv_offset`` afterwards."""
        self.resid.copy_(ops.embedding(input_ids.reshape(-1), self.model.embed_tokens))
        torch.add(self.kv_cache.kv_offset[:self.batch], 1, out=self.kv_lens)
        self.builder.run()
        if self.lm_head_inside:
            return self.logits.float()
        return ops.gemm(self.final, self.model.lm_head).float()

    mega_forwrad = mega_forward   # the reference spells it this way (qwen3.py:109)
