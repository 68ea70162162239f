"""Dense decoder-only LLM (Qwen3 / Llama-3 / Seed-OSS families) on the tensor-parallel layers of this package.

API of the reference: ``DenseLLM`` / ``DenseLLMLayer`` (python/triton_dist/models/dense.py:53-241):
``set_fwd(mode)`` with modes torch / triton_dist / triton_dist_AR / triton_dist_gemm_ar, ``init_triton_dist_ctx`` /
``init_triton_dist_AR_ctx`` / ``init_triton_dist_gemm_ar_ctx`` and ``inference(input_ids, position_ids, kv_cache,
wo_lm_head)`` returning fp32 logits of the last token.  Weights come from an own safetensors reader (sharded per
rank while loading) or are random-initialised with the architecture's shapes.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..parallel.tp_attn import TP_Attn
from ..parallel.tp_mlp import TP_MLP
from ..runtime import get_runtime
from .config import ArchConfig, ModelConfig
from .safetensors_io import ShardedCheckpoint


class DenseLLMLayer:
    def __init__(self, layer_idx: int, rank: int, world_size: int, group):
        self.layer_idx = layer_idx
        self.attn = TP_Attn(rank, world_size, group)
        self.mlp = TP_MLP(rank, world_size, group)
        self.input_norm_w: Optional[torch.Tensor] = None
        self.post_norm_w: Optional[torch.Tensor] = None
        self.eps = 1e-6

    def set_fwd(self, mode: str):
        self.attn.set_fwd(mode)
        self.mlp.set_fwd(mode)

    def fwd(self, hidden: torch.Tensor, residual: Optional[torch.Tensor], position_ids, kv_cache):
        """Pre-norm block with the residual add fused into the following RMSNorm.  hidden/residual [B, S, H]."""
        shape = hidden.shape
        if residual is None:
            residual = hidden.reshape(-1, shape[-1]).clone()
            x = ops.rmsnorm(hidden.reshape(-1, shape[-1]), self.input_norm_w, self.eps)
        else:
            x = ops.rmsnorm(hidden.reshape(-1, shape[-1]), self.input_norm_w, self.eps, residual=residual)
        a = self.attn(x.reshape(shape), position_ids, kv_cache, self.layer_idx)
        x = ops.rmsnorm(a.reshape(-1, shape[-1]), self.post_norm_w, self.eps, residual=residual)
        m = self.mlp(x)
        return m.reshape(shape), residual


    def fwd_fused_decode(self, stream: torch.Tensor, position_ids, kv_cache, gemv_ctx):
        """Decode step for up to eight tokens with four fused GEMV launches plus attention: ``stream`` [M, H] holds
        the residual stream and is updated in place (norms in the GEMV prologues, all-reduce and residual add in
        their epilogues, SiLU*up in the down projection's prologue)."""
        a, m = self.attn, self.mlp
        bsz = stream.shape[0]
        qkv = ops.gemv_fused(stream, a.wqkv, norm_weight=self.input_norm_w, eps=self.eps)
        o = a._attend(qkv, position_ids, kv_cache, self.layer_idx, bsz, 1)
        ops.gemv_fused(o, a.wo, out=stream, residual=stream, ar_ctx=gemv_ctx)
        gu = ops.gemv_fused(stream, m.gate_up_proj, norm_weight=self.post_norm_w, eps=self.eps)
        ops.gemv_fused(gu, m.down_proj, out=stream, silu_mul=True, residual=stream, ar_ctx=gemv_ctx)
        return stream


class DenseLLM:
    def __init__(self, model_config: ModelConfig, group=None):
        self.rt = get_runtime()
        self.model_config = model_config
        self.arch: ArchConfig = model_config.arch()
        self.rank, self.world_size = self.rt.rank, self.rt.world_size
        self.group = group if group is not None else self.rt.group
        self.dtype = model_config.dtype
        self.device = self.rt.device
        self.mode = "torch"
        self.layers = [DenseLLMLayer(i, self.rank, self.world_size, self.group) for i in range(self.arch.num_hidden_layers)]
        self.embed_tokens: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self.final_norm_w: Optional[torch.Tensor] = None
        self.init_parameters()
        self.set_fwd("torch")

    # -- parameters -------------------------------------------------------------------------------------------
    def init_parameters(self):
        a, W, r = self.arch, self.world_size, self.rank
        ckpt = ShardedCheckpoint(self.model_config.checkpoint_dir) if self.model_config.checkpoint_dir else None
        dev, dt = self.device, self.dtype
        if ckpt is None:
            g = torch.Generator(device=dev).manual_seed(self.model_config.seed)   # replicated tensors: same seed
            self.embed_tokens = (torch.randn(a.vocab_size, a.hidden_size, device=dev, generator=g) * 0.02).to(dt)
            self.lm_head = self.embed_tokens if a.tie_word_embeddings else (
                torch.randn(a.vocab_size, a.hidden_size, device=dev, generator=g) * 0.02).to(dt)
            self.final_norm_w = torch.ones(a.hidden_size, device=dev, dtype=dt)
            for i, l in enumerate(self.layers):
                l.eps = a.rms_norm_eps
                l.input_norm_w = torch.ones(a.hidden_size, device=dev, dtype=dt)
                l.post_norm_w = torch.ones(a.hidden_size, device=dev, dtype=dt)
                l.attn.init_random(a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim, a.qk_norm,
                                   a.rope_theta, a.rms_norm_eps, dt, dev, seed=self.model_config.seed + 2 * i)
                l.mlp.init_random(a.hidden_size, a.intermediate_size, dt, dev, seed=self.model_config.seed + 2 * i + 1)
            return
        get = lambda n: ckpt.get(n).to(dev).to(dt)   # noqa: E731
        self.embed_tokens = get("model.embed_tokens.weight")
        self.lm_head = self.embed_tokens if (a.tie_word_embeddings or "lm_head.weight" not in ckpt) else get("lm_head.weight")
        self.final_norm_w = get("model.norm.weight")
        D, Hq, Hkv = a.head_dim, a.num_attention_heads, a.num_key_value_heads
        for i, l in enumerate(self.layers):
            p = f"model.layers.{i}."
            l.eps = a.rms_norm_eps
            l.input_norm_w = get(p + "input_layernorm.weight")
            l.post_norm_w = get(p + "post_attention_layernorm.weight")
            at = l.attn
            at._set_dims(a.hidden_size, Hq, Hkv, D, a.rope_theta, a.rms_norm_eps)
            q = ckpt.get_row_shard(p + "self_attn.q_proj.weight", r, W)
            if Hkv >= W:
                k = ckpt.get_row_shard(p + "self_attn.k_proj.weight", r, W)
                v = ckpt.get_row_shard(p + "self_attn.v_proj.weight", r, W)
            else:
                kvh = r * Hkv // W
                k = ckpt.get(p + "self_attn.k_proj.weight", rows=(kvh * D, (kvh + 1) * D))
                v = ckpt.get(p + "self_attn.v_proj.weight", rows=(kvh * D, (kvh + 1) * D))
            at.wqkv = torch.cat([q, k, v], 0).to(dev).to(dt).contiguous()
            at.wo = ckpt.get_col_shard(p + "self_attn.o_proj.weight", r, W).to(dev).to(dt).contiguous()
            if (p + "self_attn.q_norm.weight") in ckpt:
                at.q_norm_w = get(p + "self_attn.q_norm.weight")
                at.k_norm_w = get(p + "self_attn.k_norm.weight")
            ml = l.mlp
            gate = ckpt.get_row_shard(p + "mlp.gate_proj.weight", r, W)
            up = ckpt.get_row_shard(p + "mlp.up_proj.weight", r, W)
            ml.gate_up_proj = torch.cat([gate, up], 0).to(dev).to(dt).contiguous()
            ml.down_proj = ckpt.get_col_shard(p + "mlp.down_proj.weight", r, W).to(dev).to(dt).contiguous()
            ml.hidden, ml.inter_local = ml.down_proj.shape
        ckpt.close()

    # -- modes ------------------------------------------------------------------------------------------------
    def set_fwd(self, mode: str = "torch"):
        self.mode = mode
        for l in self.layers:
            l.set_fwd(mode)

    def _share_ctx(self, attr_names, src_attn, src_mlp):
        for l in self.layers[1:]:
            for n in attr_names:
                setattr(l.attn, n, getattr(src_attn, n))
                setattr(l.mlp, n, getattr(src_mlp, n))

    def init_triton_dist_ctx(self, max_M: int = 4096):
        """AG-GEMM / GEMM-RS contexts, one set shared by all layers (they run one after the other)."""
        l0 = self.layers[0]
        l0.attn._init_ctx(max_M)
        l0.mlp._init_ctx(max_M)
        self._share_ctx(("ag_ctx", "rs_ctx"), l0.attn, l0.mlp)
        # the batch-sharded hidden state of the last token is gathered with the low-latency packet all-gather
        self.ag_ll_ctx = ops.create_fast_allgather_context(max_ll_bytes=max(64 * 1024, 2 * max_M * self.arch.hidden_size
                                                                            // max(self.world_size, 1)))

    def init_triton_dist_AR_ctx(self, max_M: int = 4096):
        l0 = self.layers[0]
        l0.attn._init_AR_ctx(max_M)
        l0.mlp.ar_ctx = l0.attn.ar_ctx
        self._share_ctx(("ar_ctx",), l0.attn, l0.mlp)

    def init_triton_dist_gemm_ar_ctx(self, max_M: int = 256):
        l0 = self.layers[0]
        l0.attn._init_gemm_ar_ctx(max_M)
        l0.mlp.gemm_ar_ctx = l0.attn.gemm_ar_ctx   # same N = hidden for both row-parallel projections
        self._share_ctx(("gemm_ar_ctx",), l0.attn, l0.mlp)
        # decode steps of up to eight tokens take the fused GEMV path; one scratch set serves every layer
        self.gemv_ctx = ops.create_gemv_ar_context(self.arch.hidden_size)

    def _fused_decode_ok(self, B: int, S: int) -> bool:
        a = self.arch
        return (self.mode in ("triton_dist_gemm_ar", "gemm_ar") and S == 1 and getattr(self, "gemv_ctx", None) is not None
                and self.embed_tokens.is_cuda and self.embed_tokens.dtype == torch.bfloat16
                and B <= ops.GEMV_FAST_M and ops.gemv_supported(B, a.hidden_size)
                and ops.gemv_supported(B, a.intermediate_size // self.world_size)
                and ops.gemv_supported(B, a.num_attention_heads * a.head_dim // self.world_size))

    def init_ctx_for(self, mode: str, max_M: int):
        if mode == "torch":
            return
        if mode in ("triton_dist", "ag_rs"):
            self.init_triton_dist_ctx(max_M)
        elif mode in ("triton_dist_AR", "allreduce"):
            self.init_triton_dist_AR_ctx(max_M)
        else:
            self.init_triton_dist_gemm_ar_ctx(max_M)

    # -- forward ----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def inference(self, input_ids: torch.Tensor, position_ids: torch.Tensor, kv_cache, wo_lm_head: bool = False):
        """input_ids / position_ids [B, S] -> fp32 logits [B, vocab] of the last position (or the last hidden state).
        In the ag_rs mode the batch is sharded over the ranks inside the layers and gathered before the LM head."""
        sharded = self.mode in ("triton_dist", "ag_rs") and self.world_size > 1
        B, S = input_ids.shape
        ids = input_ids
        if sharded:
            assert B % self.world_size == 0, "ag_rs mode shards the batch over the ranks"
            bl = B // self.world_size
            ids = input_ids[self.rank * bl:(self.rank + 1) * bl]
        hidden = ops.embedding(ids, self.embed_tokens)
        kv_cache.begin_step(position_ids, B, S)   # cache rows and kv lengths are the same for every layer
        try:
            return self._layers_and_head(hidden, ids, position_ids, kv_cache, B, S, sharded, wo_lm_head)
        finally:
            kv_cache.end_step()

    def _layers_and_head(self, hidden, ids, position_ids, kv_cache, B, S, sharded, wo_lm_head):
        if self._fused_decode_ok(B, S):
            stream = hidden.reshape(B, -1)
            for l in self.layers:
                l.fwd_fused_decode(stream, position_ids, kv_cache, self.gemv_ctx)
            if wo_lm_head:
                return ops.rmsnorm(stream, self.final_norm_w, self.arch.rms_norm_eps)
            return ops.gemv_fused(stream, self.lm_head, norm_weight=self.final_norm_w, eps=self.arch.rms_norm_eps).float()
        residual = None
        for l in self.layers:
            hidden, residual = l.fwd(hidden, residual, position_ids, kv_cache)
        H = hidden.shape[-1]
        x = ops.rmsnorm(hidden.reshape(-1, H), self.final_norm_w, self.arch.rms_norm_eps, residual=residual)
        x = x.reshape(hidden.shape[0], S, H)[:, -1, :].contiguous()
        if sharded:
            x = ops.all_gather_ll(x, self.ag_ll_ctx).reshape(-1, H) if getattr(self, 'ag_ll_ctx', None) is not None \
                else ops.all_gather(x, None)
        if wo_lm_head:
            return x
        return ops.gemm(x, self.lm_head).float()

    def finalize(self):
        if getattr(self, "gemv_ctx", None) is not None:
            self.gemv_ctx.finalize()
            self.gemv_ctx = None
        l0 = self.layers[0]
        l0.attn.finalize()
        l0.mlp.ar_ctx = None if l0.mlp.ar_ctx is l0.attn.ar_ctx else l0.mlp.ar_ctx
        l0.mlp.gemm_ar_ctx = None
        l0.mlp.finalize()
