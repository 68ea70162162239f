"""Serving engine: prefill, switch to the overlapped backend, capture one decode step in a CUDA graph, replay.

API of the reference: ``Engine`` (python/triton_dist/models/engine.py:37-189): attributes ``backend``, ``no_graph``,
``enable_profile`` are set by the caller; ``serve(input_ids, gen_len)`` returns the generated token ids.
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from .. import ops
from ..runtime import get_runtime
from ..utils.misc import logger
from .config import ModelConfig
from .kv_cache import KV_Cache


class Engine:
    def __init__(self, model_config: ModelConfig, temperature: float = 0.0, top_p: float = 1.0, verbose: bool = False,
                 group=None, model=None):
        from . import AutoLLM

        self.rt = get_runtime()
        self.model_config = model_config
        self.temperature, self.top_p, self.verbose = temperature, top_p, verbose
        self.model = model if model is not None else AutoLLM.from_pretrained(model_config, group)
        self.backend = "torch"
        self.no_graph = False
        self.enable_profile = False
        self.kv_cache: Optional[KV_Cache] = None
        self.graph = None
        self.last_decode_ms: Optional[float] = None

    def _init_kv_cache(self, bsz: int):
        a = self.model.arch
        kv_heads = max(1, a.num_key_value_heads // self.rt.world_size)
        self.kv_cache = KV_Cache(a.num_hidden_layers, bsz, self.model_config.max_length, kv_heads, a.head_dim,
                                 self.model_config.dtype, self.rt.device)

    def _decode_step(self):
        pos = self.kv_cache.kv_offset[:self._bsz].to(torch.int64).unsqueeze(1)
        self._logits.copy_(self.model.inference(self._ids, pos, self.kv_cache))

    def _init_cuda_graph(self):
        """Three warm-up steps on a side stream, then capture one whole decode step."""
        off = self.kv_cache.kv_offset.clone()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                self._decode_step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.rt.host_barrier()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._decode_step()
        self.kv_cache.kv_offset.copy_(off)
        torch.cuda.synchronize()
        self.rt.host_barrier()

    @torch.no_grad()
    def serve(self, input_ids: torch.Tensor, gen_len: int) -> torch.Tensor:
        """Prefill ``input_ids`` [B, S] with the torch backend, then generate ``gen_len`` tokens with ``self.backend``."""
        B, S = input_ids.shape
        self._bsz = B
        input_ids = input_ids.to(self.rt.device)
        self._init_kv_cache(B)
        pos = torch.arange(S, device=self.rt.device, dtype=torch.int64).unsqueeze(0).expand(B, S).contiguous()
        self.model.set_fwd("torch")
        logits = self.model.inference(input_ids, pos, self.kv_cache)
        self.kv_cache.inc_offset(S)
        nxt = ops.sample_token(logits, self.temperature, self.top_p)
        out = [nxt]
        # switch backend
        self.model.init_ctx_for(self.backend, max(B, 1))
        self.model.set_fwd(self.backend)
        self._ids = nxt.reshape(B, 1).clone()
        self._logits = torch.empty_like(logits)
        use_graph = (not self.no_graph) and self.rt.is_cuda
        if use_graph:
            self._init_cuda_graph()
        if self.rt.is_cuda:
            torch.cuda.synchronize()
        self.rt.host_barrier()
        t0 = time.perf_counter()
        for _ in range(gen_len - 1):
            if use_graph:
                self.graph.replay()
            else:
                self._decode_step()
            self.kv_cache.inc_offset(1)
            nxt = ops.sample_token(self._logits, self.temperature, self.top_p)
            self._ids.copy_(nxt.reshape(B, 1))
            out.append(nxt.clone())
        if self.rt.is_cuda:
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        self.last_decode_ms = dt * 1e3 / max(gen_len - 1, 1)
        if self.verbose and self.rt.rank == 0:
            logger.info(f"decode: {self.last_decode_ms:.3f} ms/step over {gen_len - 1} steps (backend {self.backend})")
        self.rt.check_status(sync=False)
        return torch.stack(out, dim=1)
