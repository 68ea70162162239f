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
                 group=None, model=None, seed: int = 0):
        from . import AutoLLM

        self.rt = get_runtime()
        self.model_config = model_config
        self.temperature, self.top_p, self.verbose = temperature, top_p, verbose
        self.model = model if model is not None else AutoLLM.from_pretrained(model_config, group)
        self.backend = "torch"
        self.no_graph = False
        self.enable_profile = False     # True: torch.profiler over the first 64 decode steps (written under profile_dir)
        self.profile_dir = "prof"
        self.kv_cache: Optional[KV_Cache] = None
        self.graph = None
        self.last_decode_ms: Optional[float] = None
        self.last_profile: Optional[str] = None
        self.keep_logits = False          # True: serve() keeps the fp32 logits of every generated position in step_logits
        self.step_logits: list = []
        # Sampling state: one generator with the SAME seed on every rank (the process-wide generator is seeded per
        # rank), and rank 0's pick is broadcast, so all ranks feed the same token into the next step.
        self._sample_gen = torch.Generator(device=self.rt.device)
        self._sample_gen.manual_seed(int(seed))
        self._ctx_key = None      # (backend, max_M) the model's communication contexts were built for

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

    def validate_request(self, input_ids: torch.Tensor, gen_len: int):
        """Host-side check of a request against the model's limits; raises ``ValueError``.  Cache rows are addressed as
        ``batch * max_length + position``, so a prompt plus generation longer than ``max_length`` (or a token id outside
        the vocabulary) would index past the sequence's rows: such requests never reach a kernel."""
        if input_ids.dim() != 2 or input_ids.shape[0] < 1 or input_ids.shape[1] < 1:
            raise ValueError(f"input_ids must be a non-empty [batch, seq] tensor, got shape {tuple(input_ids.shape)}")
        if input_ids.dtype not in (torch.int32, torch.int64):
            raise ValueError(f"input_ids must hold integer token ids, got {input_ids.dtype}")
        gen_len = int(gen_len)
        if gen_len < 1:
            raise ValueError(f"gen_len must be at least 1, got {gen_len}")
        B, S = input_ids.shape
        max_len = int(self.model_config.max_length)
        if S + gen_len > max_len:
            raise ValueError(f"prompt ({S}) + gen_len ({gen_len}) exceeds max_length ({max_len})")
        vocab = int(self.model.arch.vocab_size)
        lo, hi = int(input_ids.min()), int(input_ids.max())
        if lo < 0 or hi >= vocab:
            raise ValueError(f"token ids must lie in [0, {vocab}), got [{lo}, {hi}]")
        if self.backend in ("triton_dist", "ag_rs") and B % max(self.rt.world_size, 1) != 0:
            raise ValueError(f"backend {self.backend} shards the batch: {B} is not a multiple of {self.rt.world_size}")

    def _sample(self, logits: torch.Tensor) -> torch.Tensor:
        nxt = ops.sample_token(logits, self.temperature, self.top_p, generator=self._sample_gen)
        if self.temperature > 0.0 and self.rt.world_size > 1:
            import torch.distributed as dist
            nxt = nxt.contiguous()
            dist.broadcast(nxt, src=0, group=self.rt.group)
        return nxt

    def _ensure_ctx(self, max_M: int):
        """Communication contexts are built once per (backend, capacity) and reused by later ``serve`` calls; a change
        of backend or a larger batch releases the old symmetric-heap buffers first."""
        key = (self.backend, max_M)
        if self._ctx_key is not None and self._ctx_key[0] == key[0] and self._ctx_key[1] >= key[1]:
            return
        if self._ctx_key is not None and hasattr(self.model, "finalize"):
            if self.rt.is_cuda:
                torch.cuda.synchronize()
            self.rt.host_barrier()
            self.model.finalize()
        self.model.init_ctx_for(self.backend, max_M)
        self._ctx_key = key

    @torch.no_grad()
    def serve(self, input_ids: torch.Tensor, gen_len: int) -> torch.Tensor:
        """Prefill ``input_ids`` [B, S] with the torch backend, then generate ``gen_len`` tokens with ``self.backend``.
        Requests that do not fit the model (see :meth:`validate_request`) raise ``ValueError`` before any launch."""
        self.validate_request(input_ids, gen_len)
        B, S = input_ids.shape
        self._bsz = B
        input_ids = input_ids.to(self.rt.device)
        if self.kv_cache is None or self.kv_cache.batch_size != B:
            self._init_kv_cache(B)
            self.graph = None
        else:
            self.kv_cache.clear()
        pos = torch.arange(S, device=self.rt.device, dtype=torch.int64).unsqueeze(0).expand(B, S).contiguous()
        self.model.set_fwd("torch")
        logits = self.model.inference(input_ids, pos, self.kv_cache)
        self.kv_cache.inc_offset(S)
        nxt = self._sample(logits)
        out = [nxt]
        self.step_logits = [logits.float().clone()] if self.keep_logits else []
        # switch backend
        self._ensure_ctx(max(B, 1))
        self.model.set_fwd(self.backend)
        self._ids = nxt.reshape(B, 1).clone()
        self._logits = torch.empty_like(logits)
        use_graph = (not self.no_graph) and self.rt.is_cuda
        if use_graph:
            self._init_cuda_graph()
        if self.rt.is_cuda:
            torch.cuda.synchronize()
        self.rt.host_barrier()
        def one_step():
            if use_graph:
                self.graph.replay()
            else:
                self._decode_step()
            self.kv_cache.inc_offset(1)
            if self.keep_logits:
                self.step_logits.append(self._logits.float().clone())
            nxt = self._sample(self._logits)
            self._ids.copy_(nxt.reshape(B, 1))
            out.append(nxt.clone())

        n_steps = gen_len - 1
        n_prof = min(n_steps, 64) if self.enable_profile else 0
        t0 = time.perf_counter()
        if n_prof:
            # the first (at most 64) decode steps run under torch.profiler; rank 0 writes the merged trace of all ranks
            from ..utils.profile import group_profile
            name = f"decode_{self.backend}"
            with group_profile(name, True, group=self.rt.cpu_group, out_dir=self.profile_dir):
                for _ in range(n_prof):
                    one_step()
            self.last_profile = f"{self.profile_dir}/{name}.json.tar.gz"
            t0 = time.perf_counter()
        for _ in range(n_steps - n_prof):
            one_step()
        if self.rt.is_cuda:
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        n_timed = max(n_steps - n_prof, 1)
        self.last_decode_ms = dt * 1e3 / n_timed
        if self.verbose and self.rt.rank == 0:
            logger.info(f"decode: {self.last_decode_ms:.3f} ms/step over {n_timed} steps (backend {self.backend})")
        self.rt.check_status(sync=False)
        return torch.stack(out, dim=1)
