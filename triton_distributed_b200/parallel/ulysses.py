"""Ulysses sequence parallelism: QKV projection -> sequence-to-head all-to-all, and head-to-sequence all-to-all -> O
projection.

API of the reference: ``SpUlysessQKVGemmAll2AllKernel`` (kernels/nvidia/sp_ulysess_qkv_gemm_all2all.py:447-844,
``forward`` / ``pre_attn_a2a``) and ``SpUlysessOAll2AllGemmKernel`` (sp_ulysess_o_all2all_gemm.py:395-703,
``forward`` / ``post_attn_a2a``).

QKV side (GPU): the exchange happens in the GEMM epilogue.  The weight rows are regrouped once per weight so that the
heads of destination rank d are contiguous ([q heads of d | k heads of d | v heads of d]); the projection then runs as
one tcgen05 GEMM per destination whose output tensor IS the destination's receive buffer: every finished tile is
TMA-stored straight into peer memory at row offset ``rank * s_local``, there is no local QKV tensor, no permute and no
separate exchange kernel.  A rank barrier before the GEMMs (peers have finished reading the previous result) and one
after them (all blocks have landed) are the only synchronisation.  Destinations are visited starting with the next
rank, the own block last.

O side (GPU): ``a2a_cols_kernel`` (csrc/ep_a2a.cu) pushes, for every destination, this rank's head block of the
attention output into the column block ``[rank * hl * D, ...)`` of the destination's ``[s_local, heads * D]`` GEMM input
(entry announcement per rank, arrival flags per source), then the O projection runs on the assembled rows.

Variable-length batches: ``seq_lens_cpu`` (one entry per sequence, each divisible by the world size) only changes the
number of local rows; both directions work on the packed ``[sum(len) / W, ...]`` layout the reference uses.
CPU / single rank: the same data movement through ``all_to_all_single_2d``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import _native, ops
from ..ops.common import new_ctx_dev
from ..runtime import get_runtime


def _local_rows(seq_lens_cpu: Optional[List[int]], world: int, fallback: int) -> int:
    if seq_lens_cpu is None:
        return fallback
    lens = [int(x) for x in seq_lens_cpu]
    if any(n % world for n in lens):
        raise ValueError("ulysses: every sequence length must be divisible by the sequence-parallel size")
    return sum(n // world for n in lens)


class SpUlysessQKVGemmAll2AllKernel:
    def __init__(self, world_group=None, nnodes: int = 1, sp_size: Optional[int] = None, max_batch_size: int = 1,
                 num_head: int = 32, max_seqlen: int = 4096, head_dim: int = 128, max_num_comm_buf: int = 1,
                 input_dtype: torch.dtype = torch.bfloat16, output_dtype: torch.dtype = torch.bfloat16, **kw):
        rt = get_runtime()
        self.rt = rt
        self.W = rt.world_size if sp_size is None else sp_size
        self.num_head, self.head_dim = num_head, head_dim
        self.hl = num_head // self.W
        self.max_rows = max_batch_size * max_seqlen             # gathered rows (all positions)
        self.dtype = output_dtype
        self.a2a_ctx = ops.create_all_to_all_single_2d_context(self.max_rows, 3 * self.hl * head_dim, output_dtype)
        self.recv = None
        self._w_cache: Dict[Tuple[int, int], torch.Tensor] = {}
        if rt.is_cuda and self.W > 1:
            self.recv = rt.symm_tensor((self.max_rows, 3 * self.hl * head_dim), output_dtype, zero=False)

    # ------------------------------------------------------------------ weight layout
    def _dest_major_weight(self, weight: torch.Tensor) -> torch.Tensor:
        """[3 * heads * D, H] -> [W, 3 * hl * D, H] with the q, k and v rows of destination d's heads contiguous.  Built once
        per weight tensor (keyed by storage address and version)."""
        key = (weight.data_ptr(), weight._version)
        w = self._w_cache.get(key)
        if w is None:
            H = weight.shape[1]
            w = (weight.reshape(3, self.W, self.hl * self.head_dim, H).permute(1, 0, 2, 3)
                 .reshape(self.W, 3 * self.hl * self.head_dim, H).contiguous())
            self._w_cache = {key: w}
        return w

    # ------------------------------------------------------------------ exchange only
    def pre_attn_a2a(self, qkv_local: torch.Tensor, seq_lens_cpu: Optional[List[int]] = None) -> torch.Tensor:
        """[s_local, 3, heads, D] on every rank -> [s_local * W, 3, heads / W, D] (all positions, this rank's heads)."""
        W = self.W
        s_local = _local_rows(seq_lens_cpu, W, qkv_local.shape[0])
        hl = self.hl
        if W == 1:
            return qkv_local
        # destination-major rows: block d holds this rank's positions restricted to rank d's heads
        x = qkv_local.reshape(s_local, 3, W, hl, self.head_dim).permute(2, 0, 1, 3, 4).contiguous()
        x = x.reshape(W * s_local, 3 * hl * self.head_dim)
        y = ops.all_to_all_single_2d(self.a2a_ctx, x, [s_local] * W, [s_local] * W)
        return y.reshape(W * s_local, 3, hl, self.head_dim)

    # ------------------------------------------------------------------ projection + exchange
    def forward(self, inputs: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                seq_lens_cpu: Optional[List[int]] = None) -> torch.Tensor:
        """inputs [s_local, H], weight [3 * heads * D, H] -> [S, 3, heads / W, D]."""
        W, rt = self.W, self.rt
        s_local = _local_rows(seq_lens_cpu, W, inputs.shape[0])
        if s_local != inputs.shape[0]:
            raise ValueError("ulysses: inputs do not match seq_lens_cpu")
        fused = (W > 1 and self.recv is not None and bias is None and _native.use_native(inputs, weight)
                 and inputs.dtype == torch.bfloat16 and W * s_local <= self.max_rows)
        if not fused:
            qkv = ops.gemm(inputs, weight)
            if bias is not None:
                qkv = qkv + bias
            return self.pre_attn_a2a(qkv.reshape(inputs.shape[0], 3, self.num_head, self.head_dim), seq_lens_cpu)
        wd = self._dest_major_weight(weight)
        x = inputs.contiguous()
        rt.barrier_all_on_stream()                  # every peer is done with the previous contents of its buffer
        for i in range(1, W + 1):
            d = (rt.rank + i) % W
            dst = rt.peer_view(self.recv, d)[rt.rank * s_local:(rt.rank + 1) * s_local]
            ops.gemm(x, wd[d], out=dst)             # the epilogue's TMA stores land in rank d's memory
        rt.barrier_all_on_stream()                  # all blocks of all ranks have landed
        return self.recv[:W * s_local].view(W * s_local, 3, self.hl, self.head_dim)

    qkv_pack_a2a = pre_attn_a2a


class SpUlysessOAll2AllGemmKernel:
    def __init__(self, world_group=None, nnodes: int = 1, sp_size: Optional[int] = None, max_batch_size: int = 1,
                 num_head: int = 32, max_seqlen: int = 4096, head_dim: int = 128, input_dtype: torch.dtype = torch.bfloat16,
                 output_dtype: torch.dtype = torch.bfloat16, **kw):
        rt = get_runtime()
        self.rt = rt
        self.W = rt.world_size if sp_size is None else sp_size
        self.num_head, self.head_dim = num_head, head_dim
        self.hl = num_head // self.W
        self.max_rows = max_batch_size * max_seqlen
        self.a2a_ctx = ops.create_all_to_all_single_2d_context(self.max_rows, self.hl * head_dim, output_dtype)
        self.gathered = None
        if rt.is_cuda and self.W > 1:
            max_local = (self.max_rows + self.W - 1) // self.W
            self.gathered = rt.symm_tensor((max_local, num_head * head_dim), input_dtype, zero=False)
            self.flags = rt.symm_tensor((2, 8), torch.int32)
            self.ctx_dev = new_ctx_dev(rt)
            torch.cuda.synchronize()
            rt.host_barrier()

    def post_attn_a2a(self, attn_out: torch.Tensor, seq_lens_cpu: Optional[List[int]] = None) -> torch.Tensor:
        """[S, heads / W, D] (all positions, local heads) -> [s_local, heads, D] (local positions, all heads)."""
        W = self.W
        if W == 1:
            return attn_out
        S = attn_out.shape[0]
        s_local = _local_rows(seq_lens_cpu, W, S // W)
        hl = self.hl
        x = attn_out.reshape(S, hl * self.head_dim)
        if (self.gathered is not None and _native.use_native(x) and x.dtype == self.gathered.dtype and x.stride(1) == 1
                and (hl * self.head_dim * x.element_size()) % 16 == 0 and s_local <= self.gathered.shape[0]):
            lib = _native.load(True)
            lib.a2a_cols(self.rt.heap, x, self.gathered, s_local, self.flags, self.ctx_dev, 8,
                         self.rt.config.wait_timeout_s)
            return self.gathered[:s_local].view(s_local, self.num_head, self.head_dim)
        x = x.contiguous()                                              # rows already ordered by destination rank
        y = ops.all_to_all_single_2d(self.a2a_ctx, x, [s_local] * W, [s_local] * W)   # [W(src heads), s_local, hl*D]
        return y.reshape(W, s_local, hl, self.head_dim).permute(1, 0, 2, 3).reshape(s_local, self.num_head, self.head_dim)

    def forward(self, inputs: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                seq_lens_cpu: Optional[List[int]] = None) -> torch.Tensor:
        """inputs [S, heads / W, D], weight [H, heads * D] -> [s_local, H]."""
        x = self.post_attn_a2a(inputs, seq_lens_cpu)
        out = ops.gemm(x.reshape(x.shape[0], -1), weight)
        if bias is not None:
            out = out + bias
        return out
