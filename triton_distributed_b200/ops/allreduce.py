"""All-reduce library: one-shot push, two-shot push, NVLS one-shot, NVLS two-shot; auto-selection by size.

API of the reference: ``AllReduceMethod`` (python/triton_dist/kernels/allreduce.py:28-61),
``create_allreduce_ctx`` / ``all_reduce`` / ``get_auto_allreduce_method``
(python/triton_dist/kernels/nvidia/allreduce.py:108, :1129, :1101).  The ring / tree / TMA variants of the
reference collapse on a single NVSwitch domain; their enum members are kept and map onto the four kernels.
CPU / reference path: ``torch.distributed.all_reduce``.
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from .common import new_ctx_dev, ref_all_reduce, sm_count
from ..tools.autotuner import current_config
from ..utils.oplog import logged_op

MAX_CTAS = 64


class AllReduceMethod(enum.Enum):
    Unknown = 0
    OneShot = 1
    TwoShot = 2
    DoubleTree = 3            # served by TwoShot here (no tree on a full-bandwidth switch)
    OneShot_TMA = 4           # served by OneShot
    OneShot_Multimem = 5
    TwoShot_Multimem = 6
    TwoShot_Multimem_ST = 7   # served by TwoShot_Multimem (it already broadcasts with multimem.st)
    OneShot_LL = 8            # served by OneShot
    TwoShot_LL = 9            # served by TwoShot


_KERNEL_METHOD = {
    AllReduceMethod.OneShot: 0, AllReduceMethod.OneShot_TMA: 0, AllReduceMethod.OneShot_LL: 0,
    AllReduceMethod.TwoShot: 1, AllReduceMethod.DoubleTree: 1, AllReduceMethod.TwoShot_LL: 1,
    AllReduceMethod.OneShot_Multimem: 2,
    AllReduceMethod.TwoShot_Multimem: 3, AllReduceMethod.TwoShot_Multimem_ST: 3,
}


@dataclass
class AllReduceContext:
    rt: Runtime
    workspace_nbytes: int
    rank: int
    world_size: int
    workspace: Optional[torch.Tensor] = None   # heap, uint8 [2 * half]
    flags: Optional[torch.Tensor] = None       # heap [2][2][W][MAX_CTAS]
    ctx_dev: Optional[torch.Tensor] = None
    calls: int = 0

    def chunk_bytes(self, method: AllReduceMethod) -> int:
        """Largest message one launch can take with this workspace."""
        half = self.workspace_nbytes // 2
        k = _KERNEL_METHOD[method]
        if k == 0:
            b = half // self.world_size
        elif k == 2:
            b = half
        else:
            b = half // 2
        return max(16, b // (16 * self.world_size) * (16 * self.world_size))

    def finalize(self):
        if self.workspace is not None:
            self.rt.symm_free(self.workspace)
            self.rt.symm_free(self.flags)
            self.workspace = None


def create_allreduce_ctx(workspace_nbytes: int, rank: Optional[int] = None, world_size: Optional[int] = None,
                         local_world_size: Optional[int] = None) -> AllReduceContext:
    """Allocate the symmetric workspace (collective call)."""
    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    world_size = rt.world_size if world_size is None else world_size
    workspace_nbytes = max(int(workspace_nbytes), 64 * 1024)
    workspace_nbytes = (workspace_nbytes + 511) // 512 * 512
    ctx = AllReduceContext(rt=rt, workspace_nbytes=workspace_nbytes, rank=rank, world_size=world_size)
    if rt.is_cuda and world_size > 1:
        ctx.workspace = rt.symm_tensor((workspace_nbytes,), torch.uint8, zero=False)
        ctx.flags = rt.symm_tensor((2, 2, world_size, MAX_CTAS), torch.int32)
        ctx.ctx_dev = new_ctx_dev(rt)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def get_auto_allreduce_method(nbytes: int, has_multicast: Optional[bool] = None) -> AllReduceMethod:
    """Size thresholds: NVLS one-shot for latency-bound sizes, NVLS two-shot for bandwidth-bound ones;
    without NVLS the push variants with the same split (reference thresholds: allreduce.py:1101-1126)."""
    if has_multicast is None:
        try:
            has_multicast = get_runtime().has_multicast
        except RuntimeError:
            has_multicast = False
    if has_multicast:
        return AllReduceMethod.OneShot_Multimem if nbytes <= 256 * 1024 else AllReduceMethod.TwoShot_Multimem
    return AllReduceMethod.OneShot if nbytes <= 128 * 1024 else AllReduceMethod.TwoShot


def _ctas_for(nbytes: int, device) -> int:
    # ~32 KB per CTA, at least 1, at most MAX_CTAS: small messages stay latency-optimal
    return int(max(1, min(MAX_CTAS, nbytes // (32 * 1024))))


def _ar_meta(x, *args, **kw):
    return {"shape": {"numel": x.numel(), "dtype": str(x.dtype)}, "bytes": x.numel() * x.element_size()}


@logged_op("all_reduce", _ar_meta)
def all_reduce(x: torch.Tensor, method: Optional[AllReduceMethod] = None, ctx: Optional[AllReduceContext] = None,
               output: Optional[torch.Tensor] = None, max_sm: int = -1,
               straggler_option: Optional[Tuple[int, float]] = None) -> torch.Tensor:
    """Sum ``x`` over all ranks.  Messages larger than the workspace are processed in chunks."""
    rt = get_runtime() if ctx is None else ctx.rt
    if straggler_option is not None and straggler_option[0] == rt.rank:
        time.sleep(float(straggler_option[1]))
    if (not _native.use_native(x)) or rt.world_size == 1 or x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        res = ref_all_reduce(x, rt.group)
        if output is not None:
            output.copy_(res)
            return output
        return res
    if ctx is None:
        raise ValueError("all_reduce on GPU tensors needs a context from create_allreduce_ctx")
    lib = _native.load(True)
    x = x.contiguous()
    if output is None:
        output = torch.empty_like(x)
    nbytes = x.numel() * x.element_size()
    if method is None or method == AllReduceMethod.Unknown:
        tuned = current_config().get("allreduce_method")       # a method the contextual autotuner is trying / chose
        method = AllReduceMethod[tuned] if isinstance(tuned, str) else get_auto_allreduce_method(nbytes, rt.has_multicast)
    if _KERNEL_METHOD[method] >= 2 and not rt.has_multicast:
        method = AllReduceMethod.OneShot if _KERNEL_METHOD[method] == 2 else AllReduceMethod.TwoShot
    k = _KERNEL_METHOD[method]
    xin = x.view(-1).view(torch.uint8)
    xout = output.view(-1).view(torch.uint8)
    pad = (-nbytes) % 16
    if pad:
        # rare: pad to 16 bytes through a staging copy
        xin = torch.cat([xin, torch.zeros(pad, dtype=torch.uint8, device=x.device)])
        xout_full = torch.empty_like(xin)
    else:
        xout_full = xout
    total = xin.numel()
    chunk = ctx.chunk_bytes(method)
    off = 0
    while off < total:
        n = min(chunk, total - off)
        ctas = _ctas_for(n, x.device)
        if max_sm > 0:
            ctas = min(ctas, max_sm)
        lib.all_reduce(rt.heap, xin[off:off + n].view(x.dtype), xout_full[off:off + n].view(x.dtype), ctx.workspace,
                       ctx.flags, ctx.ctx_dev, k, False, MAX_CTAS, ctas, rt.config.wait_timeout_s)
        off += n
        ctx.calls += 1
    if pad:
        xout.copy_(xout_full[:nbytes])
    return output
