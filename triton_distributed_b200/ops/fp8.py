"""Block-scaled fp8 (e4m3) operands for the tensor-parallel GEMMs: 1 x 128 scales for activations, 128 x 128 scales
for weights (the DeepSeek-V3 recipe the reference's EP path uses for its payloads,
python/triton_dist/kernels/nvidia/low_latency_all_to_all.py:36-118, tutorials/04-deepseek-infer-all2all.py:185-215:
``scale = amax / 448`` per group of 128).

GPU path: ``csrc/gemm_fp8_sm100.cu`` - ``tcgen05.mma.kind::f8f6f4`` on CTA pairs, one fresh TMEM accumulator per
128-wide K block, promoted with ``a_s[m, kb] * b_s[n / 128, kb]`` into register accumulators by eight epilogue warps
while the tensor core works on the next block.  ``ag_gemm_fp8`` / ``gemm_rs_fp8`` are the same launch with the
all-gather (fp8 rows + scales pushed by comm CTAs, half the NVLink bytes of the bf16 op) or the reduce-scatter (bf16
partial tiles stored into the owner's slot, own segment summed in the epilogue) fused in; no torch or NCCL call is on
that path.  CPU tensors (and the ``*_reference`` functions) use the plain PyTorch restatement with the same
accumulation order, which is the oracle of the GPU tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from .common import new_ctx_dev, ref_all_gather, ref_reduce_scatter, sm_count

BLOCK = 128
FP8_MAX = 448.0


def _fp8_dtype():
    return torch.float8_e4m3fn


def quantize_act_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x`` [M, K] -> (fp8 [M, K], fp32 scales [M, K / 128]); K must be a multiple of 128."""
    M, K = x.shape
    assert K % BLOCK == 0, "K must be a multiple of 128"
    if _native.use_native(x) and x.dtype == torch.bfloat16 and x.is_contiguous():
        q, scale = _native.load(True).fp8_quant(x)      # own kernel: one warp per row, amax / 448 per 128 values
        return q, scale
    xb = x.float().reshape(M, K // BLOCK, BLOCK)
    scale = xb.abs().amax(-1).clamp_min(1e-10) / FP8_MAX
    q = (xb / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).to(_fp8_dtype())
    return q.reshape(M, K), scale


def quantize_weight_128x128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w`` [N, K] -> (fp8 [N, K], fp32 scales [ceil(N / 128), K / 128])."""
    N, K = w.shape
    assert K % BLOCK == 0, "K must be a multiple of 128"
    nb = (N + BLOCK - 1) // BLOCK
    wp = torch.zeros(nb * BLOCK, K, dtype=torch.float32, device=w.device)
    wp[:N] = w.float()
    wb = wp.reshape(nb, BLOCK, K // BLOCK, BLOCK)
    scale = wb.abs().amax(dim=(1, 3)).clamp_min(1e-10) / FP8_MAX
    q = (wb / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(_fp8_dtype())
    return q.reshape(nb * BLOCK, K)[:N].contiguous(), scale


def dequantize_act_1x128(q: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    M, K = q.shape
    return (q.float().reshape(M, K // BLOCK, BLOCK) * scale[..., None]).reshape(M, K).to(dtype)


def dequantize_weight_128x128(q: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    N, K = q.shape
    nb = scale.shape[0]
    qp = torch.zeros(nb * BLOCK, K, dtype=torch.float32, device=q.device)
    qp[:N] = q.float()
    w = qp.reshape(nb, BLOCK, K // BLOCK, BLOCK) * scale[:, None, :, None]
    return w.reshape(nb * BLOCK, K)[:N].to(dtype)


def gemm_fp8_blockscaled_reference(a_q, a_s, b_q, b_s) -> torch.Tensor:
    """fp32 reference with the accumulation order of a block-scaled kernel: one partial product per 128-wide K
    block, scaled by ``a_s[m, kb] * b_s[n / 128, kb]`` and summed in fp32."""
    M, K = a_q.shape
    N = b_q.shape[0]
    kb = K // BLOCK
    a = a_q.float().reshape(M, kb, BLOCK)
    b = b_q.float().reshape(N, kb, BLOCK)
    part = torch.einsum("mkc,nkc->kmn", a, b)                               # [kb, M, N]
    bs = b_s.repeat_interleave(BLOCK, dim=0)[:N]                            # [N, kb]
    return (part * a_s.t()[:, :, None] * bs.t()[:, None, :]).sum(0)


def _native_ok(*ts) -> bool:
    return _native.use_native(*ts)


def gemm_fp8_blockscaled(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor,
                         out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, num_ctas: int = 0,
                         stats: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``(a_q, a_s)`` [M, K] with 1 x 128 scales times ``(b_q, b_s)`` [N, K] with 128 x 128 scales -> [M, N].
    CUDA tensors run the native fp8 kernel (bf16 output); CPU tensors the PyTorch restatement."""
    if _native_ok(a_q, a_s, b_q, b_s) and out_dtype == torch.bfloat16:
        lib = _native.load(True)
        if out is None:
            out = torch.empty((a_q.shape[0], b_q.shape[0]), dtype=torch.bfloat16, device=a_q.device)
        lib.gemm_fp8(a_q, a_s.contiguous(), b_q, b_s.contiguous(), out, num_ctas, stats)
        return out
    res = gemm_fp8_blockscaled_reference(a_q, a_s, b_q, b_s).to(out_dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


@dataclass
class AGGemmFp8Context:
    rt: Runtime
    max_M: int
    K: int
    n_comm_ctas: int = 0
    workspace: Optional[torch.Tensor] = None      # heap uint8 [2][max_M][K]
    ws_scales: Optional[torch.Tensor] = None      # heap fp32 [2][max_M][K/128]
    flags: Optional[torch.Tensor] = None          # heap int32 [2][W][max_chunks]
    ctx_dev: Optional[torch.Tensor] = None
    max_chunks: int = 0
    stats: Optional[torch.Tensor] = None

    @property
    def max_seg_rows(self) -> int:
        return self.max_M // self.rt.world_size

    def finalize(self):
        for n in ("workspace", "ws_scales", "flags"):
            t = getattr(self, n)
            if t is not None:
                self.rt.symm_free(t)
                setattr(self, n, None)


def create_ag_gemm_fp8_context(max_M: int, K: int, n_comm_ctas: int = 0) -> AGGemmFp8Context:
    """Symmetric workspace for the gathered fp8 rows and their scales (collective call)."""
    rt = get_runtime()
    W = rt.world_size
    max_M = (max_M + W - 1) // W * W
    ctx = AGGemmFp8Context(rt=rt, max_M=max_M, K=K, n_comm_ctas=n_comm_ctas)
    if rt.is_cuda and W > 1:
        ctx.max_chunks = (ctx.max_seg_rows + 127) // 128
        ctx.workspace = rt.symm_tensor((2, max_M, K), torch.uint8, zero=False, sync=False)
        ctx.ws_scales = rt.symm_tensor((2, max_M, K // BLOCK), torch.float32, zero=False, sync=False)
        ctx.flags = rt.symm_tensor((2, W, ctx.max_chunks), torch.int32, sync=False)
        ctx.ctx_dev = new_ctx_dev(rt)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def ag_gemm_fp8_reference(a_q, a_s, b_q, b_s, group=None) -> torch.Tensor:
    """All-gather of the fp8 rows and scales with torch.distributed, then the block-scaled reference product."""
    a_all = ref_all_gather(a_q.view(torch.uint8), group).view(_fp8_dtype())
    s_all = ref_all_gather(a_s, group)
    return gemm_fp8_blockscaled_reference(a_all, s_all, b_q, b_s)


def ag_gemm_fp8(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor,
                ctx: Optional[AGGemmFp8Context] = None, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a_q`` [M / W, K] row shard with scales [M / W, K / 128], ``b_q`` [N / W, K] column-parallel weight with scales
    -> [M, N / W] bf16.  On GPUs the all-gather of rows and scales runs inside the GEMM launch."""
    if not _native_ok(a_q, a_s, b_q, b_s):
        res = ag_gemm_fp8_reference(a_q, a_s, b_q, b_s, group).to(torch.bfloat16)
        if out is not None:
            out.copy_(res)
            return out
        return res
    rt = get_runtime()
    W = rt.world_size
    if W == 1:
        return gemm_fp8_blockscaled(a_q, a_s, b_q, b_s, out=out)
    if ctx is None:
        raise ValueError("ag_gemm_fp8 on GPUs needs a context from create_ag_gemm_fp8_context")
    lib = _native.load(True)
    m, K = a_q.shape
    N = b_q.shape[0]
    if out is None:
        out = torch.empty((m * W, N), dtype=torch.bfloat16, device=a_q.device)
    n_sms = sm_count(a_q.device)
    from .ag_gemm import pick_comm_ctas
    # half the bytes per row of the bf16 op, twice the tensor rate: same bytes-per-GEMM-time ratio
    n_comm = ctx.n_comm_ctas or pick_comm_ctas(m, N, W, 256, n_sms, True, K)
    n_comm = max(2, min(n_comm + (n_comm & 1), n_sms - 2))
    lib.ag_gemm_fp8(rt.heap, a_q.contiguous(), a_s.contiguous(), b_q, b_s.contiguous(), out, ctx.workspace, ctx.ws_scales,
                    ctx.flags, ctx.ctx_dev, ctx.max_seg_rows, ctx.max_chunks, n_comm, n_sms, rt.config.wait_timeout_s,
                    ctx.stats)
    return out


@dataclass
class GemmRSFp8Context:
    rt: Runtime
    max_M: int
    N: int
    slots: Optional[torch.Tensor] = None     # heap bf16 [2][W][max_M/W][N]
    flags: Optional[torch.Tensor] = None     # heap int32 [2][W][max_tiles]
    ctx_dev: Optional[torch.Tensor] = None
    max_tiles: int = 0
    stats: Optional[torch.Tensor] = None

    @property
    def max_seg_rows(self) -> int:
        return self.max_M // self.rt.world_size

    def finalize(self):
        for n in ("slots", "flags"):
            t = getattr(self, n)
            if t is not None:
                self.rt.symm_free(t)
                setattr(self, n, None)


def create_gemm_rs_fp8_context(max_M: int, N: int) -> GemmRSFp8Context:
    rt = get_runtime()
    W = rt.world_size
    max_M = (max_M + W - 1) // W * W
    ctx = GemmRSFp8Context(rt=rt, max_M=max_M, N=N)
    if rt.is_cuda and W > 1:
        seg = ctx.max_seg_rows
        ctx.max_tiles = ((seg + 127) // 128) * ((N + 127) // 128)
        ctx.slots = rt.symm_tensor((2, W, seg, N), torch.bfloat16, zero=False, sync=False)
        ctx.flags = rt.symm_tensor((2, W, ctx.max_tiles), torch.int32, sync=False)
        ctx.ctx_dev = new_ctx_dev(rt)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def gemm_rs_fp8_reference(a_q, a_s, b_q, b_s, group=None) -> torch.Tensor:
    return ref_reduce_scatter(gemm_fp8_blockscaled_reference(a_q, a_s, b_q, b_s), group)


def gemm_rs_fp8(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor,
                ctx: Optional[GemmRSFp8Context] = None, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a_q`` [M, K / W] with scales [M, K / W / 128], ``b_q`` [N, K / W] row-parallel weight with scales ->
    this rank's [M / W, N] bf16 block of the sum over ranks; the reduce-scatter runs inside the GEMM launch."""
    if not _native_ok(a_q, a_s, b_q, b_s):
        res = gemm_rs_fp8_reference(a_q, a_s, b_q, b_s, group).to(torch.bfloat16)
        if out is not None:
            out.copy_(res)
            return out
        return res
    rt = get_runtime()
    W = rt.world_size
    if W == 1:
        return gemm_fp8_blockscaled(a_q, a_s, b_q, b_s, out=out)
    if ctx is None:
        raise ValueError("gemm_rs_fp8 on GPUs needs a context from create_gemm_rs_fp8_context")
    lib = _native.load(True)
    M, N = a_q.shape[0], b_q.shape[0]
    if N != ctx.N:
        raise ValueError(f"gemm_rs_fp8: N={N} differs from the context's N={ctx.N}")
    if out is None:
        out = torch.empty((M // W, N), dtype=torch.bfloat16, device=a_q.device)
    lib.gemm_rs_fp8(rt.heap, a_q, a_s.contiguous(), b_q, b_s.contiguous(), out, ctx.slots, ctx.flags, ctx.ctx_dev,
                    ctx.max_seg_rows, ctx.max_tiles, sm_count(a_q.device), rt.config.wait_timeout_s, ctx.stats)
    return out
