"""Tutorial 08 - GEMM overlapped with the reduce-scatter of its output.

    torchrun --nproc-per-node 4 tutorials/08-overlapping-gemm-reduce-scatter.py

Row-parallel linear layer: every rank holds a K-slice of the weight and produces a full-size partial result that must
be summed over the ranks and scattered by rows.  ``gemm_rs`` runs ONE kernel: the epilogue of every tile TMA-stores
the partial tile directly into the owner rank's memory and raises a per-tile flag; tiles are visited starting with
the next rank's rows so that the own rows come last, and those are summed with the partials that have arrived by then
straight from the fp32 accumulators.  The baseline is cuBLAS followed by NCCL reduce-scatter.  Reference:
tutorials/08-overlapping-gemm-reduce-scatter.py, kernels/nvidia/gemm_reduce_scatter.py.
"""
import torch
from _common import done, say, start

from triton_distributed_b200 import ops
from triton_distributed_b200.utils import device_time_ms

rt = start()
W = rt.world_size
M, K, N = 8192, 8192, 4096                         # global sizes; K is sharded
a = (torch.randn(M, K // W, device=rt.device) * 0.1).to(torch.bfloat16)
b = (torch.randn(N, K // W, device=rt.device) * 0.05).to(torch.bfloat16)

ctx = ops.create_gemm_rs_context(max_M=M, N=N)
out = ops.gemm_rs(a, b, ctx)
ref = ops.gemm_rs_reference(a, b, rt.group)
err = (out.float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
assert err < 3e-2, err
if rt.is_cuda:
    t_own = min(device_time_ms(lambda: ops.gemm_rs(a, b, ctx), 10, 3))
    t_ref = min(device_time_ms(lambda: ops.gemm_rs_reference(a, b, rt.group), 10, 3))
    say(rt, f"fused {t_own:.3f} ms, cuBLAS + NCCL {t_ref:.3f} ms (this rank, best of 10)")
say(rt, f"GEMM + reduce-scatter matches the reference (rel err {err:.4f})")
ctx.finalize()
done(rt, "08-gemm-rs")
