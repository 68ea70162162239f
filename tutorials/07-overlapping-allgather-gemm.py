"""Tutorial 07 - all-gather overlapped with the GEMM that consumes it.

    torchrun --nproc-per-node 4 tutorials/07-overlapping-allgather-gemm.py

Column-parallel linear layer: the activations are sharded by rows, the weight by output columns.  ``ag_gemm`` runs
ONE kernel: a few CTAs push the local shard into every peer's workspace (bulk-TMA copies over NVLink, one flag per
128-row chunk) while the other CTAs run the tcgen05 GEMM, starting with the local rows and waiting per tile for
exactly the chunk it needs.  The baseline is NCCL all-gather followed by cuBLAS.  Reference:
tutorials/07-overlapping-allgather-gemm.py, kernels/nvidia/allgather_gemm.py.
"""
import torch
from _common import done, say, start

from triton_distributed_b200 import ops
from triton_distributed_b200.utils import device_time_ms

rt = start()
W = rt.world_size
M, K, N = 8192, 4096, 8192                         # global sizes
a = torch.randn(M // W, K, device=rt.device).to(torch.bfloat16)
b = (torch.randn(N // W, K, device=rt.device) * 0.02).to(torch.bfloat16)

ctx = ops.create_ag_gemm_context(max_M=M, K=K, dtype=torch.bfloat16)
out = ops.ag_gemm(a, b, ctx)
ref = ops.ag_gemm_reference(a, b, rt.group)
err = (out.float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
assert err < 2e-2, err
if rt.is_cuda:
    t_own = min(device_time_ms(lambda: ops.ag_gemm(a, b, ctx), 10, 3))
    t_ref = min(device_time_ms(lambda: ops.ag_gemm_reference(a, b, rt.group), 10, 3))
    say(rt, f"fused {t_own:.3f} ms, NCCL + cuBLAS {t_ref:.3f} ms (this rank, best of 10)")
say(rt, f"all-gather + GEMM matches the reference (rel err {err:.4f})")
ctx.finalize()
done(rt, "07-ag-gemm")
