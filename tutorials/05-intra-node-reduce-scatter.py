"""Tutorial 05 - reduce-scatter inside one NVSwitch domain.

    torchrun --nproc-per-node 4 tutorials/05-intra-node-reduce-scatter.py

``reduce_scatter_2d_op`` sums a [M, N] tensor over the ranks and leaves rank r with rows [r M/W, (r+1) M/W).  On an
NVLS-capable heap one ``multimem.ld_reduce`` per 16 bytes fetches the sum over all ranks from the switch; otherwise
every rank pushes its contribution to the owner and the owner adds.  Reference: tutorials/05-intra-node-reduce-scatter.py,
kernels/nvidia/reduce_scatter.py.
"""
import torch
import torch.distributed as dist
from _common import done, say, start

from triton_distributed_b200 import ops

rt = start()
W = rt.world_size
M, N = 1024 * W, 2048
x = (torch.randn(M, N, device=rt.device) * (rt.rank + 1)).to(torch.bfloat16)
ctx = ops.create_reduce_scater_2d_ctx(M, N)
out = ops.reduce_scatter_2d_op(x, ctx)

ref = torch.empty(M // W, N, dtype=torch.float32, device=rt.device)
dist.reduce_scatter_tensor(ref, x.float(), group=rt.group)
err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
assert err < 2e-2, err
say(rt, f"reduce-scatter of {M}x{N} bf16 matches NCCL (rel err {err:.4f})")
done(rt, "05-reduce-scatter")
