"""Tutorial 02 - all-gather inside one NVSwitch domain.

    torchrun --nproc-per-node 4 tutorials/02-intra-node-allgather.py

Three ways to the same result: the kernel all-gather on a symmetric buffer (push over NVLink, NVLS ``multimem.st``
when the heap has a multicast mapping, or pull), the low-latency packet all-gather for small messages (data and flag
travel in the same 8-byte word, one launch, no separate signal), and NCCL as the golden.  The reference builds the
same from copy-engine pushes and its LL protocol (tutorials/02-intra-node-allgather.py,
kernels/nvidia/low_latency_allgather.py).
"""
import torch
import torch.distributed as dist
from _common import done, say, start

from triton_distributed_b200 import ops

rt = start()
W = rt.world_size
x = torch.randn(4096, 512, device=rt.device).to(torch.bfloat16) + rt.rank

ref = torch.empty(W * 4096, 512, dtype=x.dtype, device=rt.device)
dist.all_gather_into_tensor(ref, x, group=rt.group)

ctx = ops.create_fast_allgather_context(max_ll_bytes=1 << 20)
out = ops.all_gather(x, ctx)                        # throughput path (method picked from the message size)
assert torch.equal(out.reshape(ref.shape), ref)

small = x[:8].contiguous()                          # 8 KB: latency matters, use the packet protocol
out_ll = ops.all_gather_ll(small, ctx)
ref_small = torch.empty(W * 8, 512, dtype=x.dtype, device=rt.device)
dist.all_gather_into_tensor(ref_small, small, group=rt.group)
assert torch.equal(out_ll.reshape(ref_small.shape), ref_small)
say(rt, f"all-gather of {x.numel() * 2 >> 10} KB and of {small.numel() * 2 >> 10} KB per rank match NCCL")
ctx.finalize()
done(rt, "02-allgather")
