"""Tutorial 03 - inter-node all-gather: not applicable.

The reference's tutorial 03 gathers across nodes over InfiniBand with NVSHMEM (tutorials/03-inter-node-allgather.py).
This library targets one NVSwitch domain of up to eight B200s, where every peer is a load / store away; there is no
network transport in it.  Across nodes use NCCL (``torch.distributed.all_gather_into_tensor``) around the intra-node
ops, as this script does when it is launched with more than one node.
"""
import torch
import torch.distributed as dist
from _common import done, say, start

rt = start()
x = torch.full((1024,), float(rt.rank), device=rt.device)
out = torch.empty(rt.world_size * 1024, device=rt.device)
dist.all_gather_into_tensor(out, x, group=rt.group)
assert all(float(out[i * 1024]) == i for i in range(rt.world_size))
say(rt, "NCCL all-gather across the launch; see tutorial 02 for the NVLink kernels")
done(rt, "03-inter-node-allgather")
