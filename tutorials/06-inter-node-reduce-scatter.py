"""Tutorial 06 - inter-node reduce-scatter: not applicable.

The reference's tutorial 06 reduces across nodes over InfiniBand (tutorials/06-inter-node-reduce-scatter.py).  This
library covers one NVSwitch domain; across nodes wrap the intra-node op with NCCL, as here.
"""
import torch
import torch.distributed as dist
from _common import done, say, start

rt = start()
W = rt.world_size
x = torch.ones(W * 256, device=rt.device) * (rt.rank + 1)
out = torch.empty(256, device=rt.device)
dist.reduce_scatter_tensor(out, x, group=rt.group)
assert float(out[0]) == W * (W + 1) / 2
say(rt, "NCCL reduce-scatter across the launch; see tutorial 05 for the NVLink kernels")
done(rt, "06-inter-node-reduce-scatter")
