"""Tutorial 06 - two-level reduce-scatter: a library collective across nodes, this library's kernels inside a node.

    torchrun --nproc-per-node 4 tutorials/06-inter-node-reduce-scatter.py

The reference's tutorial 06 reduces across nodes over InfiniBand and inside a node over NVLink
(tutorials/06-inter-node-reduce-scatter.py): the input of every rank is cut into one piece per destination; pieces
first meet the pieces of the SAME destination index from the other nodes (network step), then the node-local
reduce-scatter finishes the sum.  With the launch split into two VIRTUAL nodes:

  level 1 (across nodes)   ranks with the same local index reduce-scatter over their "rail" group (NCCL), each keeping
                           the half of the destinations that live in its own node;
  level 2 (inside a node)  the remaining sum over the node's ranks: every rank pushes the piece of destination d into
                           slot [my local rank] of d's symmetric buffer with the peer-to-peer copy kernel, signals,
                           and the owner adds its slots (``ops.ring_reduce``, the reduction used by GEMM -> RS).

On CPU ranks (gloo) level 2 falls back to a sub-group reduce-scatter.
"""
import torch
import torch.distributed as dist
from _common import done, say, start

from triton_distributed_b200 import _native, ops
from triton_distributed_b200 import language as dl
from triton_distributed_b200.ops.common import ref_reduce_scatter

rt = start()
W, rank = rt.world_size, rt.rank
nodes = 2 if (W >= 4 and W % 2 == 0) else 1
local = W // nodes
node, lrank = rank // local, rank % local
node_groups = [dist.new_group(list(range(n * local, (n + 1) * local))) for n in range(nodes)]
rail_groups = [dist.new_group([n * local + i for n in range(nodes)]) for i in range(local)]

rows, cols = 256, 128                                   # rows of the output piece of one destination
g = torch.Generator(device=rt.device).manual_seed(100 + rank)
x = torch.randn(W, rows, cols, device=rt.device, generator=g)           # piece [d] is meant for rank d

# ---- level 1: across nodes.  After it this rank holds, for every destination of ITS node, the sum over the ranks of
# its rail (one per node).
if nodes > 1:
    # rows of the rail's reduce-scatter = node index: this rank keeps the block of its own node
    mine = ref_reduce_scatter(x.reshape(nodes, local * rows * cols), rail_groups[lrank]).reshape(local, rows, cols)
else:
    mine = x.clone()

# ---- level 2: inside the node
if rt.is_cuda and rt.heap is not None:
    lib = _native.load(True)
    slots = rt.symm_tensor((local, rows, cols), torch.float32)           # slot [source local rank]
    flags = rt.symm_tensor((W,), torch.int32)
    epoch = 1
    for i in range(local):
        dl_rank = (lrank + i) % local
        peer = node * local + dl_rank
        lib.p2p_copy(dl.symm_at(slots, peer)[lrank], mine[dl_rank].contiguous(), 8, 0)
        dl.notify(dl.symm_at(flags, peer)[rank:rank + 1], epoch)
    for i in range(local):
        dl.wait(flags[node * local + i:node * local + i + 1], epoch, geq=True)
    out = ops.ring_reduce(slots)                                         # sum of the slots
    torch.cuda.synchronize()
    rt.check_status()
else:
    out = ref_reduce_scatter(mine.reshape(local, rows * cols), node_groups[node]).reshape(rows, cols)

ref = ref_reduce_scatter(x.reshape(W, rows * cols), rt.group).reshape(rows, cols)
torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
say(rt, f"two-level reduce-scatter over {nodes} virtual node(s) x {local} rank(s) matches the flat reduce-scatter")
done(rt, "06-inter-node-reduce-scatter")
