"""Tutorial 03 - two-level all-gather: device primitives inside a node, a library collective across nodes.

    torchrun --nproc-per-node 4 tutorials/03-inter-node-allgather.py

The reference's tutorial 03 gathers across nodes with NVSHMEM over InfiniBand (tutorials/03-inter-node-allgather.py):
every rank first exchanges with the ranks of its own node over NVLink and then ships whole node blocks over the network,
so that every byte crosses the slow link once.  This library covers one NVSwitch domain, so the launch is split into two
VIRTUAL nodes to show the same composition:

  level 1 (inside a node)   the primitives of this library: a symmetric buffer, peer views (``language.symm_at``), the
                            peer-to-peer copy kernel, stream-ordered signals (``language.notify`` / ``language.wait``);
  level 2 (across nodes)    one NCCL all-gather over the "rail" group of the ranks with the same local index - the role
                            the network transport plays in the reference.

On CPU ranks (gloo) level 1 falls back to a sub-group all-gather; the data movement is the same.
"""
import torch
import torch.distributed as dist
from _common import done, say, start

from triton_distributed_b200 import _native
from triton_distributed_b200 import language as dl
from triton_distributed_b200.ops.common import ref_all_gather

rt = start()
W, rank = rt.world_size, rt.rank
nodes = 2 if (W >= 4 and W % 2 == 0) else 1
local = W // nodes
node, lrank = rank // local, rank % local
node_groups = [dist.new_group(list(range(n * local, (n + 1) * local))) for n in range(nodes)]
rail_groups = [dist.new_group([n * local + i for n in range(nodes)]) for i in range(local)]

rows, cols = 1024, 256
x = (torch.arange(rows * cols, device=rt.device, dtype=torch.float32).reshape(rows, cols) % 97 + rank).to(torch.bfloat16)

# ---- level 1: gather the shards of this node into `node_buf` [local, rows, cols]
if rt.is_cuda and rt.heap is not None:
    lib = _native.load(True)
    node_buf = rt.symm_tensor((local, rows, cols), torch.bfloat16)       # same offset on every rank
    flags = rt.symm_tensor((W,), torch.int32)                            # one arrival flag per source rank
    epoch = 1
    for i in range(local):
        peer = node * local + (lrank + i) % local                        # nearest peer first
        dst = dl.symm_at(node_buf, peer)[lrank]                          # slot [my local rank] in the peer's buffer
        lib.p2p_copy(dst, x, 8, 0)                                       # own copy kernel, plain 16-byte peer stores
        dl.notify(dl.symm_at(flags, peer)[rank:rank + 1], epoch)         # stream-ordered flag write, after the copy
    for i in range(local):
        src = node * local + i
        dl.wait(flags[src:src + 1], epoch, geq=True)                     # bounded wait: a missing peer raises, not hangs
    torch.cuda.synchronize()
    rt.check_status()
else:
    node_buf = ref_all_gather(x, node_groups[node]).reshape(local, rows, cols)

# ---- level 2: ranks with the same local index exchange whole node blocks
block = node_buf.reshape(local * rows, cols).contiguous()
full = ref_all_gather(block, rail_groups[lrank]) if nodes > 1 else block          # [nodes * local * rows, cols]

ref = ref_all_gather(x, rt.group)
assert torch.equal(full.reshape(W * rows, cols), ref)
say(rt, f"two-level all-gather over {nodes} virtual node(s) x {local} rank(s) matches the flat all-gather")
done(rt, "03-inter-node-allgather")
