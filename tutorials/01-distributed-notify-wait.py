"""Tutorial 01 - symmetric memory, notify and wait.

    torchrun --nproc-per-node 2 tutorials/01-distributed-notify-wait.py

Every rank owns a queue slot and a flag in the symmetric heap.  Rank r produces a message for rank r+1: it writes the
payload through the peer mapping of the consumer's slot (plain stores over NVLink) and then sets the consumer's flag
to the step number, stream-ordered after the copy.  The consumer's stream waits for the flag before it reads the
slot.  This is the host-side form of the producer / consumer protocol every fused kernel of the library uses
(device side: ``notify`` / ``wait_until`` in ``csrc/include/tdb/symm_device.cuh``).  The reference's version of this
tutorial is tutorials/01-distributed-notify-wait.py (Triton ``dl.notify`` / ``dl.wait``).
"""
import torch
from _common import done, say, start

import triton_distributed_b200 as tdb
from triton_distributed_b200 import language as dl

rt = start()
if not rt.is_cuda or rt.world_size < 2:
    say(rt, "needs at least two GPUs (symmetric memory is device memory); nothing to do here")
    done(rt, "01-notify-wait")
    raise SystemExit(0)

N = 1 << 16
slot = tdb.symm_tensor((N,), torch.float32)        # same offset on every rank
flag = tdb.symm_tensor((1,), torch.int32)
nxt, prv = (rt.rank + 1) % rt.world_size, (rt.rank - 1) % rt.world_size
peer_slot, peer_flag = dl.symm_at(slot, nxt), dl.symm_at(flag, nxt)

for step in range(1, 4):
    msg = torch.full((N,), float(100 * step + rt.rank), device=rt.device)
    peer_slot.copy_(msg)                            # producer: payload into the consumer's memory ...
    dl.notify(peer_flag, step)                      # ... then the flag, ordered after the copy on this stream
    dl.wait(flag, step, geq=True)                   # consumer: the stream stalls until the flag arrives
    got = slot.clone()
    torch.cuda.synchronize()
    assert torch.all(got == 100 * step + prv), (step, got[:4])
    rt.host_barrier()                               # do not overwrite a slot the consumer is still reading
say(rt, "every rank received its predecessor's message three times")
done(rt, "01-notify-wait")
