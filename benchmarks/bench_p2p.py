"""NVLink calibration (torchrun, >= 2 GPUs): bandwidth of pushing / pulling a buffer to / from the next rank with
(a) SM vector ld/st, (b) bulk-TMA ring, (c) the copy engine (cudaMemcpyAsync through Tensor.copy_), per CTA count."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import triton_distributed_b200 as tdb  # noqa: E402
from triton_distributed_b200 import _native  # noqa: E402


def main():
    tdb.initialize_distributed(seed=0)
    rt = tdb.get_runtime()
    lib = _native.load(True)
    nbytes = 256 << 20
    buf = rt.symm_tensor((nbytes,), torch.uint8)
    src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device=rt.device)
    nxt = (rt.rank + 1) % rt.world_size
    peer = rt.peer_view(buf, nxt)
    torch.cuda.synchronize()
    rt.host_barrier()

    def t(fn, iters=5):
        fn()
        torch.cuda.synchronize()
        rt.host_barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        return nbytes * iters / (s.elapsed_time(e) * 1e-3) / 1e9

    res = {}
    for mode, name in ((0, "ldst"), (1, "bulk")):
        for ctas in (1, 4, 8, 16, 32, 64):
            res[f"push_{name}_{ctas}"] = round(t(lambda: lib.p2p_copy(peer, src, ctas, mode)), 1)
            res[f"pull_{name}_{ctas}"] = round(t(lambda: lib.p2p_copy(src, peer, ctas, mode)), 1)
        res[f"local_{name}_8"] = round(t(lambda: lib.p2p_copy(buf, src, 8, mode)), 1)
    res["copy_engine_push"] = round(t(lambda: peer.copy_(src, non_blocking=True)), 1)
    res["copy_engine_pull"] = round(t(lambda: src.copy_(peer, non_blocking=True)), 1)
    if rt.rank == 0:
        print(json.dumps(res), flush=True)
    torch.cuda.synchronize()
    rt.host_barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
