"""Shared set-up of the tutorials: start the runtime from the torchrun environment and print from rank 0."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import triton_distributed_b200 as tdb  # noqa: E402


def start(seed: int = 0):
    tdb.initialize_distributed(seed=seed)
    return tdb.get_runtime()


def say(rt, *args):
    if rt.rank == 0:
        print(*args, flush=True)


def done(rt, name: str):
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    rt.host_barrier()
    say(rt, f"[{name}] OK on {rt.world_size} rank(s)")
    tdb.finalize_distributed()
