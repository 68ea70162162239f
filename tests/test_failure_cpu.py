"""Failure detection on the host: a rank that leaves between steps makes the survivors' next collective fail with an
error within the process-group timeout instead of hanging, and the watchdog reports a failed device wait taken from a
fake status page.  No GPU is involved and nothing is made to fault."""
import os
import time
import traceback

import torch.multiprocessing as mp

from dist_utils import free_port


def _rank(rank, world, port, q):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port), "TDB200_PG_TIMEOUT_S": "5"})
    try:
        import torch
        import torch.distributed as dist

        import triton_distributed_b200 as tdb

        tdb.initialize_distributed(seed=0, device="cpu")
        rt = tdb.get_runtime()
        x = torch.ones(4)
        dist.all_reduce(x, group=rt.group)                 # step 1: everybody is there
        assert float(x[0]) == world
        rt.host_barrier()
        if rank == 1:
            q.put((rank, "left"))                          # leaves between steps, nothing in flight
            os._exit(0)
        t0 = time.time()
        try:
            y = torch.ones(4)
            dist.all_reduce(y, group=rt.group)             # step 2: the peer is gone
            q.put((rank, "no error"))
        except Exception as e:  # noqa: BLE001 - any backend error is the detection
            q.put((rank, f"detected after {time.time() - t0:.1f}s: {type(e).__name__}"))
        os._exit(0)
    except Exception:
        q.put((rank, "crash: " + traceback.format_exc()))
        os._exit(1)


def test_survivor_detects_a_rank_that_left():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    msgs = {}
    while not q.empty():
        r, m = q.get()
        msgs[r] = m
    assert not alive, f"a rank hung instead of failing: {msgs}"
    assert msgs.get(1) == "left"
    assert msgs.get(0, "").startswith("detected"), msgs


class _FakeHeap:
    def __init__(self):
        self.record = {"code": 0}

    def read_status(self):
        return self.record


class _FakeRuntime:
    def __init__(self):
        self.heap = _FakeHeap()

    def read_status(self):
        return dict(self.heap.read_status())


def test_watchdog_reports_a_failed_wait_from_the_status_page():
    from triton_distributed_b200.runtime import Watchdog

    rt = _FakeRuntime()
    seen = []
    wd = Watchdog(rt, on_error=seen.append, period_s=0.01).start()
    time.sleep(0.05)
    assert not seen
    rt.heap.record = {"code": 1, "kernel": 3, "where": 2, "peer": 1, "index": 7, "expected": 5, "observed": 4}
    for _ in range(100):
        if seen:
            break
        time.sleep(0.01)
    wd.stop()
    assert seen and seen[0]["kernel"] == 3 and wd.last_record["peer"] == 1
