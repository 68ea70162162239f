"""Helpers to run a function on several CPU ranks (gloo) or to launch a torchrun script on several GPUs."""
import os
import socket
import subprocess
import sys
import traceback

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world_size, port, fn, args, err_q):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world_size), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    try:
        import triton_distributed_b200 as tdb

        tdb.initialize_distributed(seed=1234, device="cpu")
        fn(rank, world_size, *args)
        tdb.finalize_distributed()
    except Exception:
        err_q.put((rank, traceback.format_exc()))
        raise


_RENDEZVOUS_ERRORS = ("Address already in use", "EADDRINUSE", "Connection refused", "Connection reset",
                      "failed to connect", "Broken pipe")


def run_cpu_ranks(fn, world_size=2, args=()):
    """Run ``fn(rank, world_size, *args)`` on ``world_size`` gloo ranks; raises if any rank failed.  A failure of the
    rendezvous itself (the free port was taken between probing and binding) is retried once on another port."""
    try:
        _run_cpu_ranks_once(fn, world_size, args)
    except AssertionError as e:
        if not any(m in str(e) for m in _RENDEZVOUS_ERRORS):
            raise
        _run_cpu_ranks_once(fn, world_size, args)


def _run_cpu_ranks_once(fn, world_size, args):
    ctx = mp.get_context("spawn")
    err_q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world_size, port, fn, args, err_q)) for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    errors = []
    while not err_q.empty():
        errors.append(err_q.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            errors.append((-1, "rank did not finish in time"))
        elif p.exitcode != 0 and not errors:
            errors.append((-1, f"exit code {p.exitcode}"))
    if errors:
        raise AssertionError("\n".join(f"[rank {r}] {e}" for r, e in errors))


def run_gpu_script(script, nproc, extra_args=(), timeout=600, env=None):
    """Launch ``tests/multigpu/<script>`` with torchrun on ``nproc`` GPUs; returns its stdout."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "multigpu", script), *extra_args]
    e = dict(os.environ)
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    if env:
        e.update(env)
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e, cwd=ROOT)
    if res.returncode != 0:
        raise AssertionError(f"{script} failed on {nproc} GPUs\nstdout:\n{res.stdout[-6000:]}\nstderr:\n{res.stderr[-6000:]}")
    return res.stdout
