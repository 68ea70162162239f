"""The tutorials run as CPU ranks (gloo) through the ops' reference paths: keeps their API use from rotting."""
import os
import subprocess
import sys

import pytest

from dist_utils import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name,nproc", [("02-intra-node-allgather.py", 2), ("04-deepseek-infer-all2all.py", 2),
                                        ("05-intra-node-reduce-scatter.py", 2), ("03-inter-node-allgather.py", 4),
                                        ("06-inter-node-reduce-scatter.py", 4)])
def test_tutorial_runs_on_cpu_ranks(name, nproc):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tutorials", name)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert f"OK on {nproc} rank(s)" in res.stdout
