"""Launches the multi-GPU check scripts with torchrun when the box has at least two GPUs."""
import pytest
import torch

from dist_utils import run_gpu_script

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_core_two_gpus():
    out = run_gpu_script("check_core.py", 2, ["--quick"])
    assert "ALL OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_core_without_nvls():
    out = run_gpu_script("check_core.py", 2, ["--quick"], env={"TDB200_NVLS": "0", "NCCL_NVLS_ENABLE": "0"})
    assert "ALL OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_model_two_gpus():
    out = run_gpu_script("check_model.py", 2)
    assert "MODEL OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_moe_two_gpus():
    out = run_gpu_script("check_moe.py", 2)
    assert "MOE OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_parallel_two_gpus():
    out = run_gpu_script("check_parallel.py", 2)
    assert "PARALLEL OK" in out
