"""Multi-GPU model check (torchrun): every overlapped backend of the dense model against its torch (NCCL + cuBLAS)
backend, with and without CUDA graphs, on a small Qwen3-shaped model."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import triton_distributed_b200 as tdb  # noqa: E402
from triton_distributed_b200.models import ArchConfig, Engine, ModelConfig, PRESETS  # noqa: E402


def main():
    tdb.initialize_distributed(seed=3)
    rt = tdb.get_runtime()
    W = rt.world_size
    PRESETS["check"] = ArchConfig("check", 1024, 2048, 3, 16, 8, 128, 4096)
    cfg = ModelConfig(model_name="check", max_length=256, rank=rt.rank, world_size=W)
    B = 2 * W
    ids = torch.randint(0, 4096, (B, 33), device=rt.device, generator=torch.Generator(device=rt.device).manual_seed(1))
    ref = None
    for backend, graph in [("torch", False), ("triton_dist_AR", True), ("triton_dist_gemm_ar", True),
                           ("triton_dist", False), ("triton_dist", True)]:
        eng = Engine(cfg)
        eng.backend = backend
        eng.no_graph = not graph
        toks = eng.serve(ids, 8)
        torch.cuda.synchronize()
        rt.check_status()
        logits = eng._logits.float().clone()
        if ref is None:
            ref = logits
        err = (logits - ref).abs().max().item()
        tol = 0.15 * ref.abs().max().item() + 0.05
        if rt.rank == 0:
            print(f"backend {backend:22s} graph={graph} max|dlogits|={err:.4f} (tol {tol:.3f}) "
                  f"decode {eng.last_decode_ms:.3f} ms/step", flush=True)
        assert err < tol, backend
        rt.host_barrier()
    if rt.rank == 0:
        print("MODEL OK", flush=True)
    torch.cuda.synchronize()
    rt.host_barrier()
    sys.stdout.flush()
    os._exit(0)   # skip interpreter teardown: nothing left to check, and it must not delay the launcher


if __name__ == "__main__":
    main()
