"""Single-GPU GEMM benchmark: tcgen05 kernel of this package vs torch.matmul (cuBLAS), device-timed with CUDA
events, L2 flushed between iterations.  Usage: python benchmarks/bench_gemm.py [--shapes MxNxK,...] [--iters N]."""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triton_distributed_b200.ops import gemm  # noqa: E402
from triton_distributed_b200.utils import L2Flusher, device_time_ms, gemm_roofline  # noqa: E402

DEFAULT = "8192x8192x8192,8192x28672x8192,8192x3584x8192,8192x8192x3584,8192x8192x28672,2048x5120x25600"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default=DEFAULT)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--no-torch", action="store_true")
    args = ap.parse_args()
    fl = L2Flusher()
    for shp in args.shapes.split(","):
        M, N, K = (int(v) for v in shp.split("x"))
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t_own = device_time_ms(lambda: gemm(a, b, out=out, block_n=args.block_n), args.iters, args.warmup, True, fl)
        rec = {"shape": shp, "own_ms_median": statistics.median(t_own), "own_ms_min": min(t_own)}
        rec.update({f"own_{k}": v for k, v in gemm_roofline(M, N, K, statistics.median(t_own)).items()})
        if not args.no_torch:
            bt = b.t()
            t_ref = device_time_ms(lambda: torch.matmul(a, bt, out=out), args.iters, args.warmup, True, fl)
            rec["torch_ms_median"] = statistics.median(t_ref)
            rec["torch_tflops"] = 2.0 * M * N * K / statistics.median(t_ref) / 1e9
            rec["speedup_vs_torch"] = rec["torch_ms_median"] / rec["own_ms_median"]
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
