"""Gated delta rule forward: device time of the chunk-parallel tensor-core kernels and of the token-recurrent kernel for
the reference's test shapes (H heads, K = V = 128,
one sequence of T tokens; python/triton_dist/test/nvidia/test_gdn.py:78-88)."""
import argparse
import json
import os
import statistics
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triton_distributed_b200 import ops  # noqa: E402
from triton_distributed_b200.utils import device_time_ms  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--lens", default="512,2048,8192,32768")
    args = ap.parse_args()
    H, K, V = args.heads, 128, 128
    for T in [int(t) for t in args.lens.split(",")]:
        q = torch.randn(1, T, H, K, device="cuda", dtype=torch.bfloat16)
        k = F.normalize(torch.randn(1, T, H, K, device="cuda"), dim=-1).to(torch.bfloat16)
        v = torch.randn(1, T, H, V, device="cuda", dtype=torch.bfloat16)
        beta = torch.rand(1, T, H, device="cuda").to(torch.bfloat16)
        g = F.logsigmoid(torch.rand(1, T, H, device="cuda"))
        cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
        rec = {"op": "gdn_fwd", "T": T, "H": H}
        for impl in ("chunk", "recurrent"):
            ts = device_time_ms(lambda: ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, K ** -0.5, None, False, cu, impl=impl), 10, 3)
            ms = statistics.median(ts)
            rec[f"{impl}_ms"] = round(ms, 4)
            rec[f"{impl}_us_per_token"] = round(ms * 1e3 / T, 4)
        rec["chunk_speedup"] = round(rec["recurrent_ms"] / rec["chunk_ms"], 2)
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
