"""Small, self-terminating workloads for Nsight Compute captures of single kernels (one GPU, a few launches).

  python benchmarks/ncu_case.py gemm      # tcgen05 GEMM 8192 x 4096 x 4096 (inputs + output ~160 MB > L2)
  python benchmarks/ncu_case.py skinny    # decode GEMM 32 x 5120 x 3200, split-K
  python benchmarks/ncu_case.py decode    # split-KV decode attention, 16 seqs x 4096 tokens, 8 q heads / 1 kv head
  python benchmarks/ncu_case.py gemv      # decode GEMV 1 x 6400 x 5120 (65 MB of weights per launch, 4 weight copies)
"""
import sys

import torch

sys.path.insert(0, __import__("os").path.dirname(__import__("os").path.dirname(__import__("os").path.abspath(__file__))))

from triton_distributed_b200 import ops  # noqa: E402


def main():
    case = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    if case == "gemm":
        a = torch.randn(8192, 4096, device="cuda", dtype=torch.bfloat16)
        b = (torch.randn(4096, 4096, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(8192, 4096, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            ops.gemm(a, b, out=out)
    elif case == "skinny":
        a = torch.randn(32, 3200, device="cuda", dtype=torch.bfloat16)
        b = (torch.randn(5120, 3200, device="cuda") * 0.02).to(torch.bfloat16)
        for _ in range(3):
            ops.skinny_gemm(a, b)
    elif case == "gemv":
        ws = [(torch.randn(6400, 5120, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(4)]
        x = torch.randn(1, 5120, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(1, 6400, device="cuda", dtype=torch.bfloat16)
        for w in ws:
            ops.gemv_fused(x, w, out=out)
    elif case == "decode":
        B, Hq, Hkv, D, L = 16, 8, 1, 128, 4096
        k = torch.randn(B, L, Hkv, D, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(B, L, Hkv, D, device="cuda", dtype=torch.bfloat16)
        q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
        bt = ops.dense_block_table(B, "cuda")
        lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
        for _ in range(3):
            ops.gqa_fwd_batch_decode(q, k, v, None, None, lens, bt)
    torch.cuda.synchronize()
    print("done", case)


if __name__ == "__main__":
    main()
