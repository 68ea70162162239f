"""Small, self-terminating workloads for Nsight Compute captures of single kernels (one GPU, a few launches).

  python benchmarks/ncu_case.py gemm      # tcgen05 GEMM 8192 x 4096 x 4096 (inputs + output ~160 MB > L2)
  python benchmarks/ncu_case.py skinny    # decode GEMM 32 x 5120 x 3200, split-K
  python benchmarks/ncu_case.py decode    # split-KV decode attention, 16 seqs x 4096 tokens, 8 q heads / 1 kv head
  python benchmarks/ncu_case.py gemv      # decode GEMV 1 x 6400 x 5120 (65 MB of weights per launch, 4 weight copies)
  python benchmarks/ncu_case.py gemm_fp8  # block-scaled e4m3 GEMM 8192 x 3584 x 8192 (pair kernel, ~150 MB)
  python benchmarks/ncu_case.py moe       # grouped GEMM with in-kernel row gather: 8192 tokens, top-2 of 16 experts, 2048 x 2048
  python benchmarks/ncu_case.py gdn       # chunk-parallel gated delta rule, 8192 tokens x 16 heads
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
    elif case == "gemm_fp8":
        a = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
        b = (torch.randn(3584, 8192, device="cuda") * 0.02).to(torch.bfloat16)
        a_q, a_s = ops.quantize_act_1x128(a)
        b_q, b_s = ops.quantize_weight_128x128(b)
        for _ in range(3):
            ops.gemm_fp8_blockscaled(a_q, a_s, b_q, b_s)
    elif case == "moe":
        T, E, k, H, N = 8192, 16, 2, 2048, 2048
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = (torch.randn(E, N, H, device="cuda") * 0.02).to(torch.bfloat16)
        ids = torch.randint(0, E, (T, k), device="cuda", dtype=torch.int32)
        srt = ops.sort_topk_ids_align_block_size(ids, E)
        for _ in range(3):
            ops.group_gemm_gather(x, w, srt, k)
    elif case == "gdn":
        import torch.nn.functional as F
        T, H, K, V = 8192, 16, 128, 128
        q = torch.randn(1, T, H, K, device="cuda", dtype=torch.bfloat16)
        kk = F.normalize(torch.randn(1, T, H, K, device="cuda"), dim=-1).to(torch.bfloat16)
        v = torch.randn(1, T, H, V, device="cuda", dtype=torch.bfloat16)
        beta = torch.rand(1, T, H, device="cuda").to(torch.bfloat16)
        g = F.logsigmoid(torch.rand(1, T, H, device="cuda"))
        for _ in range(2):
            ops.chunk_gated_delta_rule_fwd(q, kk, v, g, beta, K ** -0.5, impl="chunk")
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
