"""Prefill attention: the tcgen05 kernel (S and PV in TMEM, KV packed by a first launch) against the mma.sync kernel and
against torch SDPA, one GPU, causal, GQA 8 query heads per KV head, head dim 128, bf16.  Device-timed with CUDA events.

  python benchmarks/bench_prefill_attn.py [--lens 2048,8192,32768] [--hq 8 --hkv 1]

FLOPs counted: 4 * S^2 * D * Hq / 2 (causal).  The Qwen3-32B TP8 shard has 8 query heads and 1 KV head per rank."""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triton_distributed_b200 import ops  # noqa: E402
from triton_distributed_b200.ops.attention import check_attention_errors  # noqa: E402
from triton_distributed_b200.utils import device_time_ms  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--lens", default="2048,8192,32768")
    ap.add_argument("--hq", type=int, default=8)
    ap.add_argument("--hkv", type=int, default=1)
    args = ap.parse_args()
    Hq, Hkv, D = args.hq, args.hkv, 128
    for S in [int(x) for x in args.lens.split(",")]:
        q = torch.randn(S, Hq, D, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(1, S, Hkv, D, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(1, S, Hkv, D, device="cuda", dtype=torch.bfloat16)
        bt = ops.dense_block_table(1, "cuda")
        cu = torch.tensor([0, S], dtype=torch.int32, device="cuda")
        lens = torch.tensor([S], dtype=torch.int32, device="cuda")
        flops = 4.0 * S * S * D * Hq / 2
        rec = {"op": "prefill_attention", "S": S, "hq": Hq, "hkv": Hkv}
        for impl in ("sm100", "mma"):
            ms = statistics.median(device_time_ms(
                lambda: ops.flash_attn_varlen(q, k, v, bt, cu, lens, S, causal=True, max_kv_len=S, impl=impl), 8, 3))
            rec[f"{impl}_ms"] = round(ms, 4)
            rec[f"{impl}_tflops"] = round(flops / ms / 1e9, 1)
        check_attention_errors()
        qs = q.transpose(0, 1).unsqueeze(0)
        ks = k[0].transpose(0, 1).unsqueeze(0)
        vs = v[0].transpose(0, 1).unsqueeze(0)
        ms = statistics.median(device_time_ms(
            lambda: torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True, enable_gqa=True), 8, 3))
        rec["torch_sdpa_ms"] = round(ms, 4)
        rec["torch_sdpa_tflops"] = round(flops / ms / 1e9, 1)
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
