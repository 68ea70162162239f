"""Distributed flash-decode latency: one query token per sequence, KV sharded over the ranks, Qwen3-32B head shapes
(64 query / 8 KV heads, head dim 128, bf16), global context 32 k / 128 k / 1 M tokens.

  torchrun --nproc-per-node N benchmarks/bench_flash_decode.py [--ctx 32768,131072,1048576] [--batch 1] [--iters 30]

Arms, all device-timed with CUDA events around a CUDA graph of several calls (max over ranks; the calls rotate over
KV-cache copies that together exceed L2, so nothing is re-read from L2):
  fused      SpGQAFlashDecodeAttention, one launch (split-KV + packet exchange + LSE merge)
  two_launch the same layer with the exchange + merge as a second launch
  nccl       own split-KV kernel with LSE output, then NCCL all-gather of (out, LSE) and a PyTorch merge
             (what a library-collective implementation does)
Also printed: local KV bytes / time as a fraction of the measured HBM copy bandwidth.  With N = 1 the script times the
local split-KV step on the shard an 8-rank job would hold (`--emulate-world 8`), which bounds the multi-rank number
from below.  The reference's published curve: 58 us at 128 k and 300 us at 1 M on 8 x H800 (README.md:200-202).
"""
import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import triton_distributed_b200 as tdb  # noqa: E402
from triton_distributed_b200.ops.attention import gqa_fwd_batch_decode, merge_attention_partials  # noqa: E402
from triton_distributed_b200.parallel import SpGQAFlashDecodeAttention  # noqa: E402
from triton_distributed_b200.utils import load_peaks  # noqa: E402


def timed_us(fns, iters, warmup, rt):
    """Median device time of one call in microseconds, max over ranks.  ``fns`` are equivalent calls on different copies
    of the KV cache (together larger than L2, so no call finds its KV in L2); two rounds over them are captured in one
    CUDA graph, which is how a decode loop issues the step, and the graph is replayed ``iters`` times."""
    for _ in range(warmup):
        for fn in fns:
            fn()
    torch.cuda.synchronize()
    if rt.world_size > 1:
        dist.barrier(group=rt.group)
    g = torch.cuda.CUDAGraph()
    reps = 2 * len(fns)
    with torch.cuda.graph(g):
        for _ in range(2):
            for fn in fns:
                fn()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if rt.world_size > 1:
            dist.barrier(group=rt.group)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3 / reps)
    t = torch.tensor(ts, device="cuda", dtype=torch.float64)
    if rt.world_size > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.group)
    return statistics.median(t.tolist())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctx", default="32768,131072,1048576", help="global context lengths")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--hq", type=int, default=64)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--page", type=int, default=64)
    ap.add_argument("--emulate-world", type=int, default=8, help="with one GPU: shard size of a job of this many ranks")
    args = ap.parse_args()
    tdb.initialize_distributed(seed=0)
    rt = tdb.get_runtime()
    W, dev = rt.world_size, rt.device
    B, Hq, Hkv, D, page = args.batch, args.hq, args.hkv, 128, args.page
    shard_world = W if W > 1 else args.emulate_world
    hbm = load_peaks()["hbm_gbs"]
    layer = SpGQAFlashDecodeAttention(rt.rank, 0, W, 1, Hq, Hkv, D, D, page_size=page, max_allowed_batch=B)
    for ctx in [int(c) for c in args.ctx.split(",")]:
        local = (ctx + shard_world - 1) // shard_world
        pages_per_seq = (local + page - 1) // page
        kv_bytes = 2 * B * local * Hkv * D * 2
        copies = int(max(1, min(8, -(-(300 << 20) // kv_bytes))))       # > 2 x L2 in total
        caches = [(torch.randn(B * pages_per_seq, page, Hkv, D, device=dev, dtype=torch.bfloat16),
                   torch.randn(B * pages_per_seq, page, Hkv, D, device=dev, dtype=torch.bfloat16)) for _ in range(copies)]
        bt = torch.arange(B * pages_per_seq, dtype=torch.int32, device=dev).reshape(B, pages_per_seq)
        q = torch.randn(B, Hq, D, device=dev, dtype=torch.bfloat16)
        lens = torch.full((W, B), local, dtype=torch.int32, device=dev)
        local_lens = lens[rt.rank].contiguous()
        rec = {"op": "dist_flash_decode", "world": W, "global_ctx": ctx, "kv_per_rank": local, "batch": B, "hq": Hq,
               "hkv": Hkv, "kv_mb_per_rank": round(kv_bytes / 2 ** 20, 1), "hbm_floor_us": round(kv_bytes / (hbm * 1e3), 1),
               "timing": f"CUDA graph of {2 * copies} calls over {copies} KV copies"}
        if W > 1:
            for name, one in (("fused", True), ("two_launch", False)):
                layer.one_launch = one
                t = timed_us([(lambda kc=kc, vc=vc: layer.forward(q, kc, vc, lens, bt)) for kc, vc in caches],
                             args.iters, args.warmup, rt)
                rt.check_status()
                rec[f"{name}_us"] = round(t, 1)
                rec[f"{name}_launches"] = int(layer.last_launches)
            gathered_o = torch.empty(W, B, Hq, D, device=dev, dtype=torch.float32)
            gathered_l = torch.empty(W, B, Hq, device=dev, dtype=torch.float32)

            def nccl_arm(kc, vc):
                o, lse = gqa_fwd_batch_decode(q, kc, vc, None, None, local_lens, bt, return_lse=True)
                dist.all_gather_into_tensor(gathered_o, o.float().contiguous(), group=rt.group)
                dist.all_gather_into_tensor(gathered_l, lse.contiguous(), group=rt.group)
                return merge_attention_partials(gathered_o, gathered_l)

            rec["nccl_us"] = round(timed_us([(lambda kc=kc, vc=vc: nccl_arm(kc, vc)) for kc, vc in caches], args.iters,
                                            args.warmup, rt), 1)
            rec["fused_vs_nccl"] = round(rec["nccl_us"] / rec["fused_us"], 2)
            rec["frac_of_hbm"] = round(rec["hbm_floor_us"] / rec["fused_us"], 3)
        else:
            t = timed_us([(lambda kc=kc, vc=vc: gqa_fwd_batch_decode(q, kc, vc, None, None, local_lens, bt)) for kc, vc in caches],
                         args.iters, args.warmup, rt)
            rec["local_splitkv_us"] = round(t, 1)
            rec["frac_of_hbm"] = round(rec["hbm_floor_us"] / t, 3)
            rec["note"] = f"one GPU: local step on the shard of a {shard_world}-rank job"
        if rt.rank == 0:
            print(json.dumps(rec), flush=True)
        del caches
        torch.cuda.empty_cache()
    tdb.finalize_distributed()


if __name__ == "__main__":
    main()
