"""Single-GPU micro-benchmark of the decode-step kernels at Qwen3-32B per-rank shapes (TP given by --tp):
small-M GEMMs against torch.matmul, split-KV decode attention against its HBM roofline, and the element-wise ops.
Device-timed with CUDA events; weights are rotated over several copies so that nothing stays in L2."""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triton_distributed_b200 import ops  # noqa: E402
from triton_distributed_b200.utils import load_peaks  # noqa: E402


def timeit(fn, iters=10, warmup=3, reps=6):
    """Median device time of one call in microseconds: `reps` calls are captured in a CUDA graph (so that host launch
    cost is excluded, as in the decode engine) and the graph is replayed `iters` times."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3 / reps)
    return statistics.median(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--batches", default="1,16,64")
    ap.add_argument("--ctx", type=int, default=4096)
    args = ap.parse_args()
    tp = args.tp
    H, I, Hq, Hkv, D = 5120, 25600 // tp, 64 // tp, max(1, 8 // tp), 128
    hbm = load_peaks()["hbm_gbs"]
    shapes = {"qkv": ((Hq + 2 * Hkv) * D, H), "o_proj": (H, Hq * D), "gate_up": (2 * I, H), "down": (H, I)}
    ncopy = 6
    for B in [int(b) for b in args.batches.split(",")]:
        for name, (N, K) in shapes.items():
            ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(ncopy)]
            x = torch.randn(B, K, device="cuda", dtype=torch.bfloat16)
            out = torch.empty(B, N, device="cuda", dtype=torch.bfloat16)
            i = [0]

            def own():
                i[0] = (i[0] + 1) % ncopy
                ops.skinny_gemm(x, ws[i[0]], out=out)

            def ref():
                i[0] = (i[0] + 1) % ncopy
                torch.matmul(x, ws[i[0]].t(), out=out)

            t_own, t_ref = timeit(own), timeit(ref)
            ideal = N * K * 2 / (hbm * 1e3)
            rec = {"op": name, "B": B, "N": N, "K": K, "skinny_us": round(t_own, 2), "torch_us": round(t_ref, 2),
                   "hbm_ideal_us": round(ideal, 2), "skinny_frac_of_hbm": round(ideal / t_own, 3)}
            if ops.gemv_supported(B, K):
                def gemv():
                    i[0] = (i[0] + 1) % ncopy
                    ops.gemv_fused(x, ws[i[0]], out=out)

                t_gemv = timeit(gemv)
                rec.update({"gemv_us": round(t_gemv, 2), "gemv_frac_of_hbm": round(ideal / t_gemv, 3)})
            print(json.dumps(rec), flush=True)
            del ws
        # attention
        L = args.ctx
        k = torch.randn(B, L, Hkv, D, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(B, L, Hkv, D, device="cuda", dtype=torch.bfloat16)
        q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
        bt = ops.dense_block_table(B, "cuda")
        lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
        ws_ = ops.decode_workspace(B, Hq, D, 64, "cuda")
        t = timeit(lambda: ops.gqa_fwd_batch_decode(q, k, v, ws_, None, lens, bt))
        ideal = 2 * B * L * Hkv * D * 2 / (hbm * 1e3)
        print(json.dumps({"op": "decode_attn", "B": B, "ctx": L, "own_us": round(t, 2), "hbm_ideal_us": round(ideal, 2),
                          "own_frac_of_hbm": round(ideal / t, 3)}), flush=True)
        # element-wise
        xh = torch.randn(B, H, device="cuda", dtype=torch.bfloat16)
        w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        res = torch.randn(B, H, device="cuda", dtype=torch.bfloat16)
        gu = torch.randn(B, 2 * I, device="cuda", dtype=torch.bfloat16)
        print(json.dumps({"op": "elementwise", "B": B, "rmsnorm_us": round(timeit(lambda: ops.rmsnorm(xh, w, 1e-6, res)), 2),
                          "silu_mul_us": round(timeit(lambda: ops.silu_mul(gu)), 2)}), flush=True)


if __name__ == "__main__":
    main()
