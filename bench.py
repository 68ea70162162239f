"""Headline benchmark: the tensor-parallel MLP GEMM pair of the reference's AG-GEMM / GEMM-RS benchmark,
M=8192 tokens, hidden K=8192, intermediate N=28672, bf16, on N GPUs of one node (strong scaling: the global
problem is fixed, each rank holds 1/N of the weights and of the token rows).

One step =  ag_gemm( A[M/N, K], W1[N/N_gpus, K] ) -> H[M, N/N_gpus]      (all-gather fused into the GEMM launch)
            gemm_rs( H,          W2[K, N/N_gpus]  ) -> O[M/N_gpus, K]     (reduce-scatter fused into the GEMM launch)

Arms:
  --impl ours       this package's fused sm_100a kernels (default)
  --impl torch      all_gather_into_tensor + matmul + matmul + reduce_scatter_tensor (NCCL + cuBLAS), the
                    reference's own golden path (layers/nvidia/tp_mlp.py:231-274); for orientation only
  --impl reference  the unmodified reference from baseline/_ref; it cannot be installed offline (its build
                    needs the patched Triton submodule, which is empty in the mounted checkout), so this arm
                    prints an "unavailable" line

Prints ONE JSON line on rank 0.  Device times come from CUDA events around exactly --steps steps, max over ranks.
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_TOKENS, HIDDEN, INTER = 8192, 8192, 28672


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "torch", "reference"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-e2e-graph", action="store_true", help="end-to-end loop with plain launches instead of CUDA graphs")
    ap.add_argument("--e2e-return", default="metric", choices=["metric", "full"],
                    help="what the host reads back every step: the 4-byte checksum of the output (default), or the "
                         "whole output tensor as well (PCIe-bound at small N: 128 MB per step and direction at N=1)")
    return ap.parse_args()


def reference_unavailable():
    print(json.dumps({"impl": "reference", "unavailable":
                      "pip install of the reference fails offline: python/setup.py needs the patched Triton "
                      "submodule (3rdparty/triton is empty in the mounted checkout) and NVSHMEM"}))
    return 0


def max_over_ranks(v: float, device) -> float:
    t = torch.tensor([v], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    args = parse()
    if args.impl == "reference":
        return reference_unavailable()
    if args.warmup < 3:
        args.warmup = 3

    import triton_distributed_b200 as tdb
    from triton_distributed_b200 import ops
    from triton_distributed_b200.utils import ClockSampler

    tdb.initialize_distributed(seed=0)
    rt = tdb.get_runtime()
    W, rank, dev = rt.world_size, rt.rank, rt.device
    if W != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={W}", file=sys.stderr)
    m, n_loc = M_TOKENS // W, INTER // W
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    a_host = torch.randn(m, HIDDEN, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    a_dev = a_host.to(dev, non_blocking=True)
    w1 = (torch.randn(n_loc, HIDDEN, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(HIDDEN, n_loc, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    h = torch.empty(M_TOKENS, n_loc, device=dev, dtype=torch.bfloat16)
    o = torch.empty(m, HIDDEN, device=dev, dtype=torch.bfloat16)
    launches_per_step = 2

    if args.impl == "ours":
        ag_ctx = ops.create_ag_gemm_context(max_M=M_TOKENS, K=HIDDEN, dtype=torch.bfloat16)
        rs_ctx = ops.create_gemm_rs_context(max_M=M_TOKENS, N=HIDDEN)

        def step(a_in, out=o):
            ops.ag_gemm(a_in, w1, ag_ctx, out=h)
            ops.gemm_rs(h, w2, rs_ctx, out=out)
            return out
    else:
        full = torch.empty(M_TOKENS, HIDDEN, device=dev, dtype=torch.bfloat16)
        part = torch.empty(M_TOKENS, HIDDEN, device=dev, dtype=torch.bfloat16)
        w1t, w2t = w1.t(), w2.t()

        def step(a_in, out=o):
            if W > 1:
                dist.all_gather_into_tensor(full, a_in, group=rt.group)
                torch.matmul(full, w1t, out=h)
                torch.matmul(h, w2t, out=part)
                dist.reduce_scatter_tensor(out, part, group=rt.group)
            else:
                torch.matmul(a_in, w1t, out=h)
                torch.matmul(h, w2t, out=out)
            return out

    def sync_all():
        torch.cuda.synchronize()
        if W > 1:
            dist.barrier(group=rt.group)
        torch.cuda.synchronize()

    # The clock sampler is an nvidia-smi child process: it is started before the warm-up and the timed region only
    # begins once it has delivered its first sample, so its start-up (driver initialisation of the query tool) never
    # overlaps the timed launches.
    sampler = ClockSampler(gpu_index=rt.local_rank).start() if rank == 0 else None
    # ------------------------------------------------------------------ device-timed kernel path
    for _ in range(args.warmup):
        step(a_dev)
    sync_all()
    if sampler is not None:
        sampler.wait_first_sample(5.0)
    sync_all()
    if sampler is not None:
        sampler.begin_window()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(a_dev)
    e1.record()
    sync_all()
    if sampler is not None:
        sampler.end_window()
    ms_total = max_over_ranks(e0.elapsed_time(e1), dev)
    rt.check_status(sync=False)
    ms_per_step = ms_total / args.steps
    flops_per_step = 2 * (2.0 * M_TOKENS * HIDDEN * INTER)
    tflops = flops_per_step / (ms_per_step * 1e-3) / 1e12

    # ------------------------------------------------------------------ end to end: H2D input, public API, D2H result
    # A serving loop: every step's input rows come from pinned host memory, the step runs through the public ops, and
    # the step's result (a 4-byte checksum of the output; with --e2e-return full the whole output too) is copied back
    # and read by the host.  Three streams form a
    # two-deep pipeline: while step i computes, step i+1's input is on its way in and step i-1's output on its way out;
    # the host launches step i and then waits for step i-1's result.  The step (two ops + checksum) is captured once
    # per buffer set in a CUDA graph, as the engine does for decode; --no-e2e-graph keeps plain launches.
    e2e = None
    if not args.no_e2e:
        h2d_stream, d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
        main_stream = torch.cuda.current_stream()
        bufs = [torch.empty_like(a_dev), torch.empty_like(a_dev)]
        outs = [torch.empty_like(o), torch.empty_like(o)]
        outs_host = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for _ in range(2)]
        chk_dev = [torch.zeros(1, dtype=torch.float32, device=dev) for _ in range(2)]
        chk_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
        in_ready = [torch.cuda.Event(), torch.cuda.Event()]     # input of buffer set b has landed
        computed = [torch.cuda.Event(), torch.cuda.Event()]     # the step on buffer set b has finished
        returned = [torch.cuda.Event(), torch.cuda.Event()]     # its output has reached the host

        graphs = [None, None]
        if not args.no_e2e_graph:
            try:
                sync_all()
                for b in range(2):
                    gph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gph):
                        chk_dev[b].zero_()
                        ops.abs_sum(step(bufs[b], outs[b]), chk_dev[b])
                    graphs[b] = gph
                sync_all()
            except Exception as ex:  # capture is an optimisation: fall back to plain launches
                graphs = [None, None]
                if rank == 0:
                    print(f"warning: CUDA graph capture of the step failed ({type(ex).__name__}); using plain launches",
                          file=sys.stderr)
                sync_all()

        def launch(i):
            b = i & 1
            with torch.cuda.stream(h2d_stream):
                h2d_stream.wait_event(computed[b])       # the step that last read this input buffer has finished
                bufs[b].copy_(a_host, non_blocking=True)
                in_ready[b].record(h2d_stream)
            main_stream.wait_event(in_ready[b])
            main_stream.wait_event(returned[b])          # the output buffer's previous contents are on the host
            if graphs[b] is not None:
                graphs[b].replay()
            else:
                chk_dev[b].zero_()
                ops.abs_sum(step(bufs[b], outs[b]), chk_dev[b])
            computed[b].record(main_stream)
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(computed[b])
                if args.e2e_return == "full":
                    outs_host[b].copy_(outs[b], non_blocking=True)
                chk_host[b].copy_(chk_dev[b], non_blocking=True)
                returned[b].record(d2h_stream)

        def collect(i):
            b = i & 1
            returned[b].synchronize()                    # the host reads the step's result
            return float(chk_host[b][0]) + 0.0 * float(outs_host[b][0, 0])

        def run_e2e(nsteps):
            last = 0.0
            for b in range(2):
                computed[b].record(main_stream)
                returned[b].record(d2h_stream)
            for i in range(nsteps):
                launch(i)
                if i > 0:
                    last = collect(i - 1)
            return collect(nsteps - 1) if nsteps > 0 else last

        run_e2e(3)
        sync_all()
        if sampler is not None:
            sampler.begin_window()
        t0 = time.perf_counter()
        chk = run_e2e(args.steps)
        sync_all()
        wall = max_over_ranks(time.perf_counter() - t0, dev)
        if sampler is not None:
            sampler.end_window()
        e2e_ms = wall * 1e3 / args.steps
        e2e = {"value": flops_per_step / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": a_host.numel() * a_host.element_size(),
               "d2h_bytes_per_step": (o.numel() * o.element_size() if args.e2e_return == "full" else 0) + 4,
               "checksum": chk, "cuda_graph": graphs[0] is not None, "pipeline_depth": 2}
    clocks = sampler.stop() if sampler is not None else None

    if rank == 0:
        rec = {
            "metric": "tp_mlp_ag_gemm_gemm_rs_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": W,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours" if args.impl == "ours" else "torch_nccl_cublas",
            "config": {"model": "AG-GEMM + GEMM-RS pair, M=8192 K=8192 N=28672 (Llama-70B-class MLP shapes)",
                       "global_batch": M_TOKENS, "seq_len": 1, "parallelism": f"tp{W}",
                       "l2": "working set per step (weights + activations) exceeds the 126 MB L2 at every N",
                       "weights": "random N(0, 0.02)", "activations": "random N(0, 1)"},
            "us_per_step": ms_per_step * 1e3,
            "tflops_per_gpu": tflops / W,
            "gpu_launches": launches_per_step * args.steps if args.impl == "ours" else 0,
            "clocks": clocks,
        }
        if e2e is not None:
            rec["e2e"] = e2e
        print(json.dumps(rec), flush=True)
    tdb.finalize_distributed()
    return 0


if __name__ == "__main__":
    sys.exit(main())
