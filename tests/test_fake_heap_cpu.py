"""Flag protocols of the fused kernels (epoch flags, parity buffers, no resets, bounded waits) among CPU ranks on a
shared-memory stand-in for the symmetric heap."""
import os

import pytest
import torch

from dist_utils import run_cpu_ranks


def _heap(rank, world, tag, nbytes=8 << 20):
    import torch.distributed as dist
    from triton_distributed_b200.runtime.fake_heap import FakeSymmHeap

    name = f"tdbfh_{tag}_{os.environ['MASTER_PORT']}"
    return FakeSymmHeap(name, rank, world, nbytes, barrier=dist.barrier)


def _ag_calls(rank, world):
    from triton_distributed_b200.runtime import fake_heap as fh

    heap = _heap(rank, world, "ag")
    rows, cols = 300, 16                     # three chunks, the last one ragged
    st = fh.create_ag_push_state(heap, rows, cols, chunk_rows=128)
    try:
        for call in range(5):
            # NaN in the half this call does not use: a read of the wrong parity or of a stale chunk shows up
            fh.poison_unused_parity(st.workspace, st.calls)
            shard = torch.full((rows, cols), float(100 * call + rank)) + torch.arange(rows).float()[:, None]
            seen = []
            full = fh.ag_push_protocol(st, shard, consume=lambda seg, c, x: seen.append((seg, c, float(x[0, 0]))),
                                       delay_s=0.05 if (call % world) == rank else 0.0)     # a different straggler per call
            for r in range(world):
                exp = torch.full((rows, cols), float(100 * call + r)) + torch.arange(rows).float()[:, None]
                assert torch.equal(full[r * rows:(r + 1) * rows], exp), (call, r)
            assert [s[0] for s in seen[:3]] == [rank] * 3                        # local segment first
            assert all(v == 100 * call + seg + 128 * c for seg, c, v in seen)    # chunks of THIS call
        assert int(st.flags.max()) == 5                                           # flags hold epochs, never reset
    finally:
        heap.close()


def _rs_calls(rank, world):
    from triton_distributed_b200.runtime import fake_heap as fh

    heap = _heap(rank, world, "rs")
    rows, cols = 200, 8
    st = fh.create_rs_scatter_state(heap, rows, cols, tile_rows=128)
    try:
        for call in range(4):
            fh.poison_unused_parity(st.slots, st.calls)
            parts = [torch.randn(world * rows, cols, generator=torch.Generator().manual_seed(17 * call + r)) for r in range(world)]
            out = fh.rs_scatter_protocol(st, parts[rank])
            ref = sum(parts)[rank * rows:(rank + 1) * rows]
            torch.testing.assert_close(out, ref, rtol=1e-6, atol=1e-6)
    finally:
        heap.close()


def _missing_rank(rank, world):
    """Rank 1 never pushes: rank 0's wait runs out and reports which peer and chunk it was waiting for."""
    from triton_distributed_b200.runtime import fake_heap as fh

    heap = _heap(rank, world, "miss")
    st = fh.create_ag_push_state(heap, 128, 4, chunk_rows=128)
    try:
        if rank == 0:
            with pytest.raises(fh.FakeWaitTimeout) as ei:
                fh.ag_push_protocol(st, torch.ones(128, 4), timeout_s=0.3)
            rec = ei.value.record
            assert rec["code"] == 1 and rec["peer"] == 1 and rec["index"] == 0 and rec["expected"] == 1 and rec["observed"] == 0
        with pytest.raises(ValueError):
            heap.symm_at(st.flags, world)            # translation checks the rank
        with pytest.raises(ValueError):
            heap.symm_at(torch.zeros(4), 0)          # ... and that the object lives in the heap
    finally:
        heap.close()


def test_ag_push_protocol_three_cpu_ranks():
    run_cpu_ranks(_ag_calls, 3)


def test_rs_scatter_protocol_two_cpu_ranks():
    run_cpu_ranks(_rs_calls, 2)


def test_missing_rank_times_out_with_a_record():
    run_cpu_ranks(_missing_rank, 2)
