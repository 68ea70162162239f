"""Symmetric heap, device API and bounded waits on one GPU (world size 1: the rank is its own peer)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import triton_distributed_b200 as tdb

    tdb.initialize_distributed(seed=0)
    yield tdb.get_runtime()


def test_alloc_free_reuse(rt):
    a = rt.symm_tensor((1024,), torch.float32)
    off_a = rt.offset_of(a)
    b = rt.symm_tensor((333, 7), torch.bfloat16)
    assert rt.offset_of(b) >= off_a + 4096
    assert rt.is_symmetric(a) and rt.is_symmetric(b)
    a.fill_(3.0)
    assert a.sum().item() == 3072.0
    rt.symm_free(a)
    c = rt.symm_tensor((512,), torch.float32)
    assert rt.offset_of(c) == off_a  # first fit reuses the hole
    rt.symm_free(b)
    rt.symm_free(c)


def test_device_primitives_single_rank(rt):
    from triton_distributed_b200 import _native

    lib = _native.load(True)
    n = 300
    data = rt.symm_tensor((rt.world_size * n,), torch.int32)
    scratch = rt.symm_tensor((2 * n,), torch.int32)
    sig = rt.symm_tensor((32,), torch.int32)
    bar = rt.symm_tensor((16,), torch.int32)
    for epoch in (1, 2, 3):
        lib.primitives_test(rt.heap, data, scratch, sig, bar, n, epoch, 2.0)
        torch.cuda.synchronize()
        rt.check_status()
        exp = torch.arange(n, device="cuda", dtype=torch.int32) + 1000
        assert torch.equal(data[:n], exp)
        assert torch.equal(scratch[:n], exp)
        assert sig[0].item() == epoch and sig[8].item() == epoch * 100


def test_barrier_on_stream(rt):
    for _ in range(3):
        rt.barrier_all_on_stream()
    s = torch.cuda.Stream()
    rt.barrier_all_on_stream(s)
    torch.cuda.synchronize()
    rt.check_status()


def test_bounded_wait_reports_and_context_survives(rt):
    """A flag that nothing sets: the kernel must give up after the limit, report, and leave the GPU usable."""
    from triton_distributed_b200 import CommTimeoutError, _native

    lib = _native.load(True)
    flag = rt.symm_tensor((4,), torch.int32)
    lib.timeout_probe(rt.heap, flag, 5, 0.2)
    with pytest.raises(CommTimeoutError) as ei:
        rt.check_status()
    assert ei.value.record["code"] == 1 and ei.value.record["where"] == 99 and ei.value.record["expected"] == 5
    # the context is intact: a normal kernel still runs, and the status page is clear again
    x = torch.ones(1024, device="cuda")
    assert x.sum().item() == 1024
    rt.check_status()


def test_debug_translation_reports_bad_ranges(rt):
    """The checked put (what TDB200_DEBUG=1 enables in every put / get / signal): a rank outside the world or a range that
    leaves the heap is reported as status 4 and nothing is written; a valid put goes through."""
    from triton_distributed_b200 import CommTimeoutError, _native

    lib = _native.load(True)
    dst = rt.symm_tensor((64,), torch.int32)
    src = torch.arange(64, dtype=torch.int32, device="cuda")
    lib.bounds_probe(rt.heap, dst, src, 256, rt.rank)
    rt.check_status()
    assert torch.equal(dst, src)
    dst.zero_()
    lib.bounds_probe(rt.heap, dst, src, 256, rt.world_size + 3)          # no such rank
    with pytest.raises(CommTimeoutError) as ei:
        rt.check_status()
    assert ei.value.record["code"] == 4 and ei.value.record["where"] == 101 and ei.value.record["peer"] == rt.world_size + 3
    outside = torch.zeros(64, dtype=torch.int32, device="cuda")           # ordinary device memory, not a heap object
    lib.bounds_probe(rt.heap, outside, src, 256, rt.rank)
    with pytest.raises(CommTimeoutError) as ei:
        rt.check_status()
    assert ei.value.record["code"] == 4
    assert int(dst.abs().sum()) == 0 and int(outside.abs().sum()) == 0
    rt.check_status()


def test_abort_word_stops_a_wait(rt):
    from triton_distributed_b200 import CommTimeoutError, _native

    lib = _native.load(True)
    flag = rt.symm_tensor((4,), torch.int32)
    rt.abort()
    lib.timeout_probe(rt.heap, flag, 9, 5.0)
    torch.cuda.synchronize()
    with pytest.raises(CommTimeoutError) as ei:
        rt.check_status()
    assert ei.value.record["code"] == 5
    rt.clear_abort()


def test_stream_write_and_wait_value(rt):
    from triton_distributed_b200 import _native

    lib = _native.load(True)
    flag = rt.symm_tensor((4,), torch.int32)
    lib.stream_write_value32(flag.data_ptr(), 7)
    lib.stream_wait_value32(flag.data_ptr(), 7, True)
    torch.cuda.synchronize()
    assert flag[0].item() == 7
