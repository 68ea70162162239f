"""Tooling that needs no GPU: the contextual autotuner, the intra-kernel profiler's host side, topology probes and
the roofline helpers."""
import json
import time

import torch

from triton_distributed_b200.tools import autotuner, profiler
from triton_distributed_b200.utils import roofline, topology


def test_contextual_autotune_picks_the_fastest_config_and_caches(tmp_path):
    calls = []

    @autotuner.contextual_autotune(configs=autotuner.config_space(delay_ms=[4, 0, 2]), key=lambda n: f"n={n}",
                                   n_repeat=2, n_warmup=1, log_dir=str(tmp_path))
    def work(n):
        cfg = autotuner.current_config({"delay_ms": 0})
        calls.append(cfg["delay_ms"])
        time.sleep(cfg["delay_ms"] / 1e3)
        return n * 2

    assert work(21) == 42
    tuned = len(calls)
    assert tuned == 3 * 3 + 1 and calls[-1] == 0          # (warm-up + 2 repeats) per candidate, then the winner
    assert work(21) == 42 and len(calls) == tuned + 1      # cached: one more call only
    assert work(5) == 10 and len(calls) > tuned + 2        # another key tunes again
    log = (tmp_path / "rank-0.log").read_text()
    assert 'best {"delay_ms": 0}' in log
    assert autotuner.current_config({"x": 1}) == {"x": 1}  # outside of a tuned call the default comes back


def _record(block, group, task, start, sm, t_ns):
    tag = (block << 16) | (group << 12) | (task << 1) | int(start)
    return ((tag << 32) | (t_ns & 0xFFFFFFFF), (sm << 32) | (t_ns >> 32))


def test_profiler_decode_trace_and_sm_activity(tmp_path):
    buf = profiler.create_buffer(8, device="cpu")
    recs = [_record(3, 1, 7, True, 12, 1000), _record(3, 1, 7, False, 12, 1600),
            _record(4, 0, 9, True, 13, 1200), _record(4, 0, 9, False, 13, 2000)]
    buf[0] = len(recs)
    for i, (w0, w1) in enumerate(recs):
        buf[2 + 2 * i] = w0 - (1 << 64) if w0 >= (1 << 63) else w0
        buf[3 + 2 * i] = w1 - (1 << 64) if w1 >= (1 << 63) else w1
    dec = profiler.decode(buf)
    assert [(r["block"], r["group"], r["task"], r["start"], r["sm"], r["t_ns"]) for r in dec] == \
        [(3, 1, 7, True, 12, 1000), (3, 1, 7, False, 12, 1600), (4, 0, 9, True, 13, 1200), (4, 0, 9, False, 13, 2000)]
    trace = profiler.to_chrome_trace(dec, {7: "linear", 9: "attn"}, path=str(tmp_path / "t.json"))
    names = sorted(e["name"] for e in trace["traceEvents"])
    assert names == ["attn", "linear"] and json.load(open(tmp_path / "t.json"))["traceEvents"]
    act = profiler.sm_activity(dec)
    assert abs(act[12] - 0.6) < 1e-9 and abs(act[13] - 0.8) < 1e-9


def test_topology_probes_answer_without_a_gpu():
    d = topology.describe()
    assert isinstance(d, dict) and d["gpus"] == topology.device_count()
    assert topology.device_count() >= 0
    assert isinstance(topology.has_fullmesh_nvlink(2), bool)


def test_roofline_arithmetic():
    peaks = {"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "source": "test"}
    r = roofline.gemm_roofline(8192, 8192, 8192, 1.0, peaks=peaks)
    assert abs(r["tflops"] - 2 * 8192 ** 3 / 1e9) < 1e-6 and 0 < r["frac_of_roofline"] < 1
    f = roofline.fused_roofline(2 * 8192 * 8192 * 3584.0, 117e6, 0.5, peaks=peaks)
    assert f["roofline_ms"] >= max(f["compute_ms"], f["link_ms"]) - 1e-9


def test_speed_of_light_models():
    assert roofline.get_tensorcore_tflops("fp8", measured=False) == 2 * roofline.get_tensorcore_tflops("bf16", measured=False)
    t = roofline.estimate_gemm_sol_time_ms(8192, 8192, 8192)
    assert 0.3 < t < 1.5                                     # 1.1 PFLOP at roughly 1.6 PFLOP/s
    ag = roofline.estimate_all_gather_time_ms(8192 * 8192 * 2, 8)
    rs = roofline.estimate_reduce_scatter_time_ms(8192 * 8192 * 2, 8)
    assert abs(ag - rs) < 1e-9 and 0.1 < ag < 0.3            # 117 MB over about 770 GB/s


def test_autotuner_drives_op_knobs():
    """The launch knobs of an op come from the autotuner's active configuration: a tuned thunk sees every candidate
    through current_config() and the winner afterwards (reference: python/triton_dist/autotuner.py:43-250)."""
    import time
    from triton_distributed_b200.tools.autotuner import contextual_autotune, current_config, config_space
    from triton_distributed_b200.ops.ag_gemm import AG_GEMM_TUNE_SPACE
    from triton_distributed_b200.ops import tuned_configs

    seen = []

    @contextual_autotune(configs=config_space(n_comm_ctas=[4, 8, 16]), key=lambda n: f"n{n}", n_repeat=2, n_warmup=1)
    def thunk(n):
        c = current_config()["n_comm_ctas"]
        seen.append(c)
        time.sleep(0.001 * abs(c - 8) + 0.0005)
        return c

    assert thunk(1) == 8 and set(seen) == {4, 8, 16}
    n_calls = len(seen)
    assert thunk(1) == 8 and len(seen) == n_calls + 1          # cached: one more call, no re-tuning
    assert all({"use_multimem", "n_comm_ctas"} <= set(c) for c in AG_GEMM_TUNE_SPACE)
    hit = tuned_configs.lookup("ag_gemm", 8, 1024, 3584, 8192)
    assert hit and hit["use_multimem"] is True and hit["n_comm_ctas"] in (2, 4, 8)
    assert tuned_configs.lookup("ag_gemm", 8, 1000, 3584, 8192) is None


def test_decode_gemm_form_selection(monkeypatch):
    """Host-side choice of the decode GEMM's form: 0 splits (cluster form, launcher's choice) by default, the stream-K
    split rule only under TDB200_SKINNY_FORM=1, an explicit TDB200_GEMM_AR_SPLITS always, and the cluster shape from the
    autotuner's active configuration before the tuned table."""
    from triton_distributed_b200.ops import gemm_ar, tuned_configs
    from triton_distributed_b200.tools.autotuner import config_space, contextual_autotune

    monkeypatch.delenv("TDB200_GEMM_AR_SPLITS", raising=False)
    monkeypatch.delenv("TDB200_SKINNY_FORM", raising=False)
    assert gemm_ar.pick_gemm_ar_splits(128, 5120, 3200) == 0
    monkeypatch.setenv("TDB200_SKINNY_FORM", "1")
    assert gemm_ar.pick_gemm_ar_splits(16, 5120, 3200) == 0
    assert gemm_ar.pick_gemm_ar_splits(128, 5120, 3200) == gemm_ar.pick_stream_k_splits(128, 5120, 3200) == 1
    assert gemm_ar.pick_stream_k_splits(64, 1280, 12800) == 4          # few tiles, long K: split as far as the SMs allow
    monkeypatch.setenv("TDB200_GEMM_AR_SPLITS", "3")
    assert gemm_ar.pick_gemm_ar_splits(16, 5120, 3200) == 3
    assert [gemm_ar._mpad(m) for m in (1, 16, 17, 64, 65, 129, 256)] == [16, 16, 32, 64, 128, 256, 256]
    hit = tuned_configs.lookup("skinny_gemm", 1, 16, 2560, 5120)
    assert hit and 1 <= hit["cluster_nt"] <= 4 and 1 <= hit["cluster_s"] <= 8
    seen = []

    @contextual_autotune(configs=config_space(cluster_nt=[1, 2], cluster_s=[3]), key=lambda: "k", n_repeat=1, n_warmup=1)
    def thunk():
        seen.append(gemm_ar.cluster_config(16, 2560, 5120))

    thunk()
    assert set(seen) == {(1, 3), (2, 3)}


def test_decode_gemm_routes_misaligned_outputs_to_the_scalar_store_form(monkeypatch):
    """The cluster form stores four bf16 values at a time.  An output view whose rows do not start on 8-byte boundaries
    must go through the stream-K form (splits >= 1), and an explicit cluster shape on such a view is refused."""
    import pytest
    from triton_distributed_b200 import _native
    from triton_distributed_b200.ops import gemm_ar

    calls = []

    class FakeLib:
        def skinny_gemm_bf16(self, x, w, out, acc, cnt, splits, num_ctas, nt, s, bulk):
            calls.append((splits, nt, s, acc.numel()))

    monkeypatch.setattr(_native, "load", lambda *a, **k: FakeLib())
    monkeypatch.setattr(gemm_ar, "cluster_config", lambda M, N, K: (0, 0))
    monkeypatch.setattr(gemm_ar, "_scratch", lambda dev, need_acc, need_tiles: (torch.zeros(need_acc), torch.zeros(need_tiles)))
    x = torch.zeros(65, 64, dtype=torch.bfloat16)
    w = torch.zeros(640, 64, dtype=torch.bfloat16)
    big = torch.zeros(65, 648, dtype=torch.bfloat16)
    gemm_ar.skinny_gemm(x, w, out=big[:, :640])                 # rows 1296 bytes apart, start aligned: cluster form
    gemm_ar.skinny_gemm(x, w, out=big[:, 1:641])                # starts 2 bytes in: stream-K form
    odd = torch.zeros(65, 641, dtype=torch.bfloat16)
    gemm_ar.skinny_gemm(x, w, out=odd[:, :640])                 # row pitch 1282 bytes: stream-K form
    assert [c[0] for c in calls] == [0, 1, 1]
    assert all(c[3] >= 640 * 128 for c in calls)                # scratch sized by the token pad (65 -> 128)
    with pytest.raises(ValueError):
        gemm_ar.skinny_gemm(x, w, out=big[:, 1:641], cluster=(1, 2))

    # a table entry that does not fit this GPU is a hint: one refusal, then the launcher's own choice from then on
    class PickyLib(FakeLib):
        def skinny_gemm_bf16(self, x, w, out, acc, cnt, splits, num_ctas, nt, s, bulk):
            calls.append((splits, nt, s, acc.numel()))
            if (nt, s) == (2, 6):
                raise RuntimeError("launch_skinny_gemm: invalid configuration argument")

    del calls[:]
    monkeypatch.setattr(_native, "load", lambda *a, **k: PickyLib())
    monkeypatch.setattr(gemm_ar, "cluster_config", lambda M, N, K: (2, 6))
    monkeypatch.setattr(gemm_ar, "_UNFIT_TABLE_SHAPES", set())
    gemm_ar.skinny_gemm(x, w, out=big[:, :640])
    gemm_ar.skinny_gemm(x, w, out=big[:, :640])
    assert [(c[1], c[2]) for c in calls] == [(2, 6), (0, 0), (0, 0)]
    with pytest.raises(RuntimeError):
        gemm_ar.skinny_gemm(x, w, out=big[:, :640], cluster=(2, 6))      # an explicit request stays a demand


def test_user_tuned_table_comes_first(tmp_path, monkeypatch):
    from triton_distributed_b200.ops import tuned_configs

    path = tmp_path / "tuned.json"
    path.write_text(json.dumps([
        {"op": "skinny_gemm", "world": 1, "rows": 16, "n": 2560, "k": 5120, "config": {"cluster_nt": 1, "cluster_s": 5}},
        {"op": "skinny_gemm", "world": 1, "rows": 64, "n": 777, "k": 888, "config": {"cluster_nt": 1, "cluster_s": 2}}]))
    monkeypatch.setenv("TDB200_TUNED_CONFIGS", str(path))
    monkeypatch.setattr(tuned_configs, "_USER_TABLE", None)
    assert tuned_configs.lookup("skinny_gemm", 1, 16, 2560, 5120) == {"cluster_nt": 1, "cluster_s": 5}   # overrides
    assert tuned_configs.lookup("skinny_gemm", 1, 64, 777, 888) == {"cluster_nt": 1, "cluster_s": 2}     # adds
    assert tuned_configs.lookup("ag_gemm", 8, 1024, 3584, 8192)["n_comm_ctas"] == 4                      # built-in stays
    monkeypatch.setattr(tuned_configs, "_USER_TABLE", None)
    monkeypatch.delenv("TDB200_TUNED_CONFIGS")
    assert tuned_configs.lookup("skinny_gemm", 1, 64, 777, 888) is None


def test_cluster_exchange_index_arithmetic():
    """The row slices, receive slots and shared-memory bounds of the decode GEMM's cluster exchange
    (csrc/gemm_ar_sm100.cu, skinny_cluster_kernel), restated on the host: the S slices partition the M rows, every
    destination sees its S - 1 sources in distinct slots, and the receive area never exceeds the room the kernel
    reserves behind the part (the part's size plus eight rows)."""
    for mpad in (16, 32, 64, 128, 256):
        for M in range(1, mpad + 1):
            if M <= mpad // 2 and mpad > 16:
                continue                                   # a smaller pad would have been chosen
            for S in range(1, 9):
                rows_per = -(-M // S)
                covered = []
                for r in range(S):
                    covered += list(range(r * rows_per, min(M, (r + 1) * rows_per)))
                assert covered == list(range(M))
                for d in range(S):
                    slots = sorted((r if r < d else r - 1) for r in range(S) if r != d)
                    assert slots == list(range(S - 1))
                assert (S - 1) * rows_per <= mpad + 8


def test_op_log_records_json(tmp_path):
    import json
    import torch
    from triton_distributed_b200.utils import oplog
    from triton_distributed_b200.ops.gemm import gemm

    path = tmp_path / "ops.jsonl"
    oplog.enable(str(path))
    try:
        a, b = torch.randn(8, 64), torch.randn(16, 64)
        gemm(a, b)
        new = oplog.flush()
    finally:
        oplog.disable()
    assert new and new[-1]["op"] == "gemm" and new[-1]["shape"] == {"M": 8, "N": 16, "K": 64}
    rec = json.loads(path.read_text().splitlines()[-1])
    assert rec["us"] > 0 and "tflops" in rec and "roofline_frac" in rec
