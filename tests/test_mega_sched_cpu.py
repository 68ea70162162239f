"""The C++ task scheduler of the decode megakernel, checked on the host: every task lands in exactly one SM queue,
queues keep stage order (so a task's dependency is always earlier in every queue it could wait behind), dependency
counts match the producing stage, and the two placement policies balance the load."""
import pytest
import torch

from triton_distributed_b200 import _native

lib = _native.load(False)
pytestmark = pytest.mark.skipif(lib is None, reason="native library not built")

def _build(policy, sms=7):
    s = lib.MegaScheduler()
    op = s.add_op([], [1, 2, 3], [0.5])
    # stage graph of one layer: norm -> linear (n0 tiles x n1 splits) -> rope -> attention (b x h x splits) -> combine
    st0 = s.add_stage(1, op, 4, 1, 1, -1)        # task types: 1 norm, 2 linear, 3 rope, 4 attention split, 5 combine
    st1 = s.add_stage(2, op, 10, 3, 1, st0)      # linear: dependants wait for its n0 output tiles, not for n0 * n1 tasks
    st2 = s.add_stage(3, op, 4, 1, 1, st1)
    st3 = s.add_stage(4, op, 4, 2, 5, st2)
    st4 = s.add_stage(5, op, 4, 8, 1, st3)
    s.schedule(sms, policy)
    return s, (st0, st1, st2, st3, st4)


@pytest.mark.parametrize("policy", [0, 1])
def test_every_task_scheduled_once_in_stage_order(policy):
    sms = 7
    s, stages = _build(policy, sms)
    tasks = s.tasks_tensor()            # [n, 16] int32: type, dep_idx, dep_need, out_idx, op, a0, a1, a2, ...
    offs = s.offsets_tensor().tolist()
    assert offs[0] == 0 and offs[-1] == tasks.shape[0] and len(offs) == sms + 1
    expect = {0: 4, 1: 30, 2: 4, 3: 40, 4: 32}
    seen = {}
    for sm in range(sms):
        q = tasks[offs[sm]:offs[sm + 1]]
        out_idx = q[:, 3].tolist()
        assert out_idx == sorted(out_idx), "a queue must run its tasks in stage order"
        for row in q.tolist():
            key = (row[3], row[5], row[6], row[7])
            assert key not in seen, "task scheduled twice"
            seen[key] = sm
    for st, n in expect.items():
        assert sum(1 for k in seen if k[0] == st) == n
    # dependency bookkeeping: stage 2 waits for the 10 output tiles of the linear stage, stage 4 for all 40 attention tasks
    rows = tasks.tolist()
    assert all(r[1] == -1 for r in rows if r[3] == stages[0])
    assert all(r[1] == stages[1] and r[2] == 10 for r in rows if r[3] == stages[2])
    assert all(r[1] == stages[3] and r[2] == 40 for r in rows if r[3] == stages[4])
    per_sm = s.tasks_per_sm()
    # round robin continues where the previous stage stopped; zig-zag alternates the direction per stage and may
    # leave up to one task per stage of imbalance
    assert sum(per_sm) == 110 and max(per_sm) - min(per_sm) <= (2 if policy == 0 else 5)


def test_bad_graphs_are_rejected():
    s = lib.MegaScheduler()
    op = s.add_op([], [], [])
    with pytest.raises(RuntimeError):
        s.add_stage(1, op, 1, 1, 1, 3)        # depends on a stage that does not exist yet
    with pytest.raises(RuntimeError):
        s.add_stage(1, op + 5, 1, 1, 1, -1)   # unknown operator
    with pytest.raises(RuntimeError):
        s.add_stage(1, op, 0, 1, 1, -1)       # empty stage
