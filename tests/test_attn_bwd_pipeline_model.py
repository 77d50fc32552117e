"""Model check of the barrier protocol of the pipelined attention-backward kernel.

The kernel (``attn_bwd_pipe_kernel`` in mist_b200/csrc/attn_bwd_tcgen05.cu) runs five roles that
only meet through mbarriers: a TMA producer, an MMA issuer, the softmax threads, the dQ threads and
the in-order tensor-core queue.  This file replays the same waits, arrivals and parities in a
discrete-event simulation with random latencies and checks that

* every role finishes (no wait can starve),
* no buffer is overwritten while a reader still needs it, and nothing is read before it is written,
* no mbarrier phase is ever entered twice by the same party (an arrival never lands in a phase
  that has not been opened by the completion of the previous one).

mbarrier semantics modelled: a phase bit that flips when the expected number of arrivals is in;
``wait(parity)`` passes while the current phase bit differs from ``parity``.
"""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

Q_STAGES = 3


from protocol_sim import GroupBarrier, MBar, Resource, Sim, Task, TensorQueue  # noqa: E402


def simulate(n_iter, seed, n_soft=3, n_dq=2, slow=None, drop=(), alias=False):
    """``drop`` names waits to leave out (mutation check: the model must then report a hazard).
    ``alias``: the large-head layout, where dQ^T of a block is written over that block's S^T buffer;
    otherwise dQ^T has a tensor-memory buffer of its own."""
    sim = Sim(seed)
    slow = slow or {}

    def lat(role, lo, hi):
        return sim.lat(lo, hi) * slow.get(role, 1.0)

    kv_full = MBar(sim, "kv_full", 1)
    q_full = [MBar(sim, f"q_full{s}", 1) for s in range(Q_STAGES)]
    q_empty = [MBar(sim, f"q_empty{s}", 1) for s in range(Q_STAGES)]
    sdp_full = [MBar(sim, f"sdp_full{b}", 1) for b in range(2)]
    pds_full = MBar(sim, "pds_full", n_soft)
    pds_empty = MBar(sim, "pds_empty", 1)
    dq_full = [MBar(sim, f"dq_full{b}", 1) for b in range(2)]
    dq_empty = MBar(sim, "dq_empty", n_dq)
    final_full = MBar(sim, "final_full", 1)

    Q = [Resource(f"Q{s}") for s in range(Q_STAGES)]
    # tensor-memory buffer b holds S^T / dP^T of block it (b = it & 1) and then dQ^T of the same block
    S = [Resource(f"S/dQ{b}") for b in range(2)]
    DQ = Resource("dQ")

    def dq_buf(it):
        return S[it & 1] if alias else DQ
    P = Resource("P/dS", writers=n_soft)
    STG = Resource("dq staging", writers=n_dq)
    VEC = [Resource(f"vec{b}") for b in range(2)]
    tq = TensorQueue(sim)
    soft_sync = GroupBarrier(sim, n_soft)
    dq_sync = GroupBarrier(sim, n_dq)
    reduce_done = {"t": 0.0}

    def producer():
        if n_iter == 0:
            return
        sim.at(lat("tma", 0.5, 2.0), kv_full.arrive)
        for it in range(n_iter):
            st = it % Q_STAGES
            if it >= Q_STAGES and "q_empty" not in drop:
                yield ("wait", q_empty[st], ((it // Q_STAGES) - 1) & 1)
            Q[st].write_begin(it)
            d = lat("tma", 0.5, 3.0)

            def land(st=st, it=it):
                Q[st].write_end(it)
                q_full[st].arrive()
            sim.at(d, land)
            yield ("sleep", 0.01)

    def mma():
        if n_iter == 0:
            return
        yield ("wait", kv_full, 0)

        def issue_sdp(it):
            st, b = it % Q_STAGES, it & 1
            yield ("wait", q_full[st], (it // Q_STAGES) & 1)
            if alias and it >= 2 and "dq_empty" not in drop:
                yield ("wait", dq_empty, (it - 2) & 1)

            def start():
                Q[st].read_begin(it)
                S[b].write_begin(("S", it))

            def end():
                Q[st].read_end()
                S[b].write_end(("S", it))
            tq.op(lat("mma", 0.2, 0.6), start, end)
            tq.commit(sdp_full[b])

        yield from issue_sdp(0)
        for it in range(n_iter):
            st = it % Q_STAGES
            if it + 1 < n_iter:
                yield from issue_sdp(it + 1)
            yield ("wait", pds_full, it & 1)
            if not alias and it > 0 and "dq_empty" not in drop:
                yield ("wait", dq_empty, (it - 1) & 1)

            def start(it=it, st=st):
                P.read_begin(it)
                Q[st].read_begin(it)
                dq_buf(it).write_begin(("DQ", it))

            def end(it=it, st=st):
                P.read_end()
                Q[st].read_end()
                dq_buf(it).write_end(("DQ", it))
            tq.op(lat("mma", 0.3, 0.9), start, end)
            tq.commit(q_empty[st])
            tq.commit(pds_empty)
            tq.commit(dq_full[it & 1])
            yield ("sleep", 0.01)
        tq.commit(final_full)

    def softmax(tid):
        if n_iter > 0 and tid == 0:
            VEC[0].write_begin(0)
            VEC[0].write_end(0)
        yield ("barrier", soft_sync)
        for it in range(n_iter):
            b = it & 1
            yield ("wait", sdp_full[b], (it >> 1) & 1)
            VEC[b].read_begin(it)
            S[b].read_begin(("S", it))
            yield ("sleep", lat("soft", 0.2, 1.5))
            S[b].read_end()
            VEC[b].read_end()
            yield ("sleep", lat("soft", 0.1, 0.8))
            if it > 0 and "pds_empty" not in drop:
                yield ("wait", pds_empty, (it - 1) & 1)
            P.write_begin(it)
            yield ("sleep", lat("soft", 0.05, 0.3))
            P.write_end(it)
            pds_full.arrive()
            if tid == 0 and it + 1 < n_iter:
                VEC[b ^ 1].write_begin(it + 1)
                VEC[b ^ 1].write_end(it + 1)
            yield ("barrier", soft_sync)
        if n_iter > 0:
            yield ("wait", final_full, 0)

    def dq(tid):
        for it in range(n_iter):
            yield ("wait", dq_full[it & 1], (it >> 1) & 1)
            dq_buf(it).read_begin(("DQ", it))
            yield ("sleep", lat("dq", 0.1, 0.5))
            dq_buf(it).read_end()
            dq_empty.arrive()
            if tid == 0 and sim.t < reduce_done["t"]:
                yield ("sleep", reduce_done["t"] - sim.t)         # wait until the last reduce has read the tile
            yield ("barrier", dq_sync)
            STG.write_begin(it)
            yield ("sleep", lat("dq", 0.1, 0.6))
            STG.write_end(it)
            yield ("barrier", dq_sync)
            if tid == 0:
                STG.read_begin(it)
                d = lat("dq", 0.2, 1.5)
                reduce_done["t"] = sim.t + d
                sim.at(d, STG.read_end)

    tasks = [Task(sim, producer(), "producer"), Task(sim, mma(), "mma")]
    tasks += [Task(sim, softmax(i), f"softmax{i}") for i in range(n_soft)]
    tasks += [Task(sim, dq(i), f"dq{i}") for i in range(n_dq)]
    sim.run()
    stuck = [t.name for t in tasks if not t.done]
    assert not stuck, f"n_iter={n_iter} seed={seed}: stuck roles {stuck}"
    if n_iter > 0:
        assert pds_full.completed == n_iter and dq_empty.completed == n_iter
        assert sum(b.completed for b in dq_full) == n_iter
        assert sum(b.completed for b in sdp_full) == n_iter
    return sim.t


@pytest.mark.parametrize("alias", [False, True])
@pytest.mark.parametrize("n_iter", [0, 1, 2, 3, 4, 5, 8, 13])
def test_pipelined_backward_protocol_random_latencies(n_iter, alias):
    for seed in range(60):
        simulate(n_iter, seed, alias=alias)


@pytest.mark.parametrize("alias", [False, True])
@pytest.mark.parametrize("role", ["tma", "mma", "soft", "dq"])
def test_pipelined_backward_protocol_with_one_slow_role(role, alias):
    """One role twenty times slower than the rest: the others must wait for it, never run past it."""
    for seed in range(25):
        simulate(9, seed, slow={role: 20.0}, alias=alias)
        simulate(9, 1000 + seed, slow={role: 0.05}, alias=alias)


def test_pipelining_overlaps_tensor_work_with_softmax():
    """One softmax thread and one dQ thread (so that mean latencies apply): per block the softmax
    chain takes about 1.5 time units and the tensor-core work about 1.0.  Run one after the other
    they would need 2.5 per block; overlapped, the block time must stay close to the softmax chain."""
    n = 40
    per_block = sum(simulate(n, s, n_soft=1, n_dq=1) for s in range(10)) / 10 / n
    assert per_block < 2.0


@pytest.mark.parametrize("alias", [False, True])
@pytest.mark.parametrize("wait", ["q_empty", "dq_empty", "pds_empty"])
def test_model_reports_a_hazard_when_a_wait_is_left_out(wait, alias):
    """Mutation check of the model itself: without any one of the 'buffer free' waits some schedule
    must overwrite a buffer that is still needed (or desynchronise a barrier)."""
    failures = 0
    for seed in range(40):
        for slow in ({}, {"soft": 8.0}, {"mma": 8.0}, {"dq": 8.0}, {"tma": 0.05}):
            try:
                simulate(9, seed, slow=slow, drop=(wait,), alias=alias)
            except AssertionError:
                failures += 1
    assert failures > 0
