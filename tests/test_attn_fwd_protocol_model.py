"""Model check of the barrier protocol of the attention forward kernel
(``attn_fwd_kernel`` in mist_b200/csrc/attn_fwd_tcgen05.cu), for the default layout (one producer
thread requests K and V) and the layout with a producer warp of its own for V.

Roles: producer(s), MMA issuer, softmax threads, the in-order tensor-core queue.  Per key block j
(stage st = j % 2, score buffer b = j & 1):

    k_full[st], v_full[st]   producer -> MMA        the tile is in shared memory
    k_empty[st]              MMA commit -> producer the S product of block j has read K
    kv_empty[st]             MMA commit -> producer the PV product of block j has read V
    s_full[b]                MMA commit -> softmax  S of block j is in tensor memory
    s_empty[b]               softmax -> MMA         S of block j is in registers
    p_full                   softmax -> MMA         P of block j is in shared memory, O rescaled
    pv_done                  MMA commit -> softmax  the PV product of block j is complete

The simulation replays waits, arrivals and parities with random latencies and checks liveness and
that no buffer is overwritten while in use.  It also shows what the second producer is for: with one
producer the request for K of block j+1 waits behind V's stage of block j.
"""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from protocol_sim import MBar, Resource, Sim, Task, TensorQueue  # noqa: E402

STAGES = 2


def simulate(n_blocks, seed, split, n_soft=3, slow=None, drop=(), tma=(0.5, 3.0)):
    sim = Sim(seed)
    slow = slow or {}

    def lat(role, lo, hi):
        return sim.lat(lo, hi) * slow.get(role, 1.0)

    q_full = MBar(sim, "q_full", 1)
    k_full = [MBar(sim, f"k_full{s}", 1) for s in range(STAGES)]
    v_full = [MBar(sim, f"v_full{s}", 1) for s in range(STAGES)]
    k_empty = [MBar(sim, f"k_empty{s}", 1) for s in range(STAGES)]
    kv_empty = [MBar(sim, f"kv_empty{s}", 1) for s in range(STAGES)]
    s_full = [MBar(sim, f"s_full{b}", 1) for b in range(2)]
    s_empty = [MBar(sim, f"s_empty{b}", n_soft) for b in range(2)]
    p_full = MBar(sim, "p_full", n_soft)
    pv_done = MBar(sim, "pv_done", 1)

    K = [Resource(f"K{s}") for s in range(STAGES)]
    V = [Resource(f"V{s}") for s in range(STAGES)]
    S = [Resource(f"S{b}") for b in range(2)]
    P = Resource("P", writers=n_soft)
    O = Resource("O")          # accumulator: "written" by every PV product, touched by rescaling in between
    tq = TensorQueue(sim)

    def load(res, bar, j):
        res.write_begin(j)
    
        def land():
            res.write_end(j)
            bar.arrive()
        sim.at(lat("tma", *tma), land)

    def producer_kv():
        if n_blocks == 0:
            return
        sim.at(lat("tma", *tma), q_full.arrive)
        for j in range(n_blocks):
            st = j % STAGES
            if j >= STAGES and "k_empty" not in drop:
                yield ("wait", k_empty[st], ((j // STAGES) - 1) & 1)
            load(K[st], k_full[st], j)
            if split:
                continue
            if j >= STAGES and "kv_empty" not in drop:
                yield ("wait", kv_empty[st], ((j // STAGES) - 1) & 1)
            load(V[st], v_full[st], j)
            yield ("sleep", 0.01)

    def producer_v():
        for j in range(n_blocks):
            st = j % STAGES
            if j >= STAGES and "kv_empty" not in drop:
                yield ("wait", kv_empty[st], ((j // STAGES) - 1) & 1)
            load(V[st], v_full[st], j)
            yield ("sleep", 0.01)

    def mma():
        if n_blocks == 0:
            return
        yield ("wait", q_full, 0)

        def issue_s(j):
            st, b = j % STAGES, j & 1
            yield ("wait", k_full[st], (j // STAGES) & 1)
            if j >= 2 and "s_empty" not in drop:
                yield ("wait", s_empty[b], ((j >> 1) - 1) & 1)

            def start():
                K[st].read_begin(j)
                S[b].write_begin(j)

            def end():
                K[st].read_end()
                S[b].write_end(j)
            tq.op(lat("mma", 0.15, 0.3), start, end)
            tq.commit(k_empty[st])
            tq.commit(s_full[b])

        yield from issue_s(0)
        for j in range(n_blocks):
            if j + 1 < n_blocks:
                yield from issue_s(j + 1)
            st = j % STAGES
            yield ("wait", p_full, j & 1)
            yield ("wait", v_full[st], (j // STAGES) & 1)

            def start(j=j, st=st):
                P.read_begin(j)
                V[st].read_begin(j)
                O.write_begin(j)

            def end(j=j, st=st):
                P.read_end()
                V[st].read_end()
                O.write_end(j)
            tq.op(lat("mma", 0.15, 0.3), start, end)
            tq.commit(kv_empty[st])
            tq.commit(pv_done)
            yield ("sleep", 0.01)

    def softmax(tid):
        for j in range(n_blocks):
            b = j & 1
            yield ("wait", s_full[b], (j >> 1) & 1)
            S[b].read_begin(j)
            yield ("sleep", lat("soft", 0.05, 0.2))
            S[b].read_end()
            s_empty[b].arrive()
            yield ("sleep", lat("soft", 0.5, 1.5))           # max, exponentials
            if j > 0:
                if "pv_done" not in drop:
                    yield ("wait", pv_done, (j - 1) & 1)
                if tid == 0:                                    # rescaling touches the accumulator between two products
                    O.read_begin(j - 1)
                    O.read_end()
            P.write_begin(j)
            yield ("sleep", lat("soft", 0.02, 0.1))
            P.write_end(j)
            p_full.arrive()
        if n_blocks > 0:
            yield ("wait", pv_done, (n_blocks - 1) & 1)
            if tid == 0:
                O.read_begin(n_blocks - 1)
                O.read_end()

    tasks = [Task(sim, producer_kv(), "producer"), Task(sim, mma(), "mma")]
    if split:
        tasks.append(Task(sim, producer_v(), "producer_v"))
    tasks += [Task(sim, softmax(i), f"softmax{i}") for i in range(n_soft)]
    sim.run()
    stuck = [t.name for t in tasks if not t.done]
    assert not stuck, f"n_blocks={n_blocks} seed={seed} split={split}: stuck roles {stuck}"
    if n_blocks > 0:
        assert p_full.completed == n_blocks and pv_done.completed == n_blocks
    return sim.t


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("n_blocks", [0, 1, 2, 3, 4, 7, 16])
def test_forward_protocol_random_latencies(n_blocks, split):
    for seed in range(50):
        simulate(n_blocks, seed, split)


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("role", ["tma", "mma", "soft"])
def test_forward_protocol_with_one_slow_role(role, split):
    for seed in range(20):
        simulate(9, seed, split, slow={role: 20.0})
        simulate(9, 500 + seed, split, slow={role: 0.05})


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("wait", ["k_empty", "kv_empty", "pv_done"])
def test_forward_model_reports_a_hazard_when_a_wait_is_left_out(wait, split):
    """Mutation check of the model.  (``s_empty`` is not in the list: the MMA warp issues S of block
    j+2 only after it has seen ``p_full`` of block j, which already implies that S of block j has been
    read, so that wait is redundant in the kernel and the model rightly reports nothing without it.)"""
    failures = 0
    for seed in range(40):
        for slow in ({}, {"soft": 8.0}, {"mma": 8.0}, {"tma": 0.05}, {"tma": 8.0}):
            try:
                simulate(9, seed, split, slow=slow, drop=(wait,))
            except AssertionError:
                failures += 1
    assert failures > 0


def test_second_producer_shortens_the_block_time_when_loads_take_longer_than_a_block():
    """Load latency 2.0 against about 1.2 of softmax time per block: with one producer the request for K
    of block j+1 goes out only once V's stage of block j is free, about one block before its S product,
    and the pipeline waits for the load; with two producers it goes out a block earlier."""
    n = 30
    single = sum(simulate(n, s, False, n_soft=1, tma=(1.8, 2.2)) for s in range(10)) / 10
    double = sum(simulate(n, s, True, n_soft=1, tma=(1.8, 2.2)) for s in range(10)) / 10
    assert double < 0.95 * single
