"""Model of the copy ring that a gather CTA of the fused GEMM kernels drives (``gemm_comm_tcgen05.cu``: one
thread, eleven 16 KB shared-memory buffers, bulk loads from a peer completing on per-buffer barriers, bulk stores
to local memory in commit groups, sub-chunks counted on their chunk once their stores have completed).

The model replays the thread's program order with random and with extreme latencies of loads, of the read phase of
a store and of its write phase, under the completion rules of the hardware interface the kernel uses: a wait on
"all but the N youngest groups have been read" / "... have completed" returns when the slowest of the older groups
has, groups may otherwise finish in any order.  It asserts what the kernel relies on:

* a buffer is not loaded into again before the store that last used it has read it;
* a store is issued only after its load has landed, and a barrier is never two phases ahead of its wait;
* a sub-chunk is counted (and so a chunk's flag published) only after every one of its stores has completed;
* every sub-chunk is counted exactly once, and the first-in-first-out list of finished sub-chunks never holds more
  than its eight entries.

Leaving out either wait, or waiting with too large an N, must make the model report the corresponding hazard
(otherwise the model would prove nothing).
"""
import random

import pytest

BUFS, LOADS_AHEAD, STORES_READING, PUBLISH_LAG, FIFO = 11, 6, 4, 6, 8     # the kernel's constants


class Hazard(Exception):
    pass


def run(sub_chunks, lat, bufs=BUFS, loads_ahead=LOADS_AHEAD, stores_reading=STORES_READING,
        publish_lag=PUBLISH_LAG, wait_before_load=True, wait_before_count=True):
    """``sub_chunks``: pieces per sub-chunk in the CTA's order.  ``lat(kind)``: a latency sample for kind in
    {"load", "read", "write"}.  Returns the list of counted sub-chunks in order."""
    t = 0.0
    issued = stored = 0
    load_done = []                 # completion time of load n
    store_read, store_done = [], []
    pieces = [(s, p) for s, n in enumerate(sub_chunks) for p in range(n)]
    last_piece = {s: sum(sub_chunks[: s + 1]) - 1 for s in range(len(sub_chunks))}
    fifo, counted = [], []
    buffer_store = {}              # buffer -> index of the store that last used it

    def older_than_youngest(n, times):
        """Time at which all but the ``n`` youngest stores have reached the state recorded in ``times``."""
        old = times[: max(len(times) - n, 0)]
        return max(old) if old else 0.0

    while stored < len(pieces):
        while issued < len(pieces) and issued - stored < loads_ahead:
            b = issued % bufs
            if issued >= bufs and wait_before_load:
                t = max(t, older_than_youngest(stores_reading, store_read))
            if b in buffer_store and store_read[buffer_store[b]] > t:
                raise Hazard(f"load {issued} overwrites buffer {b} while store {buffer_store[b]} still reads it")
            # the barrier of buffer b must have been waited for in its previous phase
            if issued >= bufs and stored <= issued - bufs:
                raise Hazard(f"barrier of buffer {b} two phases ahead")
            load_done.append(t + lat("load"))
            issued += 1
        b = stored % bufs
        t = max(t, load_done[stored])                     # wait on the buffer's barrier
        r = t + lat("read")
        store_read.append(r)
        store_done.append(r + lat("write"))
        buffer_store[b] = stored
        stored += 1
        s, _ = pieces[stored - 1]
        if stored - 1 == last_piece[s]:
            fifo.append((s, stored))
            if len(fifo) > FIFO:
                raise Hazard("list of finished sub-chunks overflows")
        if fifo and stored - fifo[0][1] >= publish_lag:
            if wait_before_count:
                t = max(t, older_than_youngest(publish_lag, store_done))
            while fifo and stored - fifo[0][1] >= publish_lag:
                s0, mark = fifo.pop(0)
                first = mark - sub_chunks[s0]
                if max(store_done[first:mark]) > t:
                    raise Hazard(f"sub-chunk {s0} counted before its stores completed")
                counted.append(s0)
    t = max([t] + store_done)                              # wait for every group
    counted.extend(s for s, _ in fifo)
    return counted


def _random_lat(rng, scale):
    return lambda kind: rng.uniform(0.1, 1.0) * scale[kind]


@pytest.mark.parametrize("seed", range(20))
def test_ring_is_hazard_free_under_random_latencies(seed):
    rng = random.Random(seed)
    subs = [rng.choice([1, 2, 3, 7, 16, 16, 16]) for _ in range(rng.randint(1, 40))]
    scale = {"load": rng.choice([1, 10, 100]), "read": rng.choice([0.1, 1, 50]), "write": rng.choice([0.1, 1, 200])}
    assert run(subs, _random_lat(rng, scale)) == list(range(len(subs)))


@pytest.mark.parametrize("slow", ["load", "read", "write"])
def test_ring_is_hazard_free_when_one_phase_is_very_slow(slow):
    rng = random.Random(7)
    scale = {"load": 1.0, "read": 1.0, "write": 1.0}
    scale[slow] = 1000.0
    for subs in ([16] * 12, [1] * 40, [3, 1, 16, 2, 1, 1, 1, 16]):
        assert run(subs, _random_lat(rng, scale)) == list(range(len(subs)))


def test_model_reports_the_hazards_the_waits_prevent():
    rng = random.Random(3)
    slow_read = _random_lat(rng, {"load": 0.01, "read": 500.0, "write": 1.0})
    with pytest.raises(Hazard, match="still reads"):
        run([16] * 8, slow_read, wait_before_load=False)
    with pytest.raises(Hazard, match="still reads"):
        run([16] * 8, slow_read, stores_reading=BUFS - LOADS_AHEAD + 1)      # one too many stores may still read
    slow_write = _random_lat(rng, {"load": 0.01, "read": 0.01, "write": 500.0})
    with pytest.raises(Hazard, match="before its stores completed"):
        run([4] * 16, slow_write, wait_before_count=False)
    # the largest number of stores that may still be reading without a hazard is what the kernel uses or more
    assert BUFS - 1 - LOADS_AHEAD >= STORES_READING
    run([16] * 8, slow_read, stores_reading=BUFS - LOADS_AHEAD)              # the limit itself is still safe
