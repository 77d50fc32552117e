"""Exhaustive interleaving check of the flag protocol the peer-memory kernels use.

Every launch of a fused kernel (gradient reduce + Adam, all-gather -> GEMM, GEMM ->
reduce-scatter, weight gather -> GEMM) on rank ``r`` with launch counter ``e`` does:

  A. (stream order, before the launch) rank r's own buffer holds the data of launch e
  B. ready[p][r] := e  for every peer p                      (st.release.sys)
  C. for every peer p: wait ready[r][p] >= e, then read p's buffer   (ld.acquire.sys + loads)
  D. done[p][r] := e  for every peer p
  E. wait done[r][p] >= e for every peer p, then the kernel ends
  -> the next launch may overwrite rank r's buffer

The property: whenever a rank reads a peer's buffer in launch e it sees the data of launch e
(never the previous launch's, never the next one's).  The model below walks every
interleaving of the ranks' atomic steps for small cases and checks that; a variant without
step E must fail, which shows the final wait is what protects the buffers.
"""
import itertools

import pytest


def _explore(R: int, epochs: int, wait_done: bool = True):
    """Returns None when every interleaving keeps the property, else a counter-example trace."""
    peers = [[p for p in range(R) if p != r] for r in range(R)]
    # per-rank program: list of (op, arg) for one epoch
    prog = []
    for r in range(R):
        steps = [("write", None)]
        steps += [("ready", p) for p in peers[r]]
        steps += [("read", p) for p in peers[r]]
        steps += [("done", p) for p in peers[r]]
        if wait_done:
            steps += [("wait_done", p) for p in peers[r]]
        prog.append(steps)
    n = [len(s) for s in prog]

    # state: (pc per rank incl. epoch, buffer version per rank, ready matrix, done matrix)
    start = (tuple((1, 0) for _ in range(R)), (0,) * R, (0,) * (R * R), (0,) * (R * R))
    seen = {start}
    stack = [(start, ())]
    while stack:
        (pcs, ver, ready, done), trace = stack.pop()
        for r in range(R):
            e, i = pcs[r]
            if e > epochs:
                continue
            op, arg = prog[r][i]
            ver2, ready2, done2 = ver, ready, done
            if op == "write":
                ver2 = ver[:r] + (e,) + ver[r + 1:]
            elif op == "ready":
                k = arg * R + r
                ready2 = ready[:k] + (e,) + ready[k + 1:]
            elif op == "read":
                if ready[r * R + arg] < e:
                    continue                     # blocked: the peer has not announced launch e
                if ver[arg] != e:
                    return trace + ((r, e, op, arg, f"saw version {ver[arg]}"),)
            elif op == "done":
                k = arg * R + r
                done2 = done[:k] + (e,) + done[k + 1:]
            elif op == "wait_done":
                if done[r * R + arg] < e:
                    continue
            nxt = (e, i + 1) if i + 1 < n[r] else (e + 1, 0)
            state = (pcs[:r] + (nxt,) + pcs[r + 1:], ver2, ready2, done2)
            if state not in seen:
                seen.add(state)
                stack.append((state, trace + ((r, e, op, arg),)))
    # every rank must have been able to finish (no deadlock): some explored state has all done
    assert any(all(pc[0] > epochs for pc in s[0]) for s in seen), "protocol deadlocks"
    return None


@pytest.mark.parametrize("R,epochs", [(2, 3), (3, 2)])
def test_protocol_never_reads_stale_or_future_data(R, epochs):
    assert _explore(R, epochs) is None


def test_without_the_final_wait_a_buffer_is_overwritten_under_a_reader():
    trace = _explore(2, 2, wait_done=False)
    assert trace is not None and "saw version" in trace[-1][-1]


# --------------------------------------------------------------------------------------------------
# GEMM -> reduce-scatter, store form: launch e of rank s stores its tile for owner o into the slot
# slots[o][e % 2][s] (peer store), then announces done[o][s] := e; it then waits until every source has
# announced e on its own done row and sums its slots of set e % 2 (a separate kernel, in stream order
# before launch e + 1).  There is no opening flag round: the two slot sets alternate instead.  Property:
# an owner's sum of launch e reads, from every source, the tile of launch e.

def _explore_store_form(R: int, epochs: int, sets: int = 2, closing_round: bool = True):
    prog = []
    for r in range(R):
        steps = [("store", o) for o in range(R)]
        steps += [("done", o) for o in range(R) if o != r]
        if closing_round:
            steps += [("wait_done", s) for s in range(R) if s != r]
        steps += [("sum", s) for s in range(R)]
        prog.append(steps)
    # slots[o][set][s] = launch number of the tile it holds
    slots0 = tuple(0 for _ in range(R * sets * R))
    start = (tuple((1, 0) for _ in range(R)), slots0, (0,) * (R * R))
    seen = {start}
    stack = [(start, ())]
    while stack:
        (pcs, slots, done), trace = stack.pop()
        for r in range(R):
            e, i = pcs[r]
            if e > epochs:
                continue
            op, arg = prog[r][i]
            slots2, done2 = slots, done
            if op == "store":
                k = (arg * sets + e % sets) * R + r
                slots2 = slots[:k] + (e,) + slots[k + 1:]
            elif op == "done":
                k = arg * R + r
                done2 = done[:k] + (e,) + done[k + 1:]
            elif op == "wait_done":
                if done[r * R + arg] < e:
                    continue
            elif op == "sum":
                got = slots[(r * sets + e % sets) * R + arg]
                if got != e:
                    return trace + ((r, e, op, arg, f"summed the tile of launch {got}"),)
            ni = i + 1
            npc = (e + 1, 0) if ni == len(prog[r]) else (e, ni)
            state = (pcs[:r] + (npc,) + pcs[r + 1:], slots2, done2)
            if state not in seen:
                seen.add(state)
                stack.append((state, trace + ((r, e, op, arg),)))
    return None


@pytest.mark.parametrize("R,epochs", [(2, 4), (3, 3)])
def test_store_form_reduce_scatter_sums_the_tiles_of_its_own_launch(R, epochs):
    assert _explore_store_form(R, epochs) is None


def test_store_form_needs_two_slot_sets_and_the_closing_round():
    """With one slot set a fast source overwrites a tile before its owner has summed it; without the closing
    flag round an owner sums before every tile has landed."""
    bad = _explore_store_form(2, 3, sets=1)
    assert bad is not None and "summed the tile of launch" in bad[-1][-1]
    bad = _explore_store_form(2, 2, closing_round=False)
    assert bad is not None
