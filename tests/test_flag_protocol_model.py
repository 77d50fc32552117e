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
