"""Fetch order of the gather CTAs of the fused GEMM kernels (``csrc/gather_plan.cuh``), run on the host through
``mb_gather_plan_segment``: the library that the GPU runs is loaded here only for this plain C function, so the
test needs no device.  Checked for the activation gather (AG -> GEMM) and the weight gather (ZeRO-3), 2 to 8 ranks:
every remote byte is fetched exactly once, nothing of the local shard is, a chunk's counter target equals the
number of its sub-chunks, flags are unique per chunk, and the order has the properties the kernels rely on
(activations: one source at a time, starting with the next rank; weights: the first-needed chunk first and all
peers interleaved)."""
import collections
import ctypes as C

import pytest

from mist_b200.ops import native


def _lib():
    path = native.kernels_path()
    if not path.exists():
        pytest.skip("kernels library not built")
    lib = C.CDLL(str(path))
    fn = lib.mb_gather_plan_segment
    fn.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_longlong, C.c_longlong, C.c_int,
                   C.POINTER(C.c_longlong)]
    fn.restype = C.c_int
    return fn


def _sequence(fn, weights, R, me, K=0, rows=0, shard=0, chunk=0, first=0):
    out = (C.c_longlong * 5)()
    n = fn(weights, R, me, K, rows, shard, chunk, first, -1, out)
    seq = []
    for q in range(n):
        if fn(weights, R, me, K, rows, shard, chunk, first, q, out):
            seq.append(tuple(int(v) for v in out))          # (offset, bytes, flag, expected, source)
    return seq


def _check_cover(seq, remote_ranges, me_range):
    """Every byte of ``remote_ranges`` once, none of ``me_range``, and the counters add up."""
    ivs = sorted((off, off + n) for off, n, *_ in seq)
    for (a0, a1), (b0, b1) in zip(ivs, ivs[1:]):
        assert a1 <= b0, "two sub-chunks overlap"
    assert sum(b - a for a, b in ivs) == sum(b - a for a, b in remote_ranges)
    for a, b in ivs:
        assert any(lo <= a and b <= hi for lo, hi in remote_ranges)
        assert b <= me_range[0] or a >= me_range[1]
    per_flag = collections.Counter(f for _, _, f, _, _ in seq)
    expected = {f: e for _, _, f, e, _ in seq}
    assert per_flag == expected
    for off, n, *_ in seq:
        assert off % 16 == 0 and n % 16 == 0 and n > 0       # bulk copies: 16-byte addresses and sizes


@pytest.mark.parametrize("R", [2, 3, 4, 8])
@pytest.mark.parametrize("K,rows", [(5120, 1024), (4096, 8192), (520, 256), (8, 128)])
def test_activation_gather_covers_the_peers_rows_once(R, K, rows):
    fn = _lib()
    row_bytes = K * 2
    for me in range(R):
        seq = _sequence(fn, 0, R, me, K=K, rows=rows)
        shard = rows * row_bytes
        remote = [(r * shard, (r + 1) * shard) for r in range(R) if r != me]
        _check_cover(seq, remote, (me * shard, (me + 1) * shard))
        # one flag per 128-row block, numbered [rank][block]
        for off, n, flag, exp, r in seq:
            assert flag == r * (rows // 128) + (off - r * shard) // (128 * row_bytes)
        # the peers in turn, starting with the next rank; blocks of a peer in row order
        sources = [r for *_, r in seq]
        turns = [sources[i] for i in range(len(sources)) if i == 0 or sources[i] != sources[i - 1]]
        assert turns == [(me + 1 + k) % R for k in range(R - 1)]
        offs = [off for off, *_ in seq]
        for r in set(sources):
            mine = [o for o, s in zip(offs, sources) if s == r]
            assert mine == sorted(mine)


@pytest.mark.parametrize("R", [2, 3, 4, 8])
@pytest.mark.parametrize("chunk", [1 << 20, 256 << 10, 100000 * 16])
def test_weight_gather_covers_the_peers_shards_once(R, chunk):
    fn = _lib()
    h = 2560
    numel = 12 * h * h + 13 * h
    padded = -(-numel // (128 * R)) * (128 * R)
    shard = padded // R * 2
    for first in (0, 2 * (2 * h + 128), 2 * (3 * h * h + 5248), padded * 2 - 4096):
        for me in range(R):
            seq = _sequence(fn, 1, R, me, shard=shard, chunk=chunk, first=first)
            remote = [(r * shard, (r + 1) * shard) for r in range(R) if r != me]
            _check_cover(seq, remote, (me * shard, (me + 1) * shard))
            cpr = -(-shard // chunk)
            for off, n, flag, exp, r in seq:
                assert flag == r * cpr + (off - r * shard) // chunk
            # the chunk that holds the first weights comes first from its owner, unless this rank owns it
            r0 = first // shard
            if r0 != me:
                head = next(s for s in seq if s[4] == r0)
                c0 = (first - r0 * shard) // chunk
                assert head[0] == r0 * shard + c0 * chunk
            # every peer shows up within the first R - 1 chunks: a rank reads from all peers at once
            subs = -(-chunk // (16 * 16384))
            first_sources = {s[4] for s in seq[: (R - 1) * subs]}
            assert first_sources == {r for r in range(R) if r != me}
