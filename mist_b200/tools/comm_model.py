"""Communication-latency and stream-interference models, and their fitting.

(a) GPU<->GPU collectives: a 4x4 table over (inter-node, intra-node) group sizes in
    {1, 2, 4, 8} of ``(bandwidth k [GB/s], bias b [s])``; a collective of ``B`` GB over
    ``n`` ranks costs ``B / k * (n - 1) / n + b`` times an op factor
    (all_reduce 2.1, all_gather 1.0, reduce_scatter 1.1); p2p costs ``B / k``.
(b) host<->GPU copies: ``B / k + b``.
(c) interference: four channels can be busy at once -- compute (C), GPU<->GPU (G2G),
    host->GPU (C2G), GPU->host (G2C).  28 slow-down factors (4 for all four busy, 4x3 for
    each triple, 6x2 for each pair) describe how much each channel stretches while the
    others run.  The estimate peels the overlap off step by step: stretch every active
    channel by its factor, the shortest stretched channel ends first and that span is
    charged once, the others keep what is left (un-stretched again), and the same is
    repeated with fewer active channels; whatever single channel remains is added.
(d) least-squares fitting of all parameters from profiling records.

Same model family and parameter layout as the reference (mist/tools/optimize.py:201-303
comm, :465-470 copies, :552-571 and :951-1122 interference, :351-542 and :1162-1248
fitting), re-implemented on plain numpy so one call evaluates whole candidate batches.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

GROUP_SIZES = (1, 2, 4, 8)
OP_FACTORS = {"all_reduce": 2.1, "all_gather": 1.0, "reduce_scatter": 1.1, "none": 0.0}

THREE_MASKS = np.array([[1, 1, 1, 0], [1, 1, 0, 1], [1, 0, 1, 1], [0, 1, 1, 1]], dtype=bool)
TWO_MASKS = np.array([[1, 1, 0, 0], [1, 0, 1, 0], [1, 0, 0, 1], [0, 1, 1, 0], [0, 1, 0, 1], [0, 0, 1, 1]], dtype=bool)


def _size_index(n) -> np.ndarray:
    n = np.asarray(n)
    return np.where(n >= 8, 3, np.where(n >= 4, 2, np.where(n >= 2, 1, 0)))


def gpu_gpu_latency(op: str, gbytes, intra, inter, params: Sequence[float]) -> np.ndarray:
    """Seconds for a collective of ``gbytes`` GB over ``intra * inter`` ranks."""
    table = np.asarray(params, dtype=np.float64).reshape(4, 4, 2)
    gbytes = np.asarray(gbytes, dtype=np.float64)
    if op == "p2p":
        k = table[1, 0, 0] if (inter is not None and np.any(np.asarray(inter) > 1)) else table[0, 1, 0]
        return gbytes / k
    if op not in OP_FACTORS:
        raise ValueError(f"unknown collective '{op}'")
    intra = np.broadcast_to(np.asarray(intra), gbytes.shape)
    inter = np.broadcast_to(np.asarray(inter if inter is not None else 1), gbytes.shape)
    n = intra * inter
    k = table[_size_index(inter), _size_index(intra), 0]
    b = table[_size_index(inter), _size_index(intra), 1]
    lat = gbytes / k * (n - 1) / np.maximum(n, 1) + b
    lat = np.where((gbytes < 1e-5) | (n == 1), 0.0, lat)
    return lat * OP_FACTORS[op]


def host_copy_latency(gbytes, params: Sequence[float]) -> np.ndarray:
    k, b = params
    gbytes = np.asarray(gbytes, dtype=np.float64)
    return np.where(gbytes == 0, 0.0, gbytes / k + b)


def interference_estimate(C, G2G, C2G, G2C, params: Sequence[float]) -> np.ndarray:
    """Total time of the four channels running concurrently (arrays broadcast together)."""
    p = np.asarray(params, dtype=np.float64)
    if p.size != 28:
        raise ValueError(f"interference model needs 28 parameters, got {p.size}")
    X = np.stack(np.broadcast_arrays(*(np.asarray(v, dtype=np.float64) for v in (C, G2G, C2G, G2C))), axis=-1).copy()
    shape = X.shape[:-1]
    X = X.reshape(-1, 4)
    out = np.zeros(X.shape[0])

    def peel(mask: np.ndarray, factors_active: np.ndarray):
        nz = ~np.isclose(X, 0.0)
        rows = np.where(np.all(nz == mask, axis=1))[0]
        if rows.size == 0:
            return
        f = np.ones(4)
        f[mask] = factors_active
        scaled = X[rows] * f
        overlap = scaled[:, mask].min(axis=1)
        out[rows] += overlap
        rest = (scaled - overlap[:, None]) / f
        X[np.ix_(rows, np.where(mask)[0])] = rest[:, mask]

    peel(np.ones(4, dtype=bool), p[:4])
    for i, m in enumerate(THREE_MASKS):
        peel(m, p[4 + 3 * i: 7 + 3 * i])
    for i, m in enumerate(TWO_MASKS):
        peel(m, p[16 + 2 * i: 18 + 2 * i])
    out += X.sum(axis=1)
    return out.reshape(shape)


# ------------------------------------------------------------------------------- fitting
def fit_gpu_gpu_params(records: List[Dict], n_restarts: int = 4, seed: int = 0) -> List[float]:
    """``records``: dicts with ``gbytes``, ``intra``, ``inter``, ``latency`` of all-gather-only
    runs.  Returns the 32-number table; unmeasured cells keep the placeholder (4.5, 0.0)."""
    from scipy.optimize import least_squares
    table = np.tile(np.array([4.5, 0.0]), (4, 4, 1))
    by_cell: Dict[Tuple[int, int], List[Dict]] = {}
    for r in records:
        if r["intra"] * r["inter"] > 1 and r["gbytes"] > 0:
            by_cell.setdefault((int(_size_index(r["inter"])), int(_size_index(r["intra"]))), []).append(r)
    for (oi, ii), rs in by_cell.items():
        g = np.array([r["gbytes"] for r in rs])
        n = np.array([r["intra"] * r["inter"] for r in rs], dtype=np.float64)
        y = np.array([r["latency"] for r in rs])

        def resid(x):
            return (g / x[0] * (n - 1) / n + x[1] - y) / np.maximum(y, 1e-6)

        k0 = float(np.median(g * (n - 1) / n / np.maximum(y, 1e-9)))
        sol = least_squares(resid, x0=[max(k0, 1e-3), 0.0], bounds=([1e-3, 0.0], [1e5, 0.1]))
        table[oi, ii] = sol.x
    return [float(v) for v in table.reshape(-1)]


def fit_host_copy_params(gbytes: Sequence[float], latency: Sequence[float]) -> List[float]:
    from scipy.optimize import least_squares
    g, y = np.asarray(gbytes, dtype=np.float64), np.asarray(latency, dtype=np.float64)
    sel = g > 0
    g, y = g[sel], y[sel]

    def resid(x):
        return (g / x[0] + x[1] - y) / np.maximum(y, 1e-6)

    k0 = float(np.median(g / np.maximum(y, 1e-9)))
    sol = least_squares(resid, x0=[k0, 0.0], bounds=([1e-3, 0.0], [1e5, 0.1]))
    return [float(sol.x[0]), float(sol.x[1])]


def fit_interference_params(C, G2G, C2G, G2C, measured, x0: Optional[Sequence[float]] = None,
                            upper: float = 100.0) -> List[float]:
    """Fits the 28 factors step by step: pairs first (only records with exactly two busy
    channels), then triples, then the four-way factors, each time holding the others."""
    from scipy.optimize import least_squares
    C, G2G, C2G, G2C, y = (np.asarray(v, dtype=np.float64) for v in (C, G2G, C2G, G2C, measured))
    X = np.stack([C, G2G, C2G, G2C], axis=1)
    busy = ~np.isclose(X, 0.0)
    p = np.array(x0 if x0 is not None else np.ones(28), dtype=np.float64)

    def fit_slice(sl: slice, mask: np.ndarray):
        rows = np.where(np.all(busy == mask, axis=1))[0]
        if rows.size == 0:
            return

        def resid(v):
            q = p.copy()
            q[sl] = v
            pred = interference_estimate(C[rows], G2G[rows], C2G[rows], G2C[rows], q)
            return (pred - y[rows]) / np.maximum(y[rows], 1e-6)

        n = sl.stop - sl.start
        sol = least_squares(resid, x0=np.clip(p[sl], 1.0, upper), bounds=(np.ones(n), np.full(n, upper)))
        p[sl] = sol.x

    for i, m in enumerate(TWO_MASKS):
        fit_slice(slice(16 + 2 * i, 18 + 2 * i), m)
    for i, m in enumerate(THREE_MASKS):
        fit_slice(slice(4 + 3 * i, 7 + 3 * i), m)
    fit_slice(slice(0, 4), np.ones(4, dtype=bool))
    return [float(v) for v in p]


def fit_fused_overlap(rows: List[Dict]) -> Dict[str, Dict[str, float]]:
    """Fits ``fused = max(gemm, coll) + kappa * min(gemm, coll) + tau`` per kind of fused kernel from the rows
    that :mod:`mist_b200.tools.bench_fused_collectives` writes (``fused_ms``, ``gemm_ms``, ``collective_ms``).
    ``kappa`` is kept in [0, 1.5] (0: the shorter part is hidden completely, 1: nothing overlaps), ``tau`` >= 0;
    the fit minimises relative residuals.  With fewer than three rows per kind ``tau`` stays 0."""
    kinds = {"AG->GEMM": "ag_gemm", "GEMM->RS": "gemm_rs", "ZeRO-3": "zero3_gather"}
    groups: Dict[str, List[Tuple[float, float, float]]] = {}
    for r in rows:
        if "gemm_ms" not in r or "(add)" in r.get("kernel", ""):
            continue
        for prefix, key in kinds.items():
            if r["kernel"].startswith(prefix):
                groups.setdefault(key, []).append((r["fused_ms"] * 1e-3, r["gemm_ms"] * 1e-3, r["collective_ms"] * 1e-3))
    from scipy.optimize import least_squares
    out = {}
    for key, pts in groups.items():
        f = np.array([p[0] for p in pts])
        hi = np.array([max(p[1], p[2]) for p in pts])
        lo = np.array([min(p[1], p[2]) for p in pts])

        def resid(x):
            return (hi + x[0] * lo + x[1] - f) / f          # relative: short and long kernels weigh the same

        if len(pts) >= 3:
            sol = least_squares(resid, x0=[0.5, 0.0], bounds=([0.0, 0.0], [1.5, 1e-2]))
            kappa, tau = float(sol.x[0]), float(sol.x[1])
        else:
            sol = least_squares(lambda x: resid([x[0], 0.0]), x0=[0.5], bounds=([0.0], [1.5]))
            kappa, tau = float(sol.x[0]), 0.0
        out[key] = {"kappa": round(kappa, 4), "tau": round(tau, 7), "rows": len(pts)}
    return out


def fit_all(records: List[Dict]) -> Dict[str, List[float]]:
    """``records``: output of :mod:`mist_b200.tools.profile_interference` -- dicts with the
    per-channel standalone times ``C``, ``G2G``, ``C2G``, ``G2C``, the concurrent ``latency``,
    message sizes and group sizes."""
    comm_only = [dict(gbytes=r["g2g_gbytes"], intra=r["intra"], inter=r["inter"], latency=r["latency"])
                 for r in records if r["C"] == 0 and r["C2G"] == 0 and r["G2C"] == 0 and r["G2G"] > 0]
    g2g = fit_gpu_gpu_params(comm_only) if comm_only else None
    c2g_rows = [r for r in records if r["C"] == 0 and r["G2G"] == 0 and r["G2C"] == 0 and r["C2G"] > 0]
    g2c_rows = [r for r in records if r["C"] == 0 and r["G2G"] == 0 and r["C2G"] == 0 and r["G2C"] > 0]
    out: Dict[str, List[float]] = {}
    if g2g:
        out["gpu_gpu_comm_params"] = g2g
    if c2g_rows:
        out["cpu_gpu_comm_params"] = fit_host_copy_params([r["c2g_gbytes"] for r in c2g_rows],
                                                          [r["latency"] for r in c2g_rows])
    if g2c_rows:
        out["gpu_cpu_comm_params"] = fit_host_copy_params([r["g2c_gbytes"] for r in g2c_rows],
                                                          [r["latency"] for r in g2c_rows])
    multi = [r for r in records if sum(r[k] > 0 for k in ("C", "G2G", "C2G", "G2C")) >= 2]
    if multi:
        out["interference_model_params"] = fit_interference_params(
            [r["C"] for r in multi], [r["G2G"] for r in multi], [r["C2G"] for r in multi],
            [r["G2C"] for r in multi], [r["latency"] for r in multi])
    return out


def main(argv=None):
    """``comm_model.py calib.json [more.json ...]`` prints the fitted communication and interference
    parameters of the calibration records in the files; ``--fused rows.json [...]`` fits the overlap terms of
    the fused GEMM + collective kernels instead and, with ``--meta <_meta.json>``, writes them into the
    operator database's meta file under ``fused_overlap``."""
    import argparse
    import json
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("files", nargs="+")
    ap.add_argument("--fused", action="store_true", help="the files hold rows of bench_fused_collectives")
    ap.add_argument("--meta", default=None, help="operator database meta file to update (with --fused)")
    args = ap.parse_args(argv)
    recs = []
    for f in args.files:
        recs.extend(json.load(open(f)))
    if not args.fused:
        print(json.dumps(fit_all(recs), indent=1))
        return
    fit = fit_fused_overlap(recs)
    print(json.dumps(fit, indent=1))
    if args.meta:
        meta = json.load(open(args.meta))
        meta["fused_overlap"] = fit
        with open(args.meta, "w") as fh:
            json.dump(meta, fh, indent=1)
            fh.write("\n")


if __name__ == "__main__":
    main()
