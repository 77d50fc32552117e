"""``summary.json`` accumulated across the analyze / tune / exec entry points.

Keys and value formats follow the reference (benchmark/mist/analysis/run.py:221-243,
tune/tune_one_case.py:441-450, exec/benchmark_one_case.py:603-621): costs are formatted
strings with four decimals, memories are ``"[123 MB, ...]"`` strings.
"""
from __future__ import annotations

import fcntl
import json
import os
from typing import Any, Dict


def update_summary(path: str, updates: Dict[str, Any]) -> Dict[str, Any]:
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    lock = path + ".lock"
    with open(lock, "w") as lf:
        fcntl.flock(lf, fcntl.LOCK_EX)
        data = {}
        if os.path.exists(path):
            try:
                with open(path) as f:
                    data = json.load(f)
            except (json.JSONDecodeError, OSError):
                data = {}
        data.update(updates)
        with open(path, "w") as f:
            json.dump(data, f, indent=4)
        fcntl.flock(lf, fcntl.LOCK_UN)
    return data


def fmt_cost(x: float) -> str:
    return f"{x:.4f}"


def fmt_costs(xs) -> str:
    return "[" + ", ".join(f"{x:.4f}" for x in xs) + "]"


def fmt_memories(xs_bytes) -> str:
    return "[" + ", ".join(f"{x / (1 << 20):.0f} MB" for x in xs_bytes) + "]"
