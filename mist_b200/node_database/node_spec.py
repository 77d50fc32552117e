"""Operator identity for the latency database.

A :class:`NodeSpec` is an operator name plus a flat dictionary of shape / flag attributes
with concrete values; its canonical string is the database key.  Symbolic specs (values
may be sympy expressions in the micro batch size) are concretised with a mapping before
lookup (reference: mist/node_database/node_spec.py:203-476 NodeSpec and ``profile``,
mist/node_database/symbolic_node_spec.py:104-308).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

import sympy as sp


def _concrete(v, mapping: Optional[Mapping]) -> Any:
    if isinstance(v, sp.Basic):
        if mapping:
            v = v.subs({(sp.Symbol(k, integer=True, positive=True) if isinstance(k, str) else k): val
                        for k, val in mapping.items()})
        if v.free_symbols:
            raise ValueError(f"unbound symbols in spec value {v}")
        f = float(v)
        return int(round(f)) if abs(f - round(f)) < 1e-9 else f
    if isinstance(v, bool) or v is None or isinstance(v, (int, float, str)):
        return v
    return str(v)


@dataclass(frozen=True)
class NodeSpec:
    op: str
    attrs: Tuple[Tuple[str, Any], ...]

    @classmethod
    def from_dict(cls, spec: Dict[str, Any], mapping: Optional[Mapping] = None) -> "NodeSpec":
        items = tuple(sorted((k, _concrete(v, mapping)) for k, v in spec.items() if k != "op"))
        return cls(str(spec["op"]), items)

    def key(self) -> str:
        return self.op + "(" + ",".join(f"{k}={v}" for k, v in self.attrs) + ")"

    def get(self, name: str, default=None):
        for k, v in self.attrs:
            if k == name:
                return v
        return default

    def as_dict(self) -> Dict[str, Any]:
        d = dict(self.attrs)
        d["op"] = self.op
        return d

    def __repr__(self):
        return self.key()
