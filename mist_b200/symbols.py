"""Symbol manager: named sympy symbols bound to concrete example values.

Shape-symbolic analysis needs two views of a quantity such as the micro batch size: a
symbol that flows through shape arithmetic, and a concrete stand-in used whenever code
must take a branch (``if x.shape[0] % n == 0``) or allocate something real.  The manager
keeps that mapping, substitutes it into expressions, and checks / solves simple
constraints (reference: mist/symbols.py:47-233 SymbolManager with map / verify / solve /
subs).  Unlike the reference nothing in sympy is monkey-patched: expressions are only
concretised through the explicit helpers below.
"""
from __future__ import annotations

from typing import Dict, Iterable, Optional, Union

import sympy as sp

Number = Union[int, float]


class SymbolManager:
    def __init__(self):
        self._symbols: Dict[str, sp.Symbol] = {}
        self._values: Dict[sp.Symbol, Number] = {}

    # ------------------------------------------------------------------ creation / lookup
    def symbols(self, names: str, concrete: Union[Number, Iterable[Number]], integer: bool = True,
                positive: bool = True):
        """``gsm.symbols("b", 2)`` or ``gsm.symbols("b tp", (2, 1))`` -- creates (or returns)
        symbols and records their concrete stand-ins."""
        parts = names.replace(",", " ").split()
        vals = list(concrete) if isinstance(concrete, (tuple, list)) else [concrete] * len(parts)
        assert len(vals) == len(parts), "one concrete value per symbol"
        out = []
        for n, v in zip(parts, vals):
            s = self._symbols.get(n)
            if s is None:
                s = sp.Symbol(n, integer=integer, positive=positive)
                self._symbols[n] = s
            self._values[s] = v
            out.append(s)
        return out[0] if len(out) == 1 else tuple(out)

    def get(self, name: str) -> sp.Symbol:
        return self._symbols[name]

    def __contains__(self, name: str) -> bool:
        return name in self._symbols

    @property
    def mapping(self) -> Dict[sp.Symbol, Number]:
        return dict(self._values)

    def name_mapping(self) -> Dict[str, Number]:
        return {s.name: v for s, v in self._values.items()}

    # ------------------------------------------------------------------------ evaluation
    def map(self, expr, overrides: Optional[Dict] = None):
        """Concrete value of ``expr`` under the recorded mapping (``overrides`` may rebind
        symbols by object or by name)."""
        if not isinstance(expr, sp.Basic):
            if isinstance(expr, (tuple, list)):
                return type(expr)(self.map(e, overrides) for e in expr)
            return expr
        m = dict(self._values)
        for k, v in (overrides or {}).items():
            m[self._symbols[k] if isinstance(k, str) else k] = v
        val = expr.subs(m)
        if val.free_symbols:
            raise ValueError(f"unbound symbols {val.free_symbols} in {expr}")
        if val.is_integer:
            return int(val)
        f = float(val)
        return int(f) if f.is_integer() and abs(f) < 2 ** 53 else f

    def subs(self, expr, mapping: Dict):
        """Partial substitution by symbol name or object; result may stay symbolic."""
        if not isinstance(expr, sp.Basic):
            return expr
        m = {(self._symbols[k] if isinstance(k, str) else k): v for k, v in mapping.items()}
        return expr.subs(m)

    def verify(self, relation) -> bool:
        """Truth of a relation (``sp.Eq(...)``, ``a < b``...) under the concrete mapping."""
        if isinstance(relation, bool):
            return relation
        return bool(relation.subs(self._values))

    def solve(self, equation, for_symbol) -> list:
        s = self._symbols[for_symbol] if isinstance(for_symbol, str) else for_symbol
        return sp.solve(equation, s)

    def lambdify(self, expr, arg_names: Iterable[str]):
        """Numpy-callable version of ``expr`` in the named symbols (missing ones are bound
        to their concrete stand-ins first)."""
        args = [self._symbols[n] for n in arg_names]
        if not isinstance(expr, sp.Basic):
            const = expr
            return lambda *a, **k: const
        rest = {s: v for s, v in self._values.items() if s not in args}
        return sp.lambdify(args, expr.subs(rest), modules="numpy")

    def reset(self):
        self._symbols.clear()
        self._values.clear()


#: process-wide manager, same role as the reference's ``gsm``
gsm = SymbolManager()


def concrete(x, manager: SymbolManager = gsm):
    return manager.map(x)


def is_symbolic(x) -> bool:
    return isinstance(x, sp.Basic) and bool(x.free_symbols)
