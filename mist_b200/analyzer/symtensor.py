"""Shape-symbolic tensors and the tracer that records what a model does to them.

Running the *real* model code on :class:`SymTensor` inputs yields an explicit IR: a list
of :class:`Node` records, one per operator, each with symbolic output sizes, the tensors
autograd would keep for the backward pass, FLOP / byte counts for both passes, scratch
workspace and any tensor-parallel collective it implies.  Nothing is executed and nothing
in ``torch`` is patched: ``torch`` functions reach the rule table through the
``__torch_function__`` protocol, and the framework's own fused ops
(:mod:`mist_b200.ops.functional`) dispatch on the argument type.

This replaces the reference's symbolic front end -- sympy values smuggled through a
patched ``torch`` (mist/overrides/*, mist/sym_torch/symbolic_tensor.py:40-168, the ~200
wrapped ops under mist/sym_torch/impl/*, the fused-kernel rules in
mist/modules/sym_register.py:54-620) and the FX tracer plus interpreter that recover the
saved tensors afterwards (mist/tracer/symbolic_tracer.py:353-742,
mist/analyzer/recorder.py:295-519) -- by a single pass that records everything at once.
"""
from __future__ import annotations

import contextlib
import itertools
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import sympy as sp
import torch

Expr = Any  # int | sympy expression

_ITEMSIZE = {torch.bfloat16: 2, torch.float16: 2, torch.float32: 4, torch.int64: 8, torch.int32: 4,
             torch.bool: 1, torch.uint8: 1, torch.float64: 8}


def prod(xs) -> Expr:
    out = 1
    for x in xs:
        out = out * x
    return out


def simplify_int(x):
    if isinstance(x, sp.Basic):
        x = sp.simplify(x) if x.free_symbols else x
        if not x.free_symbols and x.is_number:
            f = float(x)
            return int(f) if f.is_integer() else f
    return x


@dataclass
class TensorInfo:
    tid: int                 # storage identity (views share it)
    nbytes: Expr
    is_param: bool = False
    requires_grad: bool = False
    label: str = ""


@dataclass
class Comm:
    kind: str                # all_gather | reduce_scatter | all_reduce
    nbytes: Expr             # size of the full (gathered / to-be-reduced) message
    group: str = "tp"
    overlappable: bool = False


@dataclass
class Node:
    op: str
    scope: str
    inputs: List[int]
    outputs: List[TensorInfo]
    saved: List[int] = field(default_factory=list)      # storages kept for the backward pass
    saved_extra: Expr = 0                                # small extra state (statistics, lse)
    fwd_workspace: Expr = 0
    bwd_workspace: Expr = 0
    flops_fwd: Expr = 0
    flops_bwd: Expr = 0
    bytes_fwd: Expr = 0
    bytes_bwd: Expr = 0
    comm_fwd: Optional[Comm] = None
    comm_bwd: Optional[Comm] = None
    spec: Dict[str, Any] = field(default_factory=dict)  # key of the op-latency database
    grad_bytes: Expr = 0                                 # gradients w.r.t. inputs produced in backward
    index: int = 0


class Graph:
    def __init__(self):
        self.nodes: List[Node] = []
        self.tensors: Dict[int, TensorInfo] = {}
        self.inputs: List[int] = []
        self.params: Dict[int, TensorInfo] = {}

    def scopes(self) -> List[str]:
        seen = []
        for n in self.nodes:
            if n.scope not in seen:
                seen.append(n.scope)
        return seen

    def nodes_of(self, scope: str) -> List[Node]:
        return [n for n in self.nodes if n.scope == scope]


class _Tracer:
    def __init__(self):
        self.graph = Graph()
        self.scope = "pre"
        self._ids = itertools.count(1)
        self.param_cache: Dict[int, Any] = {}     # id(parameter) -> (parameter, SymTensor), for this trace only

    def new_id(self) -> int:
        return next(self._ids)


_TRACER: Optional[_Tracer] = None


def active() -> bool:
    return _TRACER is not None


@contextlib.contextmanager
def tracing():
    """``with tracing() as graph:`` -- every op applied to a SymTensor is recorded."""
    global _TRACER
    prev, _TRACER = _TRACER, _Tracer()
    try:
        yield _TRACER.graph
    finally:
        _TRACER = prev


def set_scope(name: str):
    if _TRACER is not None:
        _TRACER.scope = name


def current_scope() -> str:
    return _TRACER.scope if _TRACER is not None else ""


class SymTensor:
    """A tensor known only by (symbolic) shape, dtype and storage identity."""

    __slots__ = ("shape", "dtype", "tid", "requires_grad", "is_param", "label", "contiguous_", "base_bytes")

    def __init__(self, shape: Sequence[Expr], dtype=torch.bfloat16, tid: Optional[int] = None,
                 requires_grad: bool = False, is_param: bool = False, label: str = "", base_bytes=None):
        self.shape = tuple(shape)
        self.dtype = dtype
        self.tid = tid if tid is not None else (_TRACER.new_id() if _TRACER else 0)
        self.requires_grad = requires_grad
        self.is_param = is_param
        self.label = label
        self.contiguous_ = True
        self.base_bytes = base_bytes   # bytes of the underlying storage when this is a view
        if _TRACER is not None and self.tid not in _TRACER.graph.tensors:
            info = TensorInfo(self.tid, self.storage_bytes, is_param, requires_grad, label)
            _TRACER.graph.tensors[self.tid] = info
            if is_param:
                _TRACER.graph.params[self.tid] = info

    # ------------------------------------------------------------------ tensor protocol
    @property
    def nbytes(self) -> Expr:
        return prod(self.shape) * _ITEMSIZE[self.dtype]

    @property
    def storage_bytes(self) -> Expr:
        return self.base_bytes if self.base_bytes is not None else self.nbytes

    @property
    def device(self):
        return torch.device("meta")

    @property
    def is_cuda(self):
        return False

    @property
    def ndim(self):
        return len(self.shape)

    def dim(self):
        return len(self.shape)

    def size(self, d=None):
        return self.shape if d is None else self.shape[d]

    def numel(self):
        return prod(self.shape)

    def stride(self, d=None):
        st, acc = [], 1
        for s in reversed(self.shape):
            st.append(acc)
            acc = acc * s
        st = tuple(reversed(st))
        return st if d is None else st[d]

    def is_contiguous(self):
        return self.contiguous_

    def data_ptr(self):
        return 0

    def element_size(self):
        return _ITEMSIZE[self.dtype]

    def _view(self, shape, contiguous=True) -> "SymTensor":
        v = SymTensor(shape, self.dtype, tid=self.tid, requires_grad=self.requires_grad, is_param=self.is_param,
                      label=self.label, base_bytes=self.storage_bytes)
        v.contiguous_ = contiguous and self.contiguous_
        return v

    # views -------------------------------------------------------------------------------
    def _resolve_shape(self, shape):
        shape = list(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)) else list(shape)
        if -1 in shape:
            known = prod(s for s in shape if not (isinstance(s, int) and s == -1))
            shape[shape.index(-1)] = simplify_int(sp.Integer(1) * self.numel() / known)
        return tuple(shape)

    def view(self, *shape):
        return self._view(self._resolve_shape(shape))

    def reshape(self, *shape):
        shp = self._resolve_shape(shape)
        if not self.contiguous_:
            return contiguous(self)._view(shp)
        return self._view(shp)

    def view_as(self, other):
        return self._view(other.shape)

    def contiguous(self):
        return contiguous(self)

    def transpose(self, a, b):
        shp = list(self.shape)
        shp[a], shp[b] = shp[b], shp[a]
        return self._view(shp, contiguous=False)

    def permute(self, *dims):
        dims = dims[0] if len(dims) == 1 and isinstance(dims[0], (tuple, list)) else dims
        return self._view([self.shape[d] for d in dims], contiguous=False)

    def t(self):
        return self.transpose(0, 1)

    def unsqueeze(self, d):
        shp = list(self.shape)
        shp.insert(d if d >= 0 else len(shp) + d + 1, 1)
        return self._view(shp)

    def squeeze(self, d=None):
        shp = [s for i, s in enumerate(self.shape) if not ((d is None or i == d % len(self.shape)) and s == 1)]
        return self._view(shp)

    def chunk(self, n, dim=-1):
        shp = list(self.shape)
        shp[dim] = simplify_int(sp.Integer(1) * shp[dim] / n)
        return tuple(self._view(shp, contiguous=False) for _ in range(n))

    def detach(self):
        v = self._view(self.shape)
        v.requires_grad = False
        return v

    def requires_grad_(self, flag=True):
        self.requires_grad = flag
        return self

    def __getitem__(self, idx):
        if not isinstance(idx, tuple):
            idx = (idx,)
        shp, d = [], 0
        for it in idx:
            if it is Ellipsis:
                keep = len(self.shape) - (len(idx) - 1) - d
                shp.extend(self.shape[d:d + keep])
                d += keep
            elif isinstance(it, slice):
                n = self.shape[d]
                if it.start is None and it.stop is None:
                    shp.append(n)
                else:
                    start = it.start or 0
                    stop = n if it.stop is None else it.stop
                    shp.append(simplify_int(stop - start))
                d += 1
            elif it is None:
                shp.append(1)
            elif isinstance(it, SymTensor):      # advanced indexing with an index tensor
                return index_select(self, it, d)
            else:
                d += 1                            # integer index drops the dimension
        shp.extend(self.shape[d:])
        return self._view(shp, contiguous=False)

    # dtype casts -------------------------------------------------------------------------
    def to(self, *args, **kwargs):
        dtype = kwargs.get("dtype")
        for a in args:
            if isinstance(a, torch.dtype):
                dtype = a
        if dtype is None or dtype == self.dtype:
            return self
        return cast(self, dtype)

    def float(self):
        return self.to(torch.float32)

    def half(self):
        return self.to(torch.float16)

    def bfloat16(self):
        return self.to(torch.bfloat16)

    # arithmetic --------------------------------------------------------------------------
    def __add__(self, o):
        return elementwise("add", self, o)

    __radd__ = __add__

    def __mul__(self, o):
        return elementwise("mul", self, o)

    __rmul__ = __mul__

    def __sub__(self, o):
        return elementwise("sub", self, o)

    def __truediv__(self, o):
        return elementwise("div", self, o)

    def mean(self, *a, **k):
        return reduce_all("mean", self)

    def sum(self, *a, **k):
        return reduce_all("sum", self)

    def backward(self, *a, **k):
        return None

    def item(self):
        return 0.0

    def __repr__(self):
        return f"SymTensor({list(self.shape)}, {str(self.dtype).replace('torch.', '')}, id={self.tid})"

    # ------------------------------------------------------------------- torch dispatch
    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        rule = TORCH_RULES.get(func)
        if rule is None:
            name = getattr(func, "__name__", str(func))
            raise NotImplementedError(f"no symbolic rule for torch function '{name}'")
        return rule(*args, **kwargs)


def is_sym(*xs) -> bool:
    return any(isinstance(x, SymTensor) for x in xs)


# ------------------------------------------------------------------------------ recording


def record(op: str, inputs: Sequence, out_shapes: Sequence[Tuple[Sequence[Expr], torch.dtype]], *,
           saved: Sequence = (), saved_extra: Expr = 0, flops_fwd: Expr = 0, flops_bwd: Expr = 0,
           bytes_fwd: Optional[Expr] = None, bytes_bwd: Optional[Expr] = None, fwd_workspace: Expr = 0,
           bwd_workspace: Expr = 0, comm_fwd: Optional[Comm] = None, comm_bwd: Optional[Comm] = None,
           spec: Optional[Dict] = None, save_outputs: Sequence[int] = (), grad_inputs: Optional[Sequence] = None):
    """Appends a node and returns its output SymTensors."""
    sym_in = [x for x in inputs if isinstance(x, SymTensor)]
    req = any(x.requires_grad for x in sym_in)
    outs = [SymTensor(shp, dt, requires_grad=req and dt in (torch.bfloat16, torch.float16, torch.float32))
            for shp, dt in out_shapes]
    if _TRACER is None:
        return outs
    in_bytes = sum((x.nbytes for x in sym_in), 0)
    out_bytes = sum((o.nbytes for o in outs), 0)
    if bytes_fwd is None:
        bytes_fwd = in_bytes + out_bytes
    gi = sym_in if grad_inputs is None else [x for x in grad_inputs if isinstance(x, SymTensor)]
    grad_bytes = sum((x.nbytes for x in gi if x.requires_grad and not x.is_param), 0) if req else 0
    if bytes_bwd is None:
        bytes_bwd = (out_bytes + in_bytes + grad_bytes) if req else 0
    saved_ids = [x.tid for x in saved if isinstance(x, SymTensor)] if req else []
    saved_ids += [outs[i].tid for i in save_outputs] if req else []
    node = Node(op=op, scope=_TRACER.scope, inputs=[x.tid for x in sym_in],
                outputs=[_TRACER.graph.tensors[o.tid] for o in outs], saved=saved_ids,
                saved_extra=saved_extra if req else 0, fwd_workspace=fwd_workspace,
                bwd_workspace=bwd_workspace if req else 0, flops_fwd=flops_fwd, flops_bwd=flops_bwd if req else 0,
                bytes_fwd=bytes_fwd, bytes_bwd=bytes_bwd, comm_fwd=comm_fwd, comm_bwd=comm_bwd if req else None,
                spec=spec or {"op": op}, grad_bytes=grad_bytes, index=len(_TRACER.graph.nodes))
    _TRACER.graph.nodes.append(node)
    return outs


# ----------------------------------------------------------------------- generic op rules
def _bshape(a, b):
    sa = a.shape if isinstance(a, SymTensor) else ()
    sb = b.shape if isinstance(b, SymTensor) else ()
    n = max(len(sa), len(sb))
    sa = (1,) * (n - len(sa)) + tuple(sa)
    sb = (1,) * (n - len(sb)) + tuple(sb)
    return tuple(y if (isinstance(x, int) and x == 1) else x for x, y in zip(sa, sb))


def elementwise(kind: str, a, b=None, out_dtype=None, saves_input: bool = False):
    ref = a if isinstance(a, SymTensor) else b
    shape = _bshape(a, b) if b is not None else ref.shape
    dt = out_dtype or ref.dtype
    if isinstance(a, SymTensor) and isinstance(b, SymTensor) and a.dtype != b.dtype:
        dt = torch.float32 if torch.float32 in (a.dtype, b.dtype) else a.dtype
    n = prod(shape)
    saved = [x for x in (a, b) if isinstance(x, SymTensor)] if (saves_input or kind in ("mul", "div")) else []
    (out,) = record(kind, [a, b], [(shape, dt)], saved=saved, flops_fwd=n, flops_bwd=2 * n)
    return out


def unary(kind: str, x: SymTensor, save: str = "input", flops_per_elem: int = 8):
    n = x.numel()
    (out,) = record(kind, [x], [(x.shape, x.dtype)], saved=[x] if save == "input" else [],
                    save_outputs=[0] if save == "output" else [], flops_fwd=flops_per_elem * n,
                    flops_bwd=flops_per_elem * n)
    return out


def cast(x: SymTensor, dtype):
    (out,) = record("cast", [x], [(x.shape, dtype)])
    return out


def contiguous(x: SymTensor):
    if x.contiguous_:
        return x
    (out,) = record("copy", [x], [(x.shape, x.dtype)])
    return out


def reduce_all(kind: str, x: SymTensor):
    (out,) = record(kind, [x], [((), torch.float32)], flops_fwd=x.numel())
    return out


def index_select(table: SymTensor, idx: SymTensor, dim: int = 0):
    shp = tuple(idx.shape) + tuple(table.shape[dim + 1:])
    (out,) = record("gather", [table, idx], [(shp, table.dtype)], saved=[idx],
                    bytes_fwd=2 * prod(shp) * _ITEMSIZE[table.dtype])
    return out


def matmul(a: SymTensor, b: SymTensor):
    # [..., m, k] @ [..., k, n]
    m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    batch = a.shape[:-2] if len(a.shape) >= len(b.shape) else b.shape[:-2]
    fl = 2 * prod(batch) * m * k * n
    (out,) = record("bmm", [a, b], [(tuple(batch) + (m, n), a.dtype)], saved=[a, b], flops_fwd=fl, flops_bwd=2 * fl,
                    spec={"op": "bmm", "batch": prod(batch), "m": m, "n": n, "k": k})
    return out


def linear_torch(x, weight, bias=None):
    from . import rules
    return rules.linear(x, weight, bias, None, None)


def softmax(x: SymTensor, dim=-1, **_):
    return unary("softmax", x, save="output", flops_per_elem=10)


def dropout(x, p=0.5, training=True, inplace=False):
    if not training or p == 0:
        return x
    (out,) = record("dropout", [x], [(x.shape, x.dtype)], saved_extra=x.numel(), flops_fwd=4 * x.numel(),
                    flops_bwd=2 * x.numel())
    return out


def cat(tensors, dim=0):
    ref = tensors[0]
    shp = list(ref.shape)
    shp[dim] = sum(t.shape[dim] for t in tensors)
    (out,) = record("cat", list(tensors), [(shp, ref.dtype)])
    return out


def cross_entropy_torch(logits, target, **kw):
    n = logits.numel()
    (out,) = record("cross_entropy", [logits, target], [((), torch.float32)], saved=[logits, target],
                    flops_fwd=6 * n, flops_bwd=4 * n)
    return out


def layer_norm_torch(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    from . import rules
    return rules.norm(x, None, weight, bias, eps, False, False)


def sdpa_torch(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False):
    from . import rules
    return rules.attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), scale, is_causal).transpose(1, 2)


TORCH_RULES: Dict[Callable, Callable] = {
    torch.matmul: matmul,
    torch.bmm: matmul,
    torch.tanh: lambda x: unary("tanh", x, save="output"),
    torch.sigmoid: lambda x: unary("sigmoid", x, save="output"),
    torch.nn.functional.gelu: lambda x, approximate="none": unary("gelu", x),
    torch.nn.functional.silu: lambda x, inplace=False: unary("silu", x),
    torch.nn.functional.relu: lambda x, inplace=False: unary("relu", x, save="output", flops_per_elem=1),
    torch.nn.functional.linear: linear_torch,
    torch.nn.functional.softmax: softmax,
    torch.softmax: softmax,
    torch.nn.functional.dropout: dropout,
    torch.nn.functional.cross_entropy: cross_entropy_torch,
    torch.nn.functional.layer_norm: layer_norm_torch,
    torch.nn.functional.scaled_dot_product_attention: sdpa_torch,
    torch.nn.functional.embedding: lambda idx, weight, *a, **k: index_select(weight, idx, 0),
    torch.cat: cat,
    torch.add: lambda a, b, **k: elementwise("add", a, b),
    torch.mul: lambda a, b: elementwise("mul", a, b),
    torch.transpose: lambda x, a, b: x.transpose(a, b),
    torch.reshape: lambda x, shape: x.reshape(shape),
    torch.Tensor.__add__: lambda a, b: elementwise("add", a, b),
    torch.Tensor.__radd__: lambda a, b: elementwise("add", a, b),
    torch.Tensor.add: lambda a, b, **k: elementwise("add", a, b),
    torch.Tensor.__mul__: lambda a, b: elementwise("mul", a, b),
    torch.Tensor.__rmul__: lambda a, b: elementwise("mul", a, b),
    torch.Tensor.__getitem__: lambda t, idx: index_select(as_sym_param(t), idx, 0),
}


def as_sym_param(p) -> SymTensor:
    """SymTensor standing for a real (usually meta-device) parameter; one per parameter and trace."""
    if isinstance(p, SymTensor) or p is None:
        return p
    cache = _TRACER.param_cache if _TRACER is not None else {}
    hit = cache.get(id(p))
    if hit is not None and hit[0] is p:
        return hit[1]
    st = SymTensor(tuple(p.shape), p.dtype, requires_grad=bool(getattr(p, "requires_grad", False)), is_param=True,
                   label="param")
    cache[id(p)] = (p, st)      # keeping the parameter alive keeps its id unique within the trace
    return st
