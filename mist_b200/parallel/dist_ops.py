"""Collectives along the token dimension (dim 0) with autograd pairs.

``group`` may be ``None`` (single rank: every op is the identity), a real
``torch.distributed`` group, or a :class:`FakeGroup` that only carries a size and a rank:
the analyzer builds models against fake groups so that shapes are the per-rank shapes of
a tensor-parallel run without any communicator (reference: mist/distributed/op.py:22-115
for the op set, mist/distributed/overrides.py:12-100 for the fake group idea).
"""
from __future__ import annotations


import torch
import torch.distributed as dist


class FakeGroup:
    """Stands in for a process group of ``size`` ranks; collectives become local shape ops."""

    def __init__(self, size: int, rank: int = 0):
        self._size, self._rank = int(size), int(rank)

    def size(self):
        return self._size

    def rank(self):
        return self._rank


def group_size(group) -> int:
    if group is None:
        return 1
    if isinstance(group, FakeGroup):
        return group.size()
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None:
        return 0
    if isinstance(group, FakeGroup):
        return group.rank()
    return dist.get_rank(group)


def _is_trivial(group) -> bool:
    return group is None or group_size(group) == 1


def all_gather_raw(x: torch.Tensor, group, async_op: bool = False):
    """Concatenates every rank's ``x`` along dim 0."""
    n = group_size(group)
    if isinstance(group, FakeGroup):
        return x.repeat(n, *([1] * (x.dim() - 1))), None
    x = x.contiguous()
    out = torch.empty(n * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
    handle = dist.all_gather_into_tensor(out, x, group=group, async_op=async_op)
    return out, handle


def reduce_scatter_raw(x: torch.Tensor, group, async_op: bool = False):
    """Sums over ranks and keeps this rank's dim-0 slice."""
    n = group_size(group)
    assert x.shape[0] % n == 0, f"dim 0 ({x.shape[0]}) must divide by the group size ({n})"
    if isinstance(group, FakeGroup):
        return x[: x.shape[0] // n].clone(), None
    x = x.contiguous()
    out = torch.empty(x.shape[0] // n, *x.shape[1:], dtype=x.dtype, device=x.device)
    handle = dist.reduce_scatter_tensor(out, x, group=group, async_op=async_op)
    return out, handle


def all_reduce_raw(x: torch.Tensor, group, async_op: bool = False):
    if isinstance(group, FakeGroup):
        return x, None
    x = x.contiguous()
    handle = dist.all_reduce(x, group=group, async_op=async_op)
    return x, handle


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_raw(x, group)[0]

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_raw(g, ctx.group)[0], None


class _AllGatherSliceGrad(torch.autograd.Function):
    """All-gather whose consumers compute the same thing on every rank (a replicated head after
    the sequence-sharded region): the incoming gradient is already complete and identical on all
    ranks, so the backward pass keeps this rank's slice instead of summing the copies."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_raw(x, group)[0]

    @staticmethod
    def backward(ctx, g):
        n, r = group_size(ctx.group), group_rank(ctx.group)
        per = g.shape[0] // n
        return g[r * per:(r + 1) * per].contiguous(), None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return reduce_scatter_raw(x, group)[0]

    @staticmethod
    def backward(ctx, g):
        return all_gather_raw(g, ctx.group)[0], None


class _AllReduce(torch.autograd.Function):
    """Sum in forward, identity in backward (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        return all_reduce_raw(x.clone() if x.requires_grad else x, group)[0]

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToGroup(torch.autograd.Function):
    """Identity in forward, sum in backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return all_reduce_raw(g.contiguous().clone(), ctx.group)[0], None


def _symbolic(x) -> bool:
    return type(x).__name__ == "SymTensor"


def _rules():
    from ..analyzer import rules
    return rules


def all_gather(x, group, replicated_consumer: bool = False):
    """Gathers dim 0 over the group.  ``replicated_consumer``: what follows is computed
    identically on every rank, so the backward pass slices the gradient instead of
    reduce-scattering it."""
    if _is_trivial(group):
        return x
    if _symbolic(x):
        return _rules().all_gather(x, group)
    return (_AllGatherSliceGrad if replicated_consumer else _AllGather).apply(x, group)


def reduce_scatter(x, group):
    if _is_trivial(group):
        return x
    return _rules().reduce_scatter(x, group) if _symbolic(x) else _ReduceScatter.apply(x, group)


def all_reduce(x, group):
    if _is_trivial(group):
        return x
    return _rules().all_reduce(x, group) if _symbolic(x) else _AllReduce.apply(x, group)


def copy_to_group(x, group):
    if _is_trivial(group):
        return x
    return _rules().copy_to_group(x, group) if _symbolic(x) else _CopyToGroup.apply(x, group)


def sync_shared_params(model: torch.nn.Module, group):
    """Broadcasts parameters tagged ``_shared_params`` from the group's first rank."""
    if _is_trivial(group) or isinstance(group, FakeGroup):
        return
    src = dist.get_global_rank(group, 0)
    for p in model.parameters():
        if getattr(p, "_shared_params", False):
            dist.broadcast(p.data, src=src, group=group)


def allreduce_sequence_parallel_grad(model: torch.nn.Module, group):
    """Sums over the tensor-parallel group the grads of parameters that live in the
    sequence-sharded region (norm weights, row-parallel biases)."""
    if _is_trivial(group) or isinstance(group, FakeGroup):
        return
    grads = [p.grad for p in model.parameters() if getattr(p, "_sequence_parallel", False) and p.grad is not None]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=group)
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off:off + n].view_as(g))
        off += n


def dim_for_rank(dim: int, world_size: int, rank: int, multiple_of: int = 1) -> int:
    """Size of ``rank``'s share when ``dim`` is split as evenly as possible in units of
    ``multiple_of`` (the first ``remainder`` ranks get one extra unit)."""
    units = dim // multiple_of
    base, rem = divmod(units, world_size)
    return (base + (1 if rank < rem else 0)) * multiple_of
