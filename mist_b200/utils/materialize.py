"""Building a model without memory and giving it memory later.

``empty_init()`` constructs modules on the meta device (shapes and dtypes only), which is how the
analyzer looks at models far larger than the host's RAM; ``materialize_module`` then allocates the
parameters on a real device and initialises them, ``materialize_tensor`` does the same for a single
tensor or meta tensor.

Reference: ``init_empty_weights`` (mist/utils/initialization.py:15-39), ``materialize_tensor`` /
``materialize_module`` (mist/utils/memory.py:100-282).  The reference picks an initialiser from the
class name; here a module that defines ``reset_parameters`` is asked to initialise itself (every layer
of this package does), and the class-name rules only cover foreign modules.
"""
from __future__ import annotations

import contextlib
from typing import Optional, Sequence

import torch
import torch.nn as nn


@contextlib.contextmanager
def empty_init(enable: bool = True):
    """Modules created inside allocate nothing: their parameters and buffers live on the meta device."""
    if not enable:
        yield
        return
    with torch.device("meta"):
        yield


def materialize_tensor(t, device="cpu", rand: bool = True, bound: float = 1e-2):
    """A real tensor with the shape / dtype / requires_grad of ``t`` (anything that is not a tensor is
    returned as is).  Floating point: N(0, ``bound``) when ``rand`` else zeros; integers: zeros or ones
    (valid indices for any table); booleans: random bits or zeros."""
    if not isinstance(t, torch.Tensor):
        return t
    device = torch.device(device)
    if t.dtype == torch.bool:
        out = (torch.rand(t.shape, device=device) < 0.5) if rand else torch.zeros(t.shape, dtype=torch.bool, device=device)
    elif t.dtype.is_floating_point or t.dtype.is_complex:
        out = torch.empty(t.shape, dtype=t.dtype, device=device)
        out.normal_(0.0, bound) if rand else out.zero_()
    else:
        out = torch.ones(t.shape, dtype=t.dtype, device=device) if rand else torch.zeros(t.shape, dtype=t.dtype, device=device)
    return out.requires_grad_(t.requires_grad) if out.dtype.is_floating_point else out


def _init_foreign(mod: nn.Module):
    name = type(mod).__name__.lower()
    w, b = getattr(mod, "weight", None), getattr(mod, "bias", None)
    with torch.no_grad():
        if "norm" in name:
            if w is not None:
                w.fill_(1.0)
            if b is not None:
                b.zero_()
        elif "embedding" in name:
            if w is not None:
                w.normal_(0.0, 1.0)
        elif "linear" in name or "dense" in name:
            if w is not None:
                nn.init.kaiming_uniform_(w, a=5 ** 0.5)
            if b is not None:
                b.zero_()
        else:
            for p in mod.parameters(recurse=False):
                p.normal_(0.0, 1e-2)


def materialize_module(mod: nn.Module, device="cpu", ignored: Optional[Sequence[nn.Module]] = None) -> nn.Module:
    """Gives every meta-device parameter and buffer of ``mod`` storage on ``device`` (in place) and
    initialises it; what already lives on a real device is only moved.  Parameters shared between
    modules stay shared.  ``ignored`` sub-modules are left untouched."""
    device = torch.device(device)
    skip = set(id(m) for m in (ignored or ()))
    for sub in mod.modules():
        if id(sub) in skip:
            continue
        was_meta = [n for n, p in sub.named_parameters(recurse=False) if p.is_meta]
        was_meta += [n for n, b in sub.named_buffers(recurse=False) if b.is_meta]
        if not was_meta:
            continue
        for n, p in list(sub.named_parameters(recurse=False)):
            if p.is_meta:
                new = nn.Parameter(torch.empty(p.shape, dtype=p.dtype, device=device), requires_grad=p.requires_grad)
                for k, v in p.__dict__.items():     # markers the engine reads (sequence parallel, tied, ...)
                    setattr(new, k, v)
                _replace_everywhere(mod, p, new)
        for n, b in list(sub.named_buffers(recurse=False)):
            if b.is_meta:
                sub._buffers[n] = torch.zeros(b.shape, dtype=b.dtype, device=device)
        if hasattr(sub, "reset_parameters"):
            sub.reset_parameters()
        else:
            _init_foreign(sub)
    mod.to(device)
    left = [n for n, p in mod.named_parameters() if p.is_meta and not _under(mod, n, skip)]
    assert not left, f"parameters still on the meta device: {left[:4]}"
    return mod


def _replace_everywhere(root: nn.Module, old: nn.Parameter, new: nn.Parameter):
    for m in root.modules():
        for n, p in list(m._parameters.items()):
            if p is old:
                m._parameters[n] = new


def _under(root: nn.Module, param_name: str, skip) -> bool:
    m = root
    for part in param_name.split(".")[:-1]:
        m = getattr(m, part)
        if id(m) in skip:
            return True
    return False
