"""Start-up adjustments that let the unmodified reference import under the library versions of this image
(torch 2.11, transformers 5.x).  Each one adds a name the reference expects and the newer library no
longer exports; nothing in the reference tree is edited.  Imported by baseline/run_reference.py before
``import mist``."""
from __future__ import annotations

import importlib
import sys

APPLIED = []


def _note(what):
    APPLIED.append(what)


def apply():
    from packaging import version
    import transformers.utils as tu
    if not hasattr(tu, "TORCH_FX_REQUIRED_VERSION"):
        tu.TORCH_FX_REQUIRED_VERSION = version.parse("1.10")
        _note("transformers.utils.TORCH_FX_REQUIRED_VERSION")
    if not hasattr(tu, "is_torch_fx_available"):
        tu.is_torch_fx_available = lambda: True
        _note("transformers.utils.is_torch_fx_available")
    if not hasattr(tu, "ENV_VARS_TRUE_VALUES"):
        tu.ENV_VARS_TRUE_VALUES = {"1", "ON", "YES", "TRUE"}
        _note("transformers.utils.ENV_VARS_TRUE_VALUES")
    if not hasattr(tu, "is_peft_available"):
        tu.is_peft_available = lambda: False
        _note("transformers.utils.is_peft_available")
    import types
    import torch
    # torch's functional optimizers are TorchScript classes compiled at import; the reference wraps
    # torch.jit.script (mist/overrides/jit.py), which breaks the name lookup of that compilation, so the
    # module is imported before the wrapper exists
    import torch.distributed.optim  # noqa: F401
    if "torch.distributed.pipeline" not in sys.modules:
        try:
            importlib.import_module("torch.distributed.pipeline")
        except ImportError:
            # removed from torch; the reference imports it and uses nothing of it
            mod = types.ModuleType("torch.distributed.pipeline")
            sys.modules["torch.distributed.pipeline"] = mod
            torch.distributed.pipeline = mod
            _note("torch.distributed.pipeline (empty module)")
    import torch.optim.adam as _adam
    import torch.optim.adamw as _adamw
    for new, old in (("_fused_adamw", "_fused_adam"), ("_single_tensor_adamw", "_single_tensor_adam")):
        if not hasattr(_adamw, new):
            # imported by name in mist/optimizers/fused_adam.py:6-7, referenced only in comments there
            setattr(_adamw, new, getattr(_adam, old))
            _note(f"torch.optim.adamw.{new}")
    import torch.distributed.fsdp as _fsdp
    if "torch.distributed.fsdp.flat_param" not in sys.modules:
        try:
            importlib.import_module("torch.distributed.fsdp.flat_param")
        except ImportError:
            priv = importlib.import_module("torch.distributed.fsdp._flat_param")
            sys.modules["torch.distributed.fsdp.flat_param"] = priv
            _fsdp.flat_param = priv
            _note("torch.distributed.fsdp.flat_param -> _flat_param")
    import einops.einops as ee
    if not hasattr(ee, "is_ellipsis_not_in_parenthesis"):
        # helper of einops <= 0.7 that the reference imports by name
        ee.is_ellipsis_not_in_parenthesis = lambda group: len(group) == 1 and group[0] == -999
        _note("einops.einops.is_ellipsis_not_in_parenthesis")
    global _EINOPS_RECONSTRUCT
    _EINOPS_RECONSTRUCT = ee._reconstruct_from_shape
    return APPLIED


_EINOPS_RECONSTRUCT = None


def after_import():
    """The reference replaces ``einops.einops._reconstruct_from_shape`` with a sympy-aware copy written
    against einops 0.6 (two arguments, recipe fields that no longer exist).  Execution works on concrete
    shapes, so the library's own function is put back once ``mist`` is imported."""
    import einops.einops as ee
    if _EINOPS_RECONSTRUCT is not None and ee._reconstruct_from_shape is not _EINOPS_RECONSTRUCT:
        ee._reconstruct_from_shape = _EINOPS_RECONSTRUCT
        _note("einops.einops._reconstruct_from_shape restored after import")
