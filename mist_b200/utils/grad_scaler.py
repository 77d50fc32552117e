"""Loss scaling for fp16 training.

``ConstantGradScaler`` multiplies the loss by a fixed factor before the backward pass; the
engine folds the inverse into the optimizer kernel's gradient divisor, so no separate
unscale pass runs over the gradients.  ``unscale_`` (explicit unscale + non-finite check) is
there for callers that step their own optimizer (reference: mist/optimizers/grad_scaler.py:
7-41, a constant scaler with the same three operations).
"""
from __future__ import annotations

from typing import Iterable

import torch


class ConstantGradScaler:
    def __init__(self, scale: float = 1.0, device=None):
        assert scale > 0.0
        self._scale = float(scale)
        self.found_inf = torch.zeros(1, dtype=torch.float32, device=device or "cpu")

    @property
    def loss_scale(self) -> float:
        return self._scale

    @property
    def inv_scale(self) -> float:
        return 1.0 / self._scale

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self._scale if self._scale != 1.0 else loss

    def unscale_(self, grads: Iterable[torch.Tensor]) -> bool:
        """Divides ``grads`` by the scale in place; returns True when any value was inf / nan
        (also recorded in ``found_inf``)."""
        grads = [g for g in grads if g is not None]
        if not grads:
            return False
        self.found_inf = self.found_inf.to(grads[0].device)
        self.found_inf.zero_()
        inv = torch.full((1,), self.inv_scale, dtype=torch.float32, device=grads[0].device)
        if grads[0].is_cuda:
            torch._amp_foreach_non_finite_check_and_unscale_(grads, self.found_inf, inv)
        else:
            for g in grads:
                if not torch.isfinite(g).all():
                    self.found_inf.fill_(1.0)
                g.mul_(self.inv_scale)
        return bool(self.found_inf.item() > 0)

    def step(self, optimizer, closure=None):
        return optimizer.step(closure)
