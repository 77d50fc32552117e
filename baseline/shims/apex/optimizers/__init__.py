import torch
import amp_C


class FusedAdam(torch.optim.Optimizer):
    """Constructor-compatible with apex.optimizers.FusedAdam; ``step`` runs torch's fused Adam(W)."""

    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8,
                 adam_w_mode=True, weight_decay=0.0, amsgrad=False, capturable=False,
                 master_weights=False, set_grad_none=True):
        if amsgrad:
            raise RuntimeError("FusedAdam does not support the AMSGrad variant.")
        defaults = dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps,
                        weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.adam_w_mode = 1 if adam_w_mode else 0
        self.capturable = capturable
        self.master_weights = master_weights
        self.set_grad_none = set_grad_none

    @torch.no_grad()
    def step(self, closure=None, **_):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            group["step"] = group.get("step", 0) + 1
            ps = [p for p in group["params"] if p.grad is not None]
            for p in ps:
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
            b1, b2 = group["betas"]
            amp_C.multi_tensor_adam(0, None, [[p.grad for p in ps], ps,
                                               [self.state[p]["exp_avg"] for p in ps],
                                               [self.state[p]["exp_avg_sq"] for p in ps]],
                                    group["lr"], b1, b2, group["eps"], group["step"], self.adam_w_mode,
                                    group["bias_correction"], group["weight_decay"])
        return loss
