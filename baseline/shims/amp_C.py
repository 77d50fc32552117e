"""apex's ``amp_C`` entry points the reference calls, on torch's fused multi-tensor kernels."""
import torch


def _steps(step, like):
    if isinstance(step, torch.Tensor):
        s = step.to(device=like.device, dtype=torch.float32).reshape(())
    else:
        s = torch.tensor(float(step), dtype=torch.float32, device=like.device)
    # torch's fused kernel increments nothing itself: it reads the step it is given
    return s


def _adam(tensor_lists, lr, beta1, beta2, eps, step, mode, bias_correction, weight_decay, inv_scale=None):
    grads, params, exp_avgs, exp_avg_sqs = tensor_lists[:4]
    if not params:
        return
    if not bias_correction:
        raise NotImplementedError("bias_correction=False is not covered by this stand-in")
    s = _steps(step, params[0])
    steps = [s for _ in params]
    fn = torch._fused_adamw_ if mode else torch._fused_adam_
    grad_scale = None
    if inv_scale is not None:
        grad_scale = (1.0 / inv_scale).to(torch.float32).reshape(())
    fn(list(params), list(grads), list(exp_avgs), list(exp_avg_sqs), [], steps,
       lr=float(lr), beta1=beta1, beta2=beta2, weight_decay=weight_decay, eps=eps,
       amsgrad=False, maximize=False, grad_scale=grad_scale, found_inf=None)


def multi_tensor_adam(chunk_size, noop_flag, tensor_lists, lr, beta1, beta2, eps, step, mode,
                      bias_correction, weight_decay):
    _adam(tensor_lists, lr, beta1, beta2, eps, step, mode, bias_correction, weight_decay)


def multi_tensor_adam_capturable(chunk_size, noop_flag, tensor_lists, lr, beta1, beta2, eps, step, mode,
                                 bias_correction, weight_decay, inv_scale):
    _adam(tensor_lists, lr, beta1, beta2, eps, step, mode, bias_correction, weight_decay, inv_scale)


def multi_tensor_adam_capturable_master(chunk_size, noop_flag, tensor_lists, lr, beta1, beta2, eps, step,
                                        mode, bias_correction, weight_decay, inv_scale):
    _adam(tensor_lists[:4], lr, beta1, beta2, eps, step, mode, bias_correction, weight_decay, inv_scale)
    for p, master in zip(tensor_lists[1], tensor_lists[4]):
        master.copy_(p)


def multi_tensor_scale(chunk_size, noop_flag, tensor_lists, scale):
    src, dst = tensor_lists
    for a, b in zip(src, dst):
        b.copy_(a if scale == 1.0 else a * scale)
