import torch


def _cast_if_autocast_enabled(*args):
    if not torch.is_autocast_enabled():
        return args
    return torch.cuda.amp.autocast_mode._cast(args, torch.get_autocast_gpu_dtype())
