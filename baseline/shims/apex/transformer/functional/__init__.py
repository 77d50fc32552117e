from . import fused_softmax  # noqa: F401
