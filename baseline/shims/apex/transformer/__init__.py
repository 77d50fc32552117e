from .enums import AttnMaskType, AttnType, LayerType, ModelType  # noqa: F401
from . import functional  # noqa: F401
