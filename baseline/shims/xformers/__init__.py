"""Stand-in for xformers (not in this image).  The reference imports it unconditionally
(mist/modules/mha.py:33) but only calls it when the device name starts with "v100"
(mist/modules/mha.py:998-1004); here the names it touches at import time exist and the attention call
itself falls back to torch's scaled-dot-product attention.  Only used by the reference arm of bench.py."""
from . import ops  # noqa: F401
