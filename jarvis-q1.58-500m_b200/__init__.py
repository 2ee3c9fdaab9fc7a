"""jarvis_b200 -- B200 (sm_100a) kernels for the Jarvis block forward, behind the reference's
module API.  Host code is Python calling hand-written CUDA through the C ABI declared in
include/jarvis_b200.h; there is no CPU fallback."""
from . import _lib  # noqa: F401
from . import ops  # noqa: F401
from . import modules  # noqa: F401
from .modules import (AssociativeLinearAttention, Jarvis, JarvisBlock, LiquidStateFusion,  # noqa: F401
                      LiquidStateFusionExt, SparseMoELayer, TernaryLinear, install)

__all__ = ["_lib", "ops", "modules", "AssociativeLinearAttention", "SparseMoELayer", "LiquidStateFusion",
           "LiquidStateFusionExt", "TernaryLinear", "JarvisBlock", "Jarvis", "install"]
