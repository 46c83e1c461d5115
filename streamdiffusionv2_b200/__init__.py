"""B200-native kernels for StreamDiffusionV2's per-chunk causal self-attention path.

Public surface:
    ops                 thin wrappers over the C ABI (rope + K/V append, cache attention, cross-attention)
    RingState           host-integer mirror of the sink + ring slot logic
    install(model)      swap the attention forwards of a CausalWanModel-shaped module for the kernels
    CausalWanModel      host-side mirror of the reference model interface (for running without it)
"""
from . import _native  # noqa: F401
from . import ops  # noqa: F401
from .ring_state import RingState  # noqa: F401
from .causal_attention import install  # noqa: F401
from .wan_model import CausalWanModel  # noqa: F401

__all__ = ["ops", "RingState", "install", "CausalWanModel"]
