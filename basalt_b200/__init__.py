"""basalt_b200 - the Basalt engine's mixture-of-experts layer hot path as hand-written CUDA for NVIDIA B200 (sm_100a),
behind a C ABI (include/basalt_b200.h) and a thin host-side mirror of the reference's operator interface (moe.py)."""
from . import capi  # noqa: F401

__all__ = ["capi", "moe", "build"]
