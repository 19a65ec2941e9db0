"""B200 (sm_100a) fused W8A8 MoE: host-side mirror of the reference's Python surface.

Reference counterparts: alpha_moe_ops.py:28-88 (wrapper), alpha_moe_python/utils.py:5-29
(interleave_tensor, get_best_config), csrc/torch_interface.cpp:105-127 (operator registration).

There is no CPU or eager fallback anywhere: `alpha_moe_b200.capi` (the ctypes binding every
entry point goes through) raises at import if libalpha_moe_b200.so is missing, and load_torch_op
raises if the operator library is.  The package itself stays importable without them so that
`python -m alpha_moe_b200.build` can create them.
"""
from __future__ import annotations

from .utils import interleave_tensor, get_best_config   # noqa: F401

_torch_op_loaded = False


def load_torch_op() -> None:
    """Registers torch.ops.alpha_moe.fused_moe_w8a8_up_down (CUDA dispatch key)."""
    global _torch_op_loaded
    if _torch_op_loaded:
        return
    import os
    import torch
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libalpha_moe_torch.so")
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m alpha_moe_b200.build` "
            "(there is no fallback implementation)")
    torch.ops.load_library(path)
    _torch_op_loaded = True
    from . import ops  # noqa: F401  (registers the fake implementation)
