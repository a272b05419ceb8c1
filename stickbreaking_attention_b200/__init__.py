"""Stick-breaking attention for NVIDIA B200 (sm_100a): hand-written CUDA kernels behind the operator
interface of shawntan/stickbreaking-attention.

    from stickbreaking_attention_b200 import sb_attn, sb_attn_varlen

``install_as_dropin()`` additionally makes ``import stickbreaking_attention`` (and its ``sb_varlen`` /
``sb_attn`` submodules) resolve to this package, for code written against the reference.
"""
import sys as _sys

from . import _cabi

_cabi.load()   # fail at import time, loudly, if the CUDA library has not been built

from . import ops, sb_attn as _sb_attn_mod, sb_varlen as _sb_varlen_mod  # noqa: E402
from .ops import (check_status, dense_row_pass, force_simt, kernel_launches, kernel_path, set_backward_scratch_budget,  # noqa: E402
                  small_backward_workspace)
from .sb_attn import sb_attn, sb_attn_fused  # noqa: E402
from .sb_varlen import sb_attn_varlen, sb_attn_varlen_fused  # noqa: E402

__all__ = ["sb_attn", "sb_attn_varlen", "sb_attn_fused", "sb_attn_varlen_fused", "check_status", "force_simt",
           "small_backward_workspace", "dense_row_pass", "set_backward_scratch_budget", "kernel_launches", "kernel_path", "install_as_dropin",
           "ops"]


def install_as_dropin(name: str = "stickbreaking_attention") -> None:
    """Registers this package under the reference's import name (refuses to shadow an import that
    already happened)."""
    this = _sys.modules[__name__]
    for alias, mod in ((name, this), (name + ".sb_varlen", _sb_varlen_mod), (name + ".sb_attn", _sb_attn_mod)):
        if alias in _sys.modules and _sys.modules[alias] is not mod:
            raise ImportError(f"{alias} is already imported from {_sys.modules[alias].__file__}")
        _sys.modules[alias] = mod
