"""``sb_attn_varlen``: stick-breaking attention over a packed variable-length batch.

Drop-in for ``stickbreaking_attention.sb_varlen.sb_attn_varlen`` (``sb_varlen/__init__.py:24-82``):
same argument order and meaning, same ``(o, rem)`` outputs, gradients for q, k, v from upstream
gradients of both outputs.
"""
from __future__ import annotations

import math

import torch

from . import ops


class StickBreakingAttention(torch.autograd.Function):
    """Autograd glue of the packed operator (reference: ``sb_varlen/__init__.py:24-68``)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlens, inv_temp, attend_current, leading_zero):
        o, rem, log_rem = ops.varlen_fwd(q, k, v, cu_seqlens, max_seqlens, inv_temp,
                                         attend_current=attend_current, leading_zero=leading_zero)
        ctx.save_for_backward(q, k, v, log_rem, cu_seqlens)
        ctx.logit_scale = inv_temp
        ctx.max_seqlens = max_seqlens
        ctx.attend_current = attend_current
        ctx.leading_zero = leading_zero
        ctx.switches = ops.switch_flags()   # the backward runs on autograd's thread: it gets the caller's switches
        return o, rem

    @staticmethod
    def backward(ctx, do, drem):
        q, k, v, log_rem, cu_seqlens = ctx.saved_tensors
        dq, dk, dv = ops.varlen_bwd(do, drem, q, k, v, cu_seqlens, ctx.max_seqlens, log_rem,
                                    ctx.logit_scale, attend_current=ctx.attend_current,
                                    leading_zero=ctx.leading_zero, switches=ctx.switches)
        return dq, dk, dv, None, None, None, None, None


def sb_attn_varlen(q, k, v, cu_seqlens, max_seqlens=None, inv_temp=None, zero_start=True,
                   attend_current=False):
    """q, k, v: ``(heads, total_tokens, head_dim)``; ``cu_seqlens``: cumulative sequence ends on the
    device, with a leading 0 iff ``zero_start``.  Returns ``o`` like q and ``rem (heads, total_tokens)``.

    ``max_seqlens`` is optional here (the reference requires it): it is only an upper bound that keeps
    the backward's scratch memory small; leaving it out costs memory, never a host synchronisation.
    The leading zero is verified on the device (see ``ops.check_status``) rather than with the
    reference's host-side ``assert cu_seqlens[0] == 0`` (``sb_varlen/__init__.py:72-74``).
    """
    if inv_temp is None:
        inv_temp = 1 / math.sqrt(q.size(-1))
    if torch.compiler.is_compiling():   # one traceable operator with its own autograd formula
        o, rem, _ = ops.functional_fwd(q, k, v, cu_seqlens, max_seqlens, inv_temp, attend_current, bool(zero_start))
        return o, rem
    return sb_attn_varlen_(q, k, v, inv_temp, cu_seqlens, max_seqlens, attend_current, bool(zero_start))


def sb_attn_varlen_(q, k, v, inv_temp, cu_seqlens, max_seqlens, attend_current, leading_zero=False):
    return StickBreakingAttention.apply(q, k, v, cu_seqlens, max_seqlens, inv_temp, attend_current,
                                        leading_zero)


class StickBreakingAttentionFused(torch.autograd.Function):
    """``out = o + rem[..., None] * v`` in one operator (forward epilogue and backward fold inside the kernels' C ABI)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlens, inv_temp, attend_current, leading_zero):
        out, _, log_rem = ops.fused_fwd(q, k, v, cu_seqlens, max_seqlens, inv_temp,
                                        attend_current=attend_current, leading_zero=leading_zero)
        ctx.save_for_backward(q, k, v, log_rem, cu_seqlens)
        ctx.args = (max_seqlens, inv_temp, attend_current, leading_zero, ops.switch_flags())
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, log_rem, cu_seqlens = ctx.saved_tensors
        max_seqlens, inv_temp, attend_current, leading_zero, switches = ctx.args
        dq, dk, dv = ops.fused_bwd(dout, q, k, v, cu_seqlens, max_seqlens, log_rem, inv_temp,
                                   attend_current=attend_current, leading_zero=leading_zero, switches=switches)
        return dq, dk, dv, None, None, None, None, None


def sb_attn_varlen_fused(q, k, v, cu_seqlens, max_seqlens=None, inv_temp=None, zero_start=True,
                         attend_current=False):
    """Same arguments as ``sb_attn_varlen``; returns the single tensor ``o + rem[..., None] * v`` that the reference's
    callers compute from its two outputs (``tests/test_varlen.py:101``), without the extra passes over o and v."""
    if inv_temp is None:
        inv_temp = 1 / math.sqrt(q.size(-1))
    if torch.compiler.is_compiling():
        return ops.functional_fwd(q, k, v, cu_seqlens, max_seqlens, inv_temp, attend_current, bool(zero_start),
                                  fuse_rem_v=True)[0]
    return StickBreakingAttentionFused.apply(q, k, v, cu_seqlens, max_seqlens, inv_temp, attend_current,
                                             bool(zero_start))
