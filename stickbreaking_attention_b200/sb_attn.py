"""``sb_attn``: stick-breaking attention over a fixed-length ``(batch, heads, tokens, head_dim)`` batch.

Drop-in for ``stickbreaking_attention.sb_attn.sb_attn`` (``sb_attn/__init__.py:16-64``).
"""
from __future__ import annotations

import math

import torch

from . import ops


class StickBreakingAttention(torch.autograd.Function):
    """Autograd glue of the fixed-length operator (reference: ``sb_attn/__init__.py:16-54``)."""

    @staticmethod
    def forward(ctx, q, k, v, inv_temp, attend_current=False):
        o, rem, log_rem = ops.attn_fwd(q, k, v, inv_temp, attend_current=attend_current)
        ctx.save_for_backward(q, k, v, log_rem)
        ctx.logit_scale = inv_temp
        ctx.attend_current = attend_current
        ctx.switches = ops.switch_flags()   # the backward runs on autograd's thread: it gets the caller's switches
        return o, rem

    @staticmethod
    def backward(ctx, do, drem):
        q, k, v, log_rem = ctx.saved_tensors
        dq, dk, dv = ops.attn_bwd(do, drem, q, k, v, log_rem, ctx.logit_scale,
                                  attend_current=ctx.attend_current, switches=ctx.switches)
        return dq, dk, dv, None, None


def sb_attn(q, k, v, inv_temp=None, zero_start=True, attend_current=False):
    """``zero_start`` is accepted and ignored, as in the reference (``sb_attn/__init__.py:57``)."""
    if inv_temp is None:
        inv_temp = 1 / math.sqrt(q.size(-1))
    if torch.compiler.is_compiling():   # one traceable operator with its own autograd formula
        o, rem, _ = ops.functional_fwd(q, k, v, None, None, inv_temp, attend_current)
        return o, rem
    return sb_attn_(q, k, v, inv_temp, attend_current=attend_current)


def sb_attn_(q, k, v, inv_temp, attend_current):
    return StickBreakingAttention.apply(q, k, v, inv_temp, attend_current)


class StickBreakingAttentionFused(torch.autograd.Function):
    """``out = o + rem[..., None] * v`` in one operator, fixed-length batch."""

    @staticmethod
    def forward(ctx, q, k, v, inv_temp, attend_current=False):
        out, _, log_rem = ops.fused_fwd(q, k, v, None, None, inv_temp, attend_current=attend_current)
        ctx.save_for_backward(q, k, v, log_rem)
        ctx.args = (inv_temp, attend_current, ops.switch_flags())
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, log_rem = ctx.saved_tensors
        inv_temp, attend_current, switches = ctx.args
        dq, dk, dv = ops.fused_bwd(dout, q, k, v, None, None, log_rem, inv_temp, attend_current=attend_current,
                                   switches=switches)
        return dq, dk, dv, None, None


def sb_attn_fused(q, k, v, inv_temp=None, zero_start=True, attend_current=False):
    """Same arguments as ``sb_attn``; returns ``o + rem[..., None] * v`` (``tests/test_attn.py:64`` of the reference)."""
    if inv_temp is None:
        inv_temp = 1 / math.sqrt(q.size(-1))
    if torch.compiler.is_compiling():
        return ops.functional_fwd(q, k, v, None, None, inv_temp, attend_current, fuse_rem_v=True)[0]
    return StickBreakingAttentionFused.apply(q, k, v, inv_temp, attend_current)
