"""CPU oracle for stick-breaking attention.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only ``tests/``, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import it.  The shipped package
never does; without its CUDA library it raises.

Parity status: PINNED.  ``tests/golden/make_golden.py`` runs the unmodified reference
(``stickbreaking_attention/sb_ref.py`` of shawntan/stickbreaking-attention) on seeded inputs and
stores its outputs and autograd gradients; ``tests/test_oracle.py`` checks every function in this
file against those vectors.

What is restated here, in this module's own code:

* ``stickbreaking_dense``        <- ``stickbreaking_attention/sb_ref.py:8-25`` (the dense oracle)
* ``varlen_dense`` / ``fixed_dense`` <- the per-sequence splitting and mask / cum-weight
  construction of ``tests/test_varlen.py:10-27`` and ``tests/test_attn.py:10-18`` (without the
  ``.cuda()`` calls and without folding ``rem * v`` into ``o``)
* ``varlen_dense_grads``         <- ``tests/test_varlen.py:29-41`` (autograd backward), extended
  to take an upstream gradient for ``rem`` as well
* ``varlen_rowblocked`` / ``varlen_rowblocked_grads``: the same function evaluated one block of
  query rows at a time with closed-form gradients, for sequence lengths where the dense L x L
  matrices do not fit.  It is pinned to the dense restatement in the tests.

Math (one head, one sequence; ``s`` = logit scale; ``allowed`` = j < i, or j <= i with
``attend_current``)::

    z[i,j]    = s * <q_i, k_j>
    lob[i,j]  = log(1 - sigmoid(z)) = -softplus(z)          (0 where not allowed)
    logA[i,j] = logsigmoid(z[i,j]) + sum_{j' > j} lob[i,j']
    A         = exp(logA)                                    (0 where not allowed)
    o_i       = sum_j A[i,j] v_j ;   rem_i = 1 - sum_j A[i,j]
"""
from __future__ import annotations

import math
from typing import Sequence

import torch
import torch.nn.functional as F

__all__ = [
    "stickbreaking_dense",
    "seq_bounds",
    "varlen_dense",
    "varlen_dense_grads",
    "fixed_dense",
    "fixed_dense_grads",
    "varlen_rowblocked",
    "varlen_rowblocked_grads",
    "flops",
]


def stickbreaking_dense(q, k, v, mask, cum_weight, scale=None):
    """Dense stick-breaking attention; follows ``sb_ref.py:8-25`` step by step.

    ``mask`` is True where a (query, key) pair is NOT allowed; ``cum_weight[j', j]`` is 1 where
    key ``j'`` lies after key ``j`` (``tril(-1)`` of ones), so that the einsum yields the
    exclusive suffix sum of ``log(1 - beta)`` over later keys.  ``scale`` defaults to
    ``1/sqrt(head_dim)`` like the reference, which has no other setting.
    """
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    z = torch.matmul(q, k.transpose(-1, -2)) * scale
    io_dtype = z.dtype
    z = z.float()
    log_beta = F.logsigmoid(z).masked_fill(mask, -1e5).to(io_dtype)
    log_one_minus_beta = F.logsigmoid(-z).masked_fill(mask, 0).to(io_dtype)
    later = torch.einsum("bhij,jk->bhik", log_one_minus_beta, cum_weight.to(log_one_minus_beta))
    att = (log_beta + later).exp()
    return torch.matmul(att, v), 1 - att.sum(dim=-1)


def seq_bounds(cu_seqlens: Sequence[int] | torch.Tensor, zero_start: bool = False):
    """(start, end) token offsets of each packed sequence.

    ``cu_seqlens`` holds sequence END offsets (``sb_varlen/__init__.py:71-74``: a leading 0 is
    present, and stripped, only with ``zero_start``).
    """
    ends = [int(x) for x in (cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else cu_seqlens)]
    if zero_start:
        assert ends[0] == 0
        ends = ends[1:]
    starts = [0] + ends[:-1]
    return list(zip(starts, ends))


def _masks(length: int, attend_current: bool, like: torch.Tensor):
    cm = torch.ones(length, length).tril(-1).to(like)
    mask = torch.ones(length, length).triu(1 if attend_current else 0).bool()
    return mask, cm


def varlen_dense(q, k, v, cu_seqlens, scale=None, attend_current=False, zero_start=False):
    """Packed ``(H, T, d)`` batch -> ``(o (H,T,d), rem (H,T))`` by running the dense function on
    each sequence separately (``tests/test_varlen.py:10-27``)."""
    bounds = seq_bounds(cu_seqlens, zero_start)
    longest = max(e - s for s, e in bounds)
    mask, cm = _masks(longest, attend_current, q)
    o_parts, r_parts = [], []
    for s, e in bounds:
        n = e - s
        o, rem = stickbreaking_dense(q[None, :, s:e], k[None, :, s:e], v[None, :, s:e],
                                     mask[:n, :n], cm[:n, :n], scale)
        o_parts.append(o[0])
        r_parts.append(rem[0])
    return torch.cat(o_parts, 1), torch.cat(r_parts, 1)


def varlen_dense_grads(q, k, v, cu_seqlens, do, drem, scale=None, attend_current=False,
                       zero_start=False):
    """``(o, rem, dq, dk, dv)`` with the gradients taken by autograd through the dense function
    (``tests/test_varlen.py:29-41``), for upstream gradients ``do`` and ``drem``."""
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    o, rem = varlen_dense(q, k, v, cu_seqlens, scale, attend_current, zero_start)
    dq, dk, dv = torch.autograd.grad((o, rem), (q, k, v), (do.to(o), drem.to(rem)))
    return o.detach(), rem.detach(), dq, dk, dv


def fixed_dense(q, k, v, scale=None, attend_current=False):
    """``(B, H, T, d)`` -> ``(o, rem (B,H,T))`` (``tests/test_attn.py:10-18``)."""
    mask, cm = _masks(q.shape[-2], attend_current, q)
    return stickbreaking_dense(q, k, v, mask, cm, scale)


def fixed_dense_grads(q, k, v, do, drem, scale=None, attend_current=False):
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    o, rem = fixed_dense(q, k, v, scale, attend_current)
    dq, dk, dv = torch.autograd.grad((o, rem), (q, k, v), (do.to(o), drem.to(rem)))
    return o.detach(), rem.detach(), dq, dk, dv


def _row_block(qb, kk, vv, i0, scale, attend_current):
    """Rows ``i0 .. i0+m`` of one sequence against keys ``0 .. i0+m``; returns z, lob, A."""
    m, n = qb.shape[-2], kk.shape[-2]
    z = torch.matmul(qb, kk.transpose(-1, -2)) * scale
    rows = torch.arange(i0, i0 + m).unsqueeze(-1)
    cols = torch.arange(n).unsqueeze(0)
    allowed = (cols <= rows) if attend_current else (cols < rows)
    lob = torch.where(allowed, F.logsigmoid(-z), torch.zeros((), dtype=z.dtype))
    # inclusive suffix sum over keys:  logsigmoid(z) + sum_{j'>j} lob  ==  z + sum_{j'>=j} lob
    suffix = torch.flip(torch.cumsum(torch.flip(lob, (-1,)), -1), (-1,))
    att = torch.where(allowed, torch.exp(z + suffix), torch.zeros((), dtype=z.dtype))
    return z, allowed, att


def varlen_rowblocked(q, k, v, cu_seqlens, scale=None, attend_current=False, zero_start=False,
                      block=1024, dtype=torch.float32):
    """Same function as ``varlen_dense``, evaluated ``block`` query rows at a time in ``dtype``.
    Needs O(block * L) memory per head instead of O(L^2)."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    o = torch.zeros_like(q)
    rem = torch.zeros(q.shape[:-1], dtype=dtype)
    for s, e in seq_bounds(cu_seqlens, zero_start):
        for i0 in range(s, e, block):
            i1 = min(i0 + block, e)
            _, _, att = _row_block(q[:, i0:i1], k[:, s:i1], v[:, s:i1], i0 - s, scale, attend_current)
            o[:, i0:i1] = torch.matmul(att, v[:, s:i1])
            rem[:, i0:i1] = 1 - att.sum(-1)
    return o, rem


def varlen_rowblocked_grads(q, k, v, cu_seqlens, do, drem, scale=None, attend_current=False,
                            zero_start=False, block=1024, dtype=torch.float32):
    """``(o, rem, dq, dk, dv)`` with closed-form gradients::

        G  = A * (<dO_i, v_j> - dR_i);  C = inclusive prefix sum of G over keys
        dz = G - sigmoid(z) * C;  dQ = s dz K;  dK = s dz^T Q;  dV = A^T dO
    """
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    q, k, v, do, drem = (t.to(dtype) for t in (q, k, v, do, drem))
    o = torch.zeros_like(q)
    rem = torch.zeros(q.shape[:-1], dtype=dtype)
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    for s, e in seq_bounds(cu_seqlens, zero_start):
        for i0 in range(s, e, block):
            i1 = min(i0 + block, e)
            kk, vv = k[:, s:i1], v[:, s:i1]
            z, allowed, att = _row_block(q[:, i0:i1], kk, vv, i0 - s, scale, attend_current)
            o[:, i0:i1] = torch.matmul(att, vv)
            rem[:, i0:i1] = 1 - att.sum(-1)
            g = att * (torch.matmul(do[:, i0:i1], vv.transpose(-1, -2)) - drem[:, i0:i1, None])
            c = torch.cumsum(g, -1)
            dz = torch.where(allowed, g - torch.sigmoid(z) * c, torch.zeros((), dtype=dtype))
            dq[:, i0:i1] = scale * torch.matmul(dz, kk)
            dk[:, s:i1] += scale * torch.matmul(dz.transpose(-1, -2), q[:, i0:i1])
            dv[:, s:i1] += torch.matmul(att.transpose(-1, -2), do[:, i0:i1])
    return o, rem, dq, dk, dv


def flops(lengths: Sequence[int], heads: int, head_dim: int, mode: str = "fwd_bwd") -> float:
    """Causal FLOP convention: forward 2*L^2*d per head per sequence, backward 2.5x that."""
    c = {"fwd": 2.0, "bwd": 5.0, "fwd_bwd": 7.0}[mode]
    return c * head_dim * heads * float(sum(int(n) * int(n) for n in lengths))
