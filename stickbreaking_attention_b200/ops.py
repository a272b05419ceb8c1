"""Host launchers and ``torch.library`` operators over the C ABI.

Mirrors the reference's launcher layer: ``varlen_fwd`` / ``varlen_bwd``
(``sb_varlen/sb_varlen_fwd.py:413-522``, ``sb_varlen/sb_varlen_bwd.py:484-641``) and the fixed-length
``attn_fwd`` / ``attn_bwd`` (``sb_attn/sb_fwd.py:139-253``, ``sb_attn/sb_bwd.py:163-297``).  Like the
reference (``utils.py:12-39``) each launcher is also registered as a mutating custom operator and is
routed through it only while ``torch.compile`` is tracing.  The operator namespace is
``stickbreaking_attention_b200`` so that both packages can be imported in one process.

Differences from the reference launchers, all on purpose:

* the saved state is ``log_rem`` (fp64, base-2) instead of the fp32 ``neg_log_acc``;
* ``max_seqlens`` is only an upper bound used to size scratch memory and may be ``None``;
* nothing is zero-initialised with separate memsets: the kernels write every output row;
* ``cu_seqlens`` is validated on the device into a status word (``check_status``), so no launcher
  synchronises with the host.
"""
from __future__ import annotations

import contextlib
import threading
from typing import Optional

import torch

from . import _cabi

NAMESPACE = "stickbreaking_attention_b200"

class _Switches(threading.local):
    """Per-thread switches (a trainer may drive several devices from several threads)."""
    force_simt = False
    bwd_recompute = False
    dense_row_pass = False


_state = _Switches()
_launches = [0]   # process-wide: the backward's launches happen on autograd's thread
_status_words: dict[int, torch.Tensor] = {}


@contextlib.contextmanager
def force_simt(enabled: bool = True):
    """Within the block (calling thread only), bf16/fp16 calls run the CUDA-core kernels too (a cross-check in tests)."""
    old = _state.force_simt
    _state.force_simt = enabled
    try:
        yield
    finally:
        _state.force_simt = old


@contextlib.contextmanager
def small_backward_workspace(enabled: bool = True):
    """Within the block (calling thread only) the backward keeps its workspace small: the dK/dV kernel recomputes the
    attention tiles from boundary values (a few KiB per tile pair) instead of reading the 64 KiB per pair the dQ kernel
    would store for it (``SB_FLAG_BWD_RECOMPUTE``).  Slower, same results to rounding."""
    old = _state.bwd_recompute
    _state.bwd_recompute = enabled
    try:
        yield
    finally:
        _state.bwd_recompute = old


@contextlib.contextmanager
def dense_row_pass(enabled: bool = True):
    """Within the block (calling thread only) the tensor-core kernels do the per-score arithmetic for every score, also
    where the product of (1 - beta) over the keys in between has underflowed to exactly 0 for a whole warp and the
    results are known to be exact zeros (``SB_FLAG_DENSE_ROW_PASS``).  Same results bit for bit; a measuring aid."""
    old = _state.dense_row_pass
    _state.dense_row_pass = enabled
    try:
        yield
    finally:
        _state.dense_row_pass = old


def switch_flags() -> int:
    """The calling thread's switches as C-ABI flag bits.  The autograd functions read them in their forward and hand
    them to their backward: autograd runs the backward on a thread of its own, which does not see the caller's."""
    return (_cabi.SB_FLAG_FORCE_SIMT if _state.force_simt else 0) | \
           (_cabi.SB_FLAG_BWD_RECOMPUTE if _state.bwd_recompute else 0) | \
           (_cabi.SB_FLAG_DENSE_ROW_PASS if _state.dense_row_pass else 0)


def kernel_launches() -> int:
    """Total kernel launches enqueued through this module since import (for benchmark accounting)."""
    return _launches[0]


def set_backward_scratch_budget(nbytes: int) -> int:
    """Process-wide upper bound on the scratch one chunk of heads of the backward may take (default 8 GiB); returns
    the previous bound.  The backward stores 64 KiB per (query tile, key tile) pair and head for its dK/dV kernel and
    works through the heads in chunks that fit the bound; a call whose single head does not fit recomputes the tiles
    instead (slower, O(tokens) scratch).  Raising the bound on a GPU with memory to spare lets long sequences take the
    stored-tiles kernels; lowering it bounds the transient allocation of every backward call."""
    return int(_cabi.load().sb_set_backward_scratch_budget(int(nbytes)))


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(idx)
    if word is None:
        word = torch.zeros(4, dtype=torch.int32, device=device)
        _status_words[idx] = word
    return word


def check_status(device=None) -> None:
    """Reads (synchronising) the device status word written by the kernels, clears it, and raises
    ``SbError`` if a kernel reported a problem since the last check."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status_word(device)
    vals = word.tolist()
    if vals[0] != 0:
        word.zero_()
        msg = _cabi.SB_DEV_MESSAGES.get(vals[0], "unknown device status {0}").format(vals[1])
        raise _cabi.SbError(f"device status {vals[0]}: {msg}")


def _require(cond: bool, msg: str):
    if not cond:
        raise ValueError(msg)


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """Unit innermost stride, 16-byte aligned base and outer strides; copies only if needed."""
    mult = 16 // t.element_size()
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(
        s % mult == 0 or n == 1 for s, n in zip(t.stride()[:-1], t.shape[:-1]))
    if t.shape[-1] % mult != 0:          # rows cannot be 16-byte multiples anyway
        ok = t.stride(-1) == 1
    return t if ok else t.contiguous()


def _fill(prm, *, fixed, q, k, v, cu_seqlens, max_seqlens, logit_scale, attend_current, leading_zero,
          fuse_rem_v=False, switches=None):
    _require(q.is_cuda, "stick-breaking attention runs on a CUDA device only (no CPU path)")
    _require(q.dtype in _cabi.SB_DTYPE, f"unsupported dtype {q.dtype}")
    _require(q.dtype == k.dtype == v.dtype, "q, k, v must share a dtype")
    _require(q.shape == k.shape == v.shape, "q, k, v must share a shape")
    _require(q.dim() == (4 if fixed else 3), "expected (B,H,T,d) for sb_attn and (H,T,d) for sb_attn_varlen")
    prm.struct_bytes = _cabi.ctypes.sizeof(_cabi.SbParams)
    prm.dtype = _cabi.SB_DTYPE[q.dtype]
    if fixed:
        prm.batch, prm.heads, prm.tokens, prm.head_dim = q.shape
        prm.num_seq = 0
        prm.cu_seqlens = None
    else:
        prm.batch = 1
        prm.heads, prm.tokens, prm.head_dim = q.shape
        _require(cu_seqlens.is_cuda and cu_seqlens.dim() == 1, "cu_seqlens must be a 1-D CUDA tensor")
        _require(cu_seqlens.dtype in (torch.int32, torch.int64), "cu_seqlens must be int32 or int64")
        _require(cu_seqlens.stride(0) == 1, "cu_seqlens must be contiguous")
        prm.num_seq = cu_seqlens.numel()
        prm.cu_seqlens = cu_seqlens.data_ptr()
        prm.cu_seqlens_int64 = int(cu_seqlens.dtype == torch.int64)
    prm.max_seqlen = 0 if max_seqlens is None else int(max_seqlens)
    prm.attend_current = int(bool(attend_current))
    prm.logit_scale = float(logit_scale)
    prm.flags = (switch_flags() if switches is None else switches) | \
                (_cabi.SB_FLAG_CHECK_LEADING_ZERO if leading_zero else 0) | \
                (_cabi.SB_FLAG_FUSE_REM_V if fuse_rem_v else 0)
    prm.q = _cabi.tensor_arg(q, fixed)
    prm.k = _cabi.tensor_arg(k, fixed)
    prm.v = _cabi.tensor_arg(v, fixed)


def _run(backward: bool, prm, device):
    lib = _cabi.load()
    need = lib.sb_workspace_bytes(prm, int(backward))
    if need == 2 ** 64 - 1:
        raise _cabi.SbError(f"invalid parameters: {lib.sb_last_error().decode()}")
    try:
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=device)
    except torch.cuda.OutOfMemoryError:
        # the stored-tiles backward asks for up to the scratch budget; where the reference would still fit (its backward
        # keeps O(tokens) state), fall back to the recomputing kernels and their few MB instead of failing
        if not backward or prm.flags & _cabi.SB_FLAG_BWD_RECOMPUTE:
            raise
        prm.flags |= _cabi.SB_FLAG_BWD_RECOMPUTE
        need = lib.sb_workspace_bytes(prm, 1)
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=device)
    prm.workspace = workspace.data_ptr()
    prm.workspace_bytes = workspace.numel()
    prm.status = _status_word(device).data_ptr()
    stream = torch.cuda.current_stream(device).cuda_stream
    fn = lib.sb_bwd if backward else lib.sb_fwd
    if device.index is None or device.index == torch.cuda.current_device():
        rc = fn(prm, stream)
    else:
        with torch.cuda.device(device):
            rc = fn(prm, stream)
    _cabi.check_call(lib, rc, "sb_bwd" if backward else "sb_fwd")
    _launches[0] += lib.sb_last_launch_count()
    # the caching allocator keeps `workspace` alive until the stream has passed this point
    return workspace


def _fwd_impl(fixed, q, k, v, cu_seqlens, max_seqlens, logit_scale, attend_current, leading_zero,
              o, rem, log_rem, fuse_rem_v=False, attn=None):
    prm = _cabi.SbParams()
    _fill(prm, fixed=fixed, q=q, k=k, v=v, cu_seqlens=cu_seqlens, max_seqlens=max_seqlens,
          logit_scale=logit_scale, attend_current=attend_current, leading_zero=leading_zero, fuse_rem_v=fuse_rem_v)
    prm.o = _cabi.tensor_arg(o, fixed)
    prm.rem = rem.data_ptr()
    prm.log_rem = log_rem.data_ptr()
    if attn is not None:
        _require(attn.dtype == torch.float32 and attn.is_contiguous() and attn.shape[:-1] == q.shape[:-1],
                 "the attention-weights buffer must be contiguous fp32 of shape (*q.shape[:-1], columns)")
        prm.attn_weights = attn.data_ptr()
        prm.attn_cols = attn.shape[-1]
    _run(False, prm, q.device)


def _bwd_impl(fixed, do, dr, q, k, v, cu_seqlens, max_seqlens, log_rem, logit_scale, attend_current,
              leading_zero, dq, dk, dv, fuse_rem_v=False, switches=None):
    prm = _cabi.SbParams()
    _fill(prm, fixed=fixed, q=q, k=k, v=v, cu_seqlens=cu_seqlens, max_seqlens=max_seqlens,
          logit_scale=logit_scale, attend_current=attend_current, leading_zero=leading_zero, fuse_rem_v=fuse_rem_v,
          switches=switches)
    prm.log_rem = log_rem.data_ptr()
    prm.d_o = _cabi.tensor_arg(do, fixed)
    prm.d_rem = dr.data_ptr() if dr is not None else None
    prm.dq = _cabi.tensor_arg(dq, fixed)
    prm.dk = _cabi.tensor_arg(dk, fixed)
    prm.dv = _cabi.tensor_arg(dv, fixed)
    _run(True, prm, q.device)


# ---- custom operators (same four names as the reference registers) ---------------------------------

@torch.library.custom_op(f"{NAMESPACE}::varlen_fwd", mutates_args={"o", "rem", "log_rem"}, device_types="cuda")
def _op_varlen_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                   max_seqlens: int, logit_scale: float, attend_current: bool, leading_zero: bool,
                   o: torch.Tensor, rem: torch.Tensor, log_rem: torch.Tensor) -> None:
    _fwd_impl(False, q, k, v, cu_seqlens, max_seqlens, logit_scale, attend_current, leading_zero, o, rem, log_rem)


@torch.library.custom_op(f"{NAMESPACE}::varlen_bwd", mutates_args={"dq", "dk", "dv"}, device_types="cuda")
def _op_varlen_bwd(do: torch.Tensor, dr: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                   cu_seqlens: torch.Tensor, max_seqlens: int, log_rem: torch.Tensor, logit_scale: float,
                   attend_current: bool, leading_zero: bool, dq: torch.Tensor, dk: torch.Tensor,
                   dv: torch.Tensor) -> None:
    _bwd_impl(False, do, dr, q, k, v, cu_seqlens, max_seqlens, log_rem, logit_scale, attend_current,
              leading_zero, dq, dk, dv)


@torch.library.custom_op(f"{NAMESPACE}::attn_fwd", mutates_args={"o", "rem", "log_rem"}, device_types="cuda")
def _op_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, logit_scale: float, attend_current: bool,
                 o: torch.Tensor, rem: torch.Tensor, log_rem: torch.Tensor) -> None:
    _fwd_impl(True, q, k, v, None, None, logit_scale, attend_current, False, o, rem, log_rem)


@torch.library.custom_op(f"{NAMESPACE}::attn_bwd", mutates_args={"dq", "dk", "dv"}, device_types="cuda")
def _op_attn_bwd(do: torch.Tensor, dr: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                 log_rem: torch.Tensor, logit_scale: float, attend_current: bool, dq: torch.Tensor,
                 dk: torch.Tensor, dv: torch.Tensor) -> None:
    _bwd_impl(True, do, dr, q, k, v, None, None, log_rem, logit_scale, attend_current, False, dq, dk, dv)


# ---- functional operators: what ``torch.compile`` traces ----------------------------------------
# The mutating operators above mirror the reference's registration.  Tracing with ``fullgraph=True`` additionally
# needs operators that allocate their own outputs, have a shape-only ("fake") implementation and carry their own
# autograd formula, so that the tracer never has to look inside the launchers (pointer alignment checks, ctypes).

@torch.library.custom_op(f"{NAMESPACE}::fwd", mutates_args=(), device_types="cuda")
def _op_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: Optional[torch.Tensor],
            max_seqlens: int, logit_scale: float, attend_current: bool, leading_zero: bool,
            fuse_rem_v: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    fixed = cu_seqlens is None
    o = torch.empty_like(q)
    rem = torch.empty(q.shape[:-1], dtype=q.dtype, device=q.device)
    log_rem = torch.empty(q.shape[:-1], dtype=torch.float64, device=q.device)
    ends = None if fixed else _strip(cu_seqlens, leading_zero)
    _fwd_impl(fixed, _tma_ready(q), _tma_ready(k), _tma_ready(v), ends, max_seqlens if max_seqlens > 0 else None,
              logit_scale, attend_current, leading_zero and not fixed, o, rem, log_rem, fuse_rem_v=fuse_rem_v)
    return o, rem, log_rem


@_op_fwd.register_fake
def _(q, k, v, cu_seqlens, max_seqlens, logit_scale, attend_current, leading_zero, fuse_rem_v):
    return (torch.empty_like(q), q.new_empty(q.shape[:-1]), q.new_empty(q.shape[:-1], dtype=torch.float64))


@torch.library.custom_op(f"{NAMESPACE}::bwd", mutates_args=(), device_types="cuda")
def _op_bwd(do: torch.Tensor, dr: Optional[torch.Tensor], q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
            cu_seqlens: Optional[torch.Tensor], max_seqlens: int, log_rem: torch.Tensor, logit_scale: float,
            attend_current: bool, leading_zero: bool, fuse_rem_v: bool,
            switches: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    fixed = cu_seqlens is None
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ends = None if fixed else _strip(cu_seqlens, leading_zero)
    if dr is None and not fuse_rem_v:
        dr = torch.zeros(q.shape[:-1], dtype=q.dtype, device=q.device)
    _bwd_impl(fixed, _tma_ready(do.to(q.dtype)), None if dr is None else dr.to(q.dtype).contiguous(), _tma_ready(q),
              _tma_ready(k), _tma_ready(v), ends, max_seqlens if max_seqlens > 0 else None, log_rem, logit_scale,
              attend_current, leading_zero and not fixed, dq, dk, dv, fuse_rem_v=fuse_rem_v, switches=switches)
    return dq, dk, dv


@_op_bwd.register_fake
def _(do, dr, q, k, v, cu_seqlens, max_seqlens, log_rem, logit_scale, attend_current, leading_zero, fuse_rem_v,
      switches):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _fwd_setup_context(ctx, inputs, output):
    q, k, v, cu_seqlens, max_seqlens, logit_scale, attend_current, leading_zero, fuse_rem_v = inputs
    ctx.save_for_backward(q, k, v, output[2], cu_seqlens)
    ctx.args = (max_seqlens, logit_scale, attend_current, leading_zero, fuse_rem_v)
    ctx.switches = switch_flags()


def _fwd_backward(ctx, do, drem, dlog_rem):
    q, k, v, log_rem, cu_seqlens = ctx.saved_tensors
    max_seqlens, logit_scale, attend_current, leading_zero, fuse_rem_v = ctx.args
    if do is None:
        do = torch.zeros_like(q)
    dq, dk, dv = _op_bwd(do, drem, q, k, v, cu_seqlens, max_seqlens, log_rem, logit_scale, attend_current,
                         leading_zero, fuse_rem_v, ctx.switches)
    return dq, dk, dv, None, None, None, None, None, None


torch.library.register_autograd(f"{NAMESPACE}::fwd", _fwd_backward, setup_context=_fwd_setup_context)


def functional_fwd(q, k, v, cu_seqlens, max_seqlens, logit_scale, attend_current=False, leading_zero=False,
                   fuse_rem_v=False):
    """``(o, rem, log_rem)`` through the functional operator ``stickbreaking_attention_b200::fwd`` (differentiable in
    q, k, v through ``::bwd``); the public functions take this route while ``torch.compile`` is tracing."""
    return _op_fwd(q, k, v, cu_seqlens, 0 if max_seqlens is None else int(max_seqlens), float(logit_scale),
                   bool(attend_current), bool(leading_zero), bool(fuse_rem_v))


def _compiling() -> bool:
    return torch.compiler.is_compiling()


# ---- launchers -----------------------------------------------------------------------------------

def _strip(cu_seqlens, leading_zero):
    return cu_seqlens[1:] if leading_zero else cu_seqlens


def varlen_fwd(q, k, v, cu_seqlens, max_seqlens: Optional[int], logit_scale: float,
               attend_current: bool = False, leading_zero: bool = False, return_attention: bool = False):
    """Packed forward.  ``cu_seqlens`` holds sequence ends, preceded by a 0 iff ``leading_zero``.
    Returns ``(o, rem, log_rem)`` like the reference returns ``(o, rem, neg_log_acc)``.

    ``return_attention=True`` (``sb_varlen_fwd.py:413-449``, where the reference marks the output TODO) also returns
    ``W``, fp32 ``(heads, tokens, max_seqlens)``: row t holds the weights of token t over the keys of its own sequence,
    indexed from the sequence start, zeros elsewhere.  A debugging aid: O(tokens * max_seqlens) memory, and the call
    runs the CUDA-core kernels whatever the dtype."""
    q, k, v = _tma_ready(q), _tma_ready(k), _tma_ready(v)
    o = torch.empty_like(q)
    rem = torch.empty(q.shape[:-1], dtype=q.dtype, device=q.device)
    log_rem = torch.empty(q.shape[:-1], dtype=torch.float64, device=q.device)
    ends = _strip(cu_seqlens, leading_zero)
    if return_attention:
        cols = q.shape[-2] if max_seqlens is None else min(int(max_seqlens), q.shape[-2])
        attn = torch.zeros((*q.shape[:-1], cols), dtype=torch.float32, device=q.device)
        _fwd_impl(False, q, k, v, ends, max_seqlens, logit_scale, attend_current, leading_zero, o, rem, log_rem,
                  attn=attn)
        return o, rem, log_rem, attn
    if _compiling():
        _op_varlen_fwd(q, k, v, ends, 0 if max_seqlens is None else int(max_seqlens), float(logit_scale),
                       bool(attend_current), bool(leading_zero), o, rem, log_rem)
    else:
        _fwd_impl(False, q, k, v, ends, max_seqlens, logit_scale, attend_current, leading_zero, o, rem, log_rem)
    return o, rem, log_rem


def varlen_bwd(do, dr, q, k, v, cu_seqlens, max_seqlens: Optional[int], log_rem, logit_scale: float,
               attend_current: bool = False, leading_zero: bool = False, switches: Optional[int] = None):
    """Packed backward; returns ``(dq, dk, dv)`` in the dtype of the inputs.  ``switches``: the ``switch_flags()`` of
    the forward call (default: the calling thread's)."""
    q, k, v, do = _tma_ready(q), _tma_ready(k), _tma_ready(v), _tma_ready(do.to(q.dtype))
    dr = dr.to(q.dtype).contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ends = _strip(cu_seqlens, leading_zero)
    if _compiling():
        _op_varlen_bwd(do, dr, q, k, v, ends, 0 if max_seqlens is None else int(max_seqlens), log_rem,
                       float(logit_scale), bool(attend_current), bool(leading_zero), dq, dk, dv)
    else:
        _bwd_impl(False, do, dr, q, k, v, ends, max_seqlens, log_rem, logit_scale, attend_current,
                  leading_zero, dq, dk, dv, switches=switches)
    return dq, dk, dv


def attn_fwd(q, k, v, logit_scale: float, attend_current: bool = False, return_attention: bool = False):
    """Fixed-length ``(B,H,T,d)`` forward; returns ``(o, rem, log_rem)``, and with ``return_attention=True`` also the
    fp32 weights ``W (B,H,T,T)`` (see ``varlen_fwd``)."""
    q, k, v = _tma_ready(q), _tma_ready(k), _tma_ready(v)
    o = torch.empty_like(q)
    rem = torch.empty(q.shape[:-1], dtype=q.dtype, device=q.device)
    log_rem = torch.empty(q.shape[:-1], dtype=torch.float64, device=q.device)
    if return_attention:
        attn = torch.zeros((*q.shape[:-1], q.shape[-2]), dtype=torch.float32, device=q.device)
        _fwd_impl(True, q, k, v, None, None, logit_scale, attend_current, False, o, rem, log_rem, attn=attn)
        return o, rem, log_rem, attn
    if _compiling():
        _op_attn_fwd(q, k, v, float(logit_scale), bool(attend_current), o, rem, log_rem)
    else:
        _fwd_impl(True, q, k, v, None, None, logit_scale, attend_current, False, o, rem, log_rem)
    return o, rem, log_rem


def attn_bwd(do, dr, q, k, v, log_rem, logit_scale: float, attend_current: bool = False,
             switches: Optional[int] = None):
    """Fixed-length backward; returns ``(dq, dk, dv)`` in the dtype of the inputs (the reference
    forces dk and dv to bf16 here, ``sb_attn/sb_bwd.py:173-174``; this keeps the input dtype)."""
    q, k, v, do = _tma_ready(q), _tma_ready(k), _tma_ready(v), _tma_ready(do.to(q.dtype))
    dr = dr.to(q.dtype).contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if _compiling():
        _op_attn_bwd(do, dr, q, k, v, log_rem, float(logit_scale), bool(attend_current), dq, dk, dv)
    else:
        _bwd_impl(True, do, dr, q, k, v, None, None, log_rem, logit_scale, attend_current, False, dq, dk, dv,
                  switches=switches)
    return dq, dk, dv


def fused_fwd(q, k, v, cu_seqlens, max_seqlens, logit_scale, attend_current=False, leading_zero=False):
    """Forward with the callers' usual next step folded in: returns ``(out, rem, log_rem)`` with
    ``out = o + rem[..., None] * v`` (``tests/test_varlen.py:101``, ``tests/test_attn.py:64`` of the reference).
    Fixed-length when ``cu_seqlens`` is None.  Always a direct call of the C ABI (``SB_FLAG_FUSE_REM_V``)."""
    fixed = cu_seqlens is None
    q, k, v = _tma_ready(q), _tma_ready(k), _tma_ready(v)
    out = torch.empty_like(q)
    rem = torch.empty(q.shape[:-1], dtype=q.dtype, device=q.device)
    log_rem = torch.empty(q.shape[:-1], dtype=torch.float64, device=q.device)
    ends = None if fixed else _strip(cu_seqlens, leading_zero)
    _fwd_impl(fixed, q, k, v, ends, max_seqlens, logit_scale, attend_current, leading_zero and not fixed, out, rem,
              log_rem, fuse_rem_v=True)
    return out, rem, log_rem


def fused_bwd(dout, q, k, v, cu_seqlens, max_seqlens, log_rem, logit_scale, attend_current=False,
              leading_zero=False, switches=None):
    """Backward of ``fused_fwd``'s ``out``: ``<d_out, v>`` goes into the gradient of rem and ``rem * d_out`` into dv
    inside the library; returns ``(dq, dk, dv)``."""
    fixed = cu_seqlens is None
    q, k, v, dout = _tma_ready(q), _tma_ready(k), _tma_ready(v), _tma_ready(dout.to(q.dtype))
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ends = None if fixed else _strip(cu_seqlens, leading_zero)
    _bwd_impl(fixed, dout, None, q, k, v, ends, max_seqlens, log_rem, logit_scale, attend_current,
              leading_zero and not fixed, dq, dk, dv, fuse_rem_v=True, switches=switches)
    return dq, dk, dv


def kernel_path(q, fixed: bool = False) -> int:
    """Which kernels a call with tensors like ``q`` takes: 0 = CUDA cores, 1 = tcgen05."""
    prm = _cabi.SbParams()
    dummy_cu = None if fixed else torch.zeros(1, dtype=torch.int32, device=q.device)
    _fill(prm, fixed=fixed, q=q, k=q, v=q, cu_seqlens=dummy_cu, max_seqlens=None, logit_scale=1.0,
          attend_current=False, leading_zero=False)
    return _cabi.load().sb_kernel_path(prm)
