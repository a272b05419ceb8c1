"""ctypes binding of ``libsb_b200.so`` (declared in ``include/sb_b200.h``).

There is no other implementation behind this module: if the library is missing or does not load,
importing the operators raises.  Nothing here falls back to PyTorch or to the CPU.
"""
from __future__ import annotations

import ctypes
import os

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libsb_b200.so")

SB_DTYPE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
SB_PATH_SIMT, SB_PATH_TCGEN05 = 0, 1
SB_STATIC_SCRATCH_BYTES = 65536
SB_FLAG_FORCE_SIMT, SB_FLAG_CHECK_LEADING_ZERO, SB_FLAG_BWD_SKIP_DKV, SB_FLAG_BWD_SKIP_DQ = 1, 2, 4, 8
SB_FLAG_BWD_RECOMPUTE = 16
SB_FLAG_FUSE_REM_V = 32
SB_FLAG_DENSE_ROW_PASS = 64
SB_DEV_MESSAGES = {
    1: "cu_seqlens is invalid (not non-decreasing, beyond the token count, longer than max_seqlens, "
       "or without its leading zero); offending sequence index: {0}",
    2: "a bounded on-chip wait timed out in barrier {0}",
}
EXPORTS = ("sb_workspace_bytes", "sb_fwd", "sb_bwd", "sb_fwd_static_scratch", "sb_set_backward_scratch_budget",
           "sb_kernel_path", "sb_last_launch_count", "sb_last_error", "sb_abi_version")
ABI_VERSION = 2


class SbTensor(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_h", ctypes.c_int64),
                ("stride_t", ctypes.c_int64)]


class SbParams(ctypes.Structure):
    _fields_ = [
        ("struct_bytes", ctypes.c_int32), ("dtype", ctypes.c_int32), ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("num_seq", ctypes.c_int32),
        ("tokens", ctypes.c_int64), ("max_seqlen", ctypes.c_int32), ("attend_current", ctypes.c_int32),
        ("cu_seqlens_int64", ctypes.c_int32), ("logit_scale", ctypes.c_float), ("flags", ctypes.c_int32),
        ("reserved", ctypes.c_int32), ("cu_seqlens", ctypes.c_void_p),
        ("q", SbTensor), ("k", SbTensor), ("v", SbTensor), ("o", SbTensor),
        ("rem", ctypes.c_void_p), ("log_rem", ctypes.c_void_p),
        ("d_o", SbTensor), ("d_rem", ctypes.c_void_p),
        ("dq", SbTensor), ("dk", SbTensor), ("dv", SbTensor),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t), ("status", ctypes.c_void_p),
        ("attn_weights", ctypes.c_void_p), ("attn_cols", ctypes.c_int64),
    ]


class SbError(RuntimeError):
    pass


_lib = None


def load(path: str | None = None) -> ctypes.CDLL:
    """Loads the library once; raises ``SbError`` with build instructions if it is absent."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    path = path or LIB_PATH
    if not os.path.exists(path):
        raise SbError(f"{path} not found. Build it with `python setup.py build_ext --inplace` or "
                      "`python stickbreaking_attention_b200/build.py`; there is no fallback implementation.")
    lib = ctypes.CDLL(path)
    lib.sb_workspace_bytes.restype = ctypes.c_size_t
    lib.sb_workspace_bytes.argtypes = [ctypes.POINTER(SbParams), ctypes.c_int]
    for name in ("sb_fwd", "sb_bwd", "sb_fwd_static_scratch"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.POINTER(SbParams), ctypes.c_void_p]
    lib.sb_kernel_path.restype = ctypes.c_int
    lib.sb_kernel_path.argtypes = [ctypes.POINTER(SbParams)]
    lib.sb_last_launch_count.restype = ctypes.c_int
    lib.sb_last_error.restype = ctypes.c_char_p
    lib.sb_set_backward_scratch_budget.restype = ctypes.c_size_t
    lib.sb_set_backward_scratch_budget.argtypes = [ctypes.c_size_t]
    lib.sb_abi_version.restype = ctypes.c_int
    if lib.sb_abi_version() != ABI_VERSION:
        raise SbError(f"{path}: ABI version {lib.sb_abi_version()} but this binding speaks {ABI_VERSION}; "
                      "rebuild with `python stickbreaking_attention_b200/build.py --force`")
    _lib = lib
    return lib


def tensor_arg(t: torch.Tensor | None, fixed: bool) -> SbTensor:
    """(H,T,d) packed or (B,H,T,d) fixed tensor -> SbTensor with element strides."""
    if t is None:
        return SbTensor(None, 0, 0, 0)
    if fixed:
        sb, sh, st, sd = t.stride()
    else:
        sb = 0
        sh, st, sd = t.stride()
    assert sd == 1 or t.shape[-1] == 1
    return SbTensor(t.data_ptr(), sb, sh, st)


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def check_call(lib, rc: int, what: str):
    if rc != 0:
        raise SbError(f"{what} failed with status {rc}: {lib.sb_last_error().decode()}")
