"""The C-ABI library loads without a GPU and exports every symbol include/sb_b200.h declares."""
import ctypes
import os
import re

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "sb_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return re.findall(r"SB_EXPORT[^;(]*?\b(sb_\w+)\s*\(", text)


def test_header_declares_the_entry_points():
    names = declared_symbols()
    for must in ("sb_fwd", "sb_bwd", "sb_workspace_bytes", "sb_kernel_path", "sb_last_error", "sb_abi_version"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from stickbreaking_attention_b200 import _cabi
    lib = _cabi.load()
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert set(_cabi.EXPORTS) <= set(declared_symbols())
    assert lib.sb_abi_version() == _cabi.ABI_VERSION == 2


def test_struct_layout_matches_header():
    """struct_bytes is checked by the library, so a mismatch between the ctypes mirror and the C
    struct shows up as an argument error from a pure host-side call."""
    from stickbreaking_attention_b200 import _cabi
    lib = _cabi.load()
    p = _cabi.SbParams()
    p.struct_bytes = ctypes.sizeof(_cabi.SbParams)
    p.dtype, p.batch, p.heads, p.head_dim, p.tokens = 1, 1, 2, 64, 1024
    p.num_seq = 3
    p.cu_seqlens = 256          # never dereferenced by the host-side queries
    assert lib.sb_workspace_bytes(p, 0) not in (0, 2 ** 64 - 1)
    assert lib.sb_workspace_bytes(p, 1) > lib.sb_workspace_bytes(p, 0)
    p.struct_bytes -= 8
    assert lib.sb_workspace_bytes(p, 0) == 2 ** 64 - 1
    assert b"struct_bytes" in lib.sb_last_error()


def test_scratch_budget_changes_the_backward_workspace():
    """sb_set_backward_scratch_budget is a host-side setting: a smaller budget gives a smaller backward workspace."""
    from stickbreaking_attention_b200 import _cabi
    lib = _cabi.load()
    p = _cabi.SbParams()
    p.struct_bytes = ctypes.sizeof(_cabi.SbParams)
    p.dtype, p.batch, p.heads, p.head_dim, p.tokens = 1, 2, 8, 128, 2048
    for name in ("q", "k", "v", "d_o", "dq", "dk", "dv"):     # plausible addresses and strides; never dereferenced
        setattr(p, name, _cabi.SbTensor(4096, 8 * 2048 * 128, 2048 * 128, 128))
    default = lib.sb_set_backward_scratch_budget(0)
    assert default == 8 << 30
    big = lib.sb_workspace_bytes(p, 1)
    per_head = 2 * 136 * 65536                       # 2 batch elements x 136 tile pairs x 64 KiB
    assert big >= 8 * per_head
    assert lib.sb_set_backward_scratch_budget(3 * per_head) == default
    assert lib.sb_workspace_bytes(p, 1) < 4 * per_head
    assert lib.sb_set_backward_scratch_budget(default) == 3 * per_head
    assert lib.sb_workspace_bytes(p, 1) == big
    p.reserved = 1
    assert lib.sb_workspace_bytes(p, 1) == 2 ** 64 - 1 and b"reserved" in lib.sb_last_error()


def test_missing_library_fails_loudly(tmp_path):
    from stickbreaking_attention_b200 import _cabi
    with pytest.raises(_cabi.SbError, match="no fallback"):
        _cabi.load(str(tmp_path / "libsb_b200.so"))
