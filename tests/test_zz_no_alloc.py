"""sb_fwd_static_scratch: the forward entry point for callers that cannot allocate device memory
(fixed-arena hosts, latency-critical loops, plain C callers without an allocator).  It must give the same
results as sb_fwd while using only the scratch array built into the library.  Collected last on purpose:
the array is shared by every call in the process, so this file runs after all other tests have had their turn."""
import ctypes

import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def _params(sb, q, k, v, cu, max_len):
    from stickbreaking_attention_b200 import _cabi, ops
    prm = _cabi.SbParams()
    ops._fill(prm, fixed=False, q=q, k=k, v=v, cu_seqlens=cu, max_seqlens=max_len,
              logit_scale=q.shape[-1] ** -0.5, attend_current=False, leading_zero=False)
    o = torch.empty_like(q)
    rem = torch.empty(q.shape[:2], dtype=q.dtype, device=q.device)
    log_rem = torch.empty(q.shape[:2], dtype=torch.float64, device=q.device)
    prm.o = _cabi.tensor_arg(o, False)
    prm.rem, prm.log_rem = rem.data_ptr(), log_rem.data_ptr()
    return prm, (o, rem, log_rem)


def _forward_both_ways(sb, device, dtype, lengths, d, seed):
    from stickbreaking_attention_b200 import _cabi
    lib = _cabi.load()
    q, k, v, _, _ = (t.to(device) for t in H.make_inputs((3, sum(lengths), d), dtype, seed=seed))
    cu = torch.tensor(lengths, dtype=torch.int32).cumsum(0).to(torch.int32).to(device)
    stream = torch.cuda.current_stream(device).cuda_stream

    prm, want = _params(sb, q, k, v, cu, max(lengths))
    ws = torch.empty(lib.sb_workspace_bytes(prm, 0), dtype=torch.uint8, device=device)
    prm.workspace, prm.workspace_bytes = ws.data_ptr(), ws.numel()
    assert lib.sb_fwd(prm, stream) == 0, lib.sb_last_error()

    prm2, got = _params(sb, q, k, v, cu, max(lengths))      # no workspace given at all
    assert lib.sb_fwd_static_scratch(prm2, stream) == 0, lib.sb_last_error()
    torch.cuda.synchronize(device)

    tol = H.TOL[dtype]["out"]
    assert H.max_abs(got[0], want[0]) <= tol
    assert H.max_abs(got[1], want[1]) <= tol
    assert H.max_abs(got[2], want[2]) <= 1e-3
    assert torch.isfinite(got[0].float()).all()


def test_static_scratch_forward_matches_sb_fwd_twice_in_a_row(cuda_device):
    import stickbreaking_attention_b200 as sb
    # two calls back to back that leave different sequence tables in the shared scratch, on both kernel paths
    _forward_both_ways(sb, cuda_device, torch.bfloat16, [300, 17, 129], 128, seed=21)
    _forward_both_ways(sb, cuda_device, torch.bfloat16, [64, 1, 200, 40, 5, 128, 77], 64, seed=22)
    _forward_both_ways(sb, cuda_device, torch.float32, [90, 33], 32, seed=23)
    sb.check_status(cuda_device)


def test_static_scratch_rejects_what_does_not_fit(cuda_device):
    import stickbreaking_attention_b200 as sb
    from stickbreaking_attention_b200 import _cabi
    lib = _cabi.load()
    n = 6000                                                   # more sequences than the built-in scratch can index
    q = torch.zeros(1, n, 64, dtype=torch.bfloat16, device=cuda_device)
    cu = torch.arange(1, n + 1, dtype=torch.int32, device=cuda_device)
    prm, _ = _params(sb, q, q, q, cu, 1)
    assert lib.sb_workspace_bytes(prm, 0) > _cabi.SB_STATIC_SCRATCH_BYTES
    rc = lib.sb_fwd_static_scratch(prm, torch.cuda.current_stream(cuda_device).cuda_stream)
    assert rc == 2 and b"scratch" in lib.sb_last_error()
    # the same rule on the CUDA-core path (fp32), whose work items are 32 tokens: 600 sequences in 262144 tokens fit
    # in bf16 (256-token items) and do not in fp32
    lengths = torch.full((600,), 436, dtype=torch.int32)
    cu = lengths.cumsum(0).to(torch.int32).to(cuda_device)
    for dtype, fits in ((torch.bfloat16, True), (torch.float32, False)):
        q = torch.zeros(1, 262144, 64, dtype=dtype, device=cuda_device)
        prm, _ = _params(sb, q, q, q, cu, 436)
        assert (lib.sb_workspace_bytes(prm, 0) <= _cabi.SB_STATIC_SCRATCH_BYTES) == fits
        rc = lib.sb_fwd_static_scratch(prm, torch.cuda.current_stream(cuda_device).cuda_stream)
        assert (rc == 0) == fits, lib.sb_last_error()
    torch.cuda.synchronize(cuda_device)
    sb.check_status(cuda_device)
