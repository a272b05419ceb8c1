"""Parity at the benchmark's full sequence lengths.

A dense oracle over 131072 tokens does not fit, so the long case is checked through (a) the oracle on sampled
blocks of query rows (o, rem and dq of a row depend on that row and its keys only), (b) exact scaling properties
and (c) structural facts; a 16384-token sequence is checked in full against the row-blocked oracle."""
import pytest
import torch

import helpers as H
from oracle import sb_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sb(cuda_device):
    import stickbreaking_attention_b200 as sb
    yield sb
    sb.check_status(cuda_device)


def oracle_rows(q, k, v, do, drem, i0, i1, scale):
    """o, rem, dq of query rows [i0, i1) of one sequence, fp32, closed-form gradients (see oracle.varlen_rowblocked_grads)."""
    q, k, v, do, drem = (t.float() for t in (q, k, v, do, drem))
    z, allowed, att = O._row_block(q[:, i0:i1], k[:, :i1], v[:, :i1], i0, scale, False)
    o = att @ v[:, :i1]
    rem = 1 - att.sum(-1)
    g = att * (do[:, i0:i1] @ v[:, :i1].transpose(-1, -2) - drem[:, i0:i1, None])
    c = torch.cumsum(g, -1)
    dz = torch.where(allowed, g - torch.sigmoid(z) * c, torch.zeros(()))
    return o, rem, scale * (dz @ k[:, :i1])


def test_16k_sequence_full_oracle(sb, cuda_device):
    dtype = torch.bfloat16
    L = 16384
    q, k, v, do, drem = H.make_inputs((1, L, 128), dtype, seed=16, recipe="reference")
    cu = torch.tensor([L])
    got = H.run_varlen(sb, q, k, v, do, drem, cu, cuda_device, max_seqlens=L)
    want = O.varlen_rowblocked_grads(q.float(), k.float(), v.float(), cu, do.float(), drem.float(), block=2048)
    H.assert_parity(got, want, dtype, "L16384")


@pytest.mark.parametrize("std", [0.5, 1.0])
def test_131072_sequence_sampled_rows_and_properties(sb, cuda_device, std):
    """One head of the long-context configuration (131072 tokens, head_dim 128, q/k/v ~ N(0, std^2))."""
    dtype = torch.bfloat16
    L, d = 131072, 128
    q, k, v, do, drem = H.make_inputs((1, L, d), dtype, seed=131, std=std)
    cu = torch.tensor([L])
    o, rem, dq, dk, dv = H.run_varlen(sb, q, k, v, do, drem, cu, cuda_device, max_seqlens=L)
    for t in (o, rem, dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    assert torch.all(o[:, 0] == 0) and torch.all(rem[:, 0] == 1)
    assert rem.float().min() >= 0 and rem.float().max() <= 1
    scale = d ** -0.5
    for i0 in (0, 4000, 65536 - 64, L - 128):
        i1 = i0 + 128
        wo, wr, wdq = oracle_rows(q, k, v, do, drem, i0, i1, scale)
        assert H.max_abs(o[:, i0:i1], wo) <= 2e-2
        assert H.max_abs(rem[:, i0:i1], wr) <= 2e-2
        assert H.rel_l2(dq[:, i0:i1], wdq) <= 5e-2
    # exact scaling (powers of two survive every rounding): doubling v doubles o and leaves rem alone;
    # doubling dO and dRem doubles every gradient
    o2, rem2, _, _, _ = H.run_varlen(sb, q, k, 2 * v, do, drem, cu, cuda_device, max_seqlens=L)
    assert torch.equal(o2.float(), 2 * o.float()) and torch.equal(rem2, rem)
    _, _, dq2, dk2, dv2 = H.run_varlen(sb, q, k, v, 2 * do, 2 * drem, cu, cuda_device, max_seqlens=L)
    for a, b in ((dq2, dq), (dk2, dk), (dv2, dv)):
        assert torch.equal(a.float(), 2 * b.float())
