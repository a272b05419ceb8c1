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


def oracle_rows(q, k, v, do, drem, i0, i1, scale, tail_keys=0):
    """o, rem, dq of query rows [i0, i1) of one sequence, fp32, closed-form gradients (see oracle.varlen_rowblocked_grads).
    With tail_keys = n also the contributions of these rows to dk and dv of the keys [i1 - n, i1)."""
    q, k, v, do, drem = (t.float() for t in (q, k, v, do, drem))
    z, allowed, att = O._row_block(q[:, i0:i1], k[:, :i1], v[:, :i1], i0, scale, False)
    o = att @ v[:, :i1]
    rem = 1 - att.sum(-1)
    g = att * (do[:, i0:i1] @ v[:, :i1].transpose(-1, -2) - drem[:, i0:i1, None])
    c = torch.cumsum(g, -1)
    dz = torch.where(allowed, g - torch.sigmoid(z) * c, torch.zeros(()))
    if tail_keys:
        dk = scale * dz[..., i1 - tail_keys:].transpose(-1, -2) @ q[:, i0:i1]
        dv = att[..., i1 - tail_keys:].transpose(-1, -2) @ do[:, i0:i1]
        return o, rem, scale * (dz @ k[:, :i1]), dk, dv
    return o, rem, scale * (dz @ k[:, :i1])


@pytest.mark.parametrize("mode", ["stored", "recompute"])
def test_16k_sequence_full_oracle(sb, cuda_device, mode):
    """One 16384-token sequence against the row-blocked oracle, in both modes of the backward (the recomputing dK/dV
    kernel is the one the 131072-token configuration takes)."""
    dtype = torch.bfloat16
    L = 16384
    q, k, v, do, drem = H.make_inputs((1, L, 128), dtype, seed=16, recipe="reference")
    cu = torch.tensor([L])
    with sb.small_backward_workspace(mode == "recompute"):
        got = H.run_varlen(sb, q, k, v, do, drem, cu, cuda_device, max_seqlens=L)
    want = O.varlen_rowblocked_grads(q.float(), k.float(), v.float(), cu, do.float(), drem.float(), block=2048)
    rep = H.assert_parity(got, want, dtype, f"L16384 {mode}")
    print(f"L16384 {mode}: max-abs o {rep['o'][0]:.3e} rem {rep['rem'][0]:.3e}, rel-L2 dq {rep['dq'][1]:.2e} "
          f"dk {rep['dk'][1]:.2e} dv {rep['dv'][1]:.2e}")


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
        assert H.worst_output_error(o[:, i0:i1], wo, dtype)[0] <= 1.0
        assert H.max_abs(rem[:, i0:i1], wr) <= 2e-2
        assert H.rel_l2(dq[:, i0:i1], wdq) <= 5e-2
    # dk and dv of the last 256 keys receive contributions from the last 256 query rows only (a key is seen by later
    # queries), so the oracle on those rows gives them in full; this workload runs the recomputing dK/dV kernel
    _, _, _, wdk, wdv = oracle_rows(q, k, v, do, drem, L - 256, L, scale, tail_keys=256)
    assert H.rel_l2(dk[:, L - 256:], wdk) <= 5e-2
    assert H.rel_l2(dv[:, L - 256:], wdv) <= 5e-2
    print(f"L131072 std={std}: rel-L2 dk tail {H.rel_l2(dk[:, L - 256:], wdk):.2e} dv tail {H.rel_l2(dv[:, L - 256:], wdv):.2e}")
    # exact scaling (powers of two survive every rounding): doubling v doubles o and leaves rem alone;
    # doubling dO and dRem doubles every gradient
    o2, rem2, _, _, _ = H.run_varlen(sb, q, k, 2 * v, do, drem, cu, cuda_device, max_seqlens=L)
    assert torch.equal(o2.float(), 2 * o.float()) and torch.equal(rem2, rem)
    _, _, dq2, dk2, dv2 = H.run_varlen(sb, q, k, v, 2 * do, 2 * drem, cu, cuda_device, max_seqlens=L)
    for a, b in ((dq2, dq), (dk2, dk), (dv2, dv)):
        assert torch.equal(a.float(), 2 * b.float())


def _check_sampled_sequences(sb, dev, q, k, v, do, drem, lengths, picks, *, backward, what):
    """Runs the whole packed batch on the GPU and compares the picked sequences (each is independent of the others)
    with the oracle run on that sequence alone."""
    cu = torch.tensor(lengths).cumsum(0)
    starts = [0] + cu.tolist()[:-1]
    if backward:
        got = H.run_varlen(sb, q, k, v, do, drem, cu, dev, max_seqlens=max(lengths))
    else:
        with torch.no_grad():
            o, rem = sb.sb_attn_varlen(q.to(dev), k.to(dev), v.to(dev), cu.to(dev), max(lengths), zero_start=False)
        got = (o.cpu(), rem.cpu())
    for t in got:
        assert torch.isfinite(t.float()).all()
    assert torch.all(got[0][:, starts] == 0) and torch.all(got[1][:, starts] == 1)
    worst = dict(o=0.0, rem=0.0, grad=0.0, abs_o=0.0)
    for s in picks:
        a, b = starts[s], starts[s] + lengths[s]
        one = torch.tensor([lengths[s]])
        want = H.oracle_varlen(q[:, a:b], k[:, a:b], v[:, a:b], do[:, a:b], drem[:, a:b], one)
        mine = [t[:, a:b] for t in got]
        if backward:
            rep = H.assert_parity(mine, want, q.dtype, f"{what} sequence {s}")
            worst["grad"] = max(worst["grad"], *(rep[n][1] for n in ("dq", "dk", "dv")))
        else:
            for name, x, y in zip(("o", "rem"), mine, want[:2]):
                ratio, err, ref, ref_rounded, val = H.worst_output_error(x, y, q.dtype)
                assert ratio <= 1.0, (f"{what} sequence {s}: {name} off by {err:.3e} at oracle value {ref:.6g} "
                                      f"(rounded {ref_rounded:.6g}, got {val:.6g})")
        worst["o"] = max(worst["o"], H.max_abs(mine[0], want[0]))
        worst["rem"] = max(worst["rem"], H.max_abs(mine[1], want[1]))
        worst["abs_o"] = max(worst["abs_o"], float(want[0].abs().max()))
    print(f"{what}: over {len(picks)} sampled sequences max-abs o {worst['o']:.3e} (largest |o| {worst['abs_o']:.2f}) "
          f"rem {worst['rem']:.3e}, largest gradient rel-L2 {worst['grad']:.2e}")
    return got


def test_many_short_sequences_forward_shape_of_the_serving_configuration(sb, cuda_device):
    """4096 sequences of 128..512 tokens, head_dim 64, q/k/v ~ N(0, 1), forward only: about 1.3 M tokens, more work
    items than fit the forward's persistent grid many times over.  Two of the configuration's 32 heads run (every head
    is independent and takes the same code; the CPU oracle sets the budget); sampled sequences against the oracle."""
    gen = torch.Generator().manual_seed(55)
    lengths = torch.randint(128, 513, (4096,), generator=gen).tolist()
    q, k, v, do, drem = H.make_inputs((2, sum(lengths), 64), torch.bfloat16, seed=56, std=1.0)
    picks = [0, 1, 777, 2048, 4094, 4095, lengths.index(max(lengths)), lengths.index(min(lengths))]
    _check_sampled_sequences(sb, cuda_device, q, k, v, do, drem, lengths, picks, backward=False, what="short")


def test_lognormal_lengths_training_configuration(sb, cuda_device):
    """65536 tokens cut into sequences of lognormal length (median 1024, clipped to 64..16384), head_dim 128, q/k/v ~
    N(0, 1), forward and backward, two of the configuration's 32 heads: the uneven mix the weight-ordered schedule is
    built for.  Sampled sequences, the longest and the shortest among them, against the oracle."""
    gen = torch.Generator().manual_seed(3)
    lengths, total = [], 65536
    while sum(lengths) < total:
        n = int(torch.exp(torch.randn((), generator=gen) + 6.931).clamp(64, 16384))
        lengths.append(min(n, total - sum(lengths)))
    q, k, v, do, drem = H.make_inputs((2, total, 128), torch.bfloat16, seed=57, std=1.0)
    order = sorted(range(len(lengths)), key=lambda i: lengths[i])
    picks = sorted({order[0], order[len(order) // 2], order[-1], 0, len(lengths) - 1})
    picks = [s for s in picks if lengths[s] <= 8192] or [order[0]]
    _check_sampled_sequences(sb, cuda_device, q, k, v, do, drem, lengths, picks, backward=True, what="lognormal")
