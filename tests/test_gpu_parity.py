"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the reference's golden vectors."""
import math

import pytest
import torch

from conftest import load_golden
import helpers as H

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.float16]


@pytest.fixture(scope="module")
def sb(cuda_device):
    import stickbreaking_attention_b200 as sb
    yield sb
    sb.check_status(cuda_device)


def cu_of(lengths, zero_start=False, dtype=torch.int64):
    ends = torch.tensor(lengths, dtype=dtype).cumsum(0).to(dtype)
    return torch.cat([torch.zeros(1, dtype=dtype), ends]) if zero_start else ends


# ---- golden vectors produced by the reference itself -------------------------------------------------

@pytest.mark.parametrize("ac", [0, 1])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_golden_tiny_varlen(sb, cuda_device, ac, dtype):
    g = load_golden(f"tiny_varlen_ac{ac}")
    ins = [g[n].to(dtype) for n in ("q", "k", "v", "do", "drem")]
    got = H.run_varlen(sb, *ins, cu_of(g["lengths"]), cuda_device, attend_current=bool(ac))
    if dtype == torch.float32:
        want = [g[n] for n in ("o", "rem", "dq", "dk", "dv")]
    else:   # the stored vectors are for the unrounded inputs; re-run the oracle on the rounded ones
        want = H.oracle_varlen(*ins, cu_of(g["lengths"]), attend_current=bool(ac))
    H.assert_parity(got, want, dtype, "tiny_varlen")


@pytest.mark.parametrize("ac", [0, 1])
def test_golden_tiny_fixed_fp32(sb, cuda_device, ac):
    g = load_golden(f"tiny_fixed_ac{ac}")
    ins = [g[n] for n in ("q", "k", "v", "do", "drem")]
    got = H.run_fixed(sb, *ins, cuda_device, attend_current=bool(ac))
    H.assert_parity(got, [g[n] for n in ("o", "rem", "dq", "dk", "dv")], torch.float32, "tiny_fixed")


@pytest.mark.parametrize("ac", [0, 1])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_golden_reference_recipe(sb, cuda_device, ac, dtype):
    """bf16-representable inputs (d=128): the bf16 tensor-core path and the fp32 path see exactly the
    inputs the reference oracle saw."""
    g = load_golden(f"recipe_varlen_ac{ac}")
    ins = [g[n].to(dtype) for n in ("q", "k", "v", "do", "drem")]
    got = H.run_varlen(sb, *ins, cu_of(g["lengths"]), cuda_device, attend_current=bool(ac))
    H.assert_parity(got, [g[n] for n in ("o", "rem", "dq", "dk", "dv")], dtype, "recipe")


def test_golden_c1_config(sb, cuda_device):
    """BASELINE config 1: H=4, d=64, lengths [128,256,64,512], seed 0, fp32, zero_start=False."""
    g = load_golden("c1")
    torch.manual_seed(0)
    shape = (4, 960, 64)
    q, k, v, do = (torch.randn(shape) for _ in range(4))
    drem = torch.randn(shape[:2])
    got = H.run_varlen(sb, q, k, v, do, drem, cu_of(g["lengths"]), cuda_device, inv_temp=1 / 8)
    stride = int(g["row_stride"])
    H.assert_parity([t[:, ::stride] for t in got], [g[n] for n in ("o", "rem", "dq", "dk", "dv")],
                    torch.float32, "c1")


# ---- seeded inputs against the oracle -------------------------------------------------------------------

RAGGED = [1, 2, 63, 64, 65, 127, 128, 129, 31, 300]


@pytest.mark.parametrize("ac", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [64, 72, 96, 128])
def test_varlen_ragged(sb, cuda_device, dtype, d, ac):
    ins = H.make_inputs((3, sum(RAGGED), d), dtype, seed=d + int(ac))
    cu = cu_of(RAGGED)
    got = H.run_varlen(sb, *ins, cu, cuda_device, attend_current=ac, max_seqlens=max(RAGGED))
    H.assert_parity(got, H.oracle_varlen(*ins, cu, attend_current=ac), dtype, "ragged")
    if not ac:   # first token of each sequence attends to nothing
        starts = [0] + cu.tolist()[:-1]
        assert torch.all(got[0][:, starts] == 0) and torch.all(got[1][:, starts] == 1)


@pytest.mark.parametrize("d", [64, 104, 128])
def test_varlen_many_uneven_sequences(sb, cuda_device, d):
    """More work items than SMs, lengths from 1 token to 21 tiles: exercises the weight-ordered item tables
    (several classes, sequences longer than one class span) and the persistent forward's walk over them."""
    gen = torch.Generator().manual_seed(5)
    lengths = torch.randint(1, 900, (70,), generator=gen).tolist() + [2600, 1, 129, 2049]
    # N(0, 1) inputs, as the benchmark configurations state them: among millions of outputs a few reach |o| > 4, where
    # one bf16 step exceeds the max-abs tolerance; helpers.out_bound says how those elements are judged
    ins = H.make_inputs((4, sum(lengths), d), torch.bfloat16, seed=d, std=1.0)
    cu = cu_of(lengths)
    got = H.run_varlen(sb, *ins, cu, cuda_device, max_seqlens=max(lengths))
    rep = H.assert_parity(got, H.oracle_varlen(*ins, cu), torch.bfloat16, "uneven")
    print(f"uneven d={d}: worst o {rep['o_worst']}, max-abs o {rep['o'][0]:.3e} rem {rep['rem'][0]:.3e}, "
          f"rel-L2 dq {rep['dq'][1]:.2e} dk {rep['dk'][1]:.2e} dv {rep['dv'][1]:.2e}")


def test_headline_benchmark_shape(sb, cuda_device):
    """The configuration the headline benchmark is quoted on, at its own shape and input distribution: 16 heads,
    head_dim 128, 8 packed sequences of 2048 tokens, q/k/v/dO/dRem ~ N(0, 1) in bf16.  The GPU runs all 16 heads; the
    oracle (dense, fp32, autograd) runs on four of them, all 8 sequences each."""
    dtype = torch.bfloat16
    lengths = [2048] * 8
    ins = H.make_inputs((16, sum(lengths), 128), dtype, seed=2, std=1.0)
    cu = cu_of(lengths)
    for small in (False, True):
        with sb.small_backward_workspace(small):
            got = H.run_varlen(sb, *ins, cu, cuda_device, max_seqlens=2048)
        heads = [0, 5, 10, 15]
        want = H.oracle_varlen(*[t[heads] for t in ins], cu)
        rep = H.assert_parity([t[heads] for t in got], want, dtype, f"headline shape small={small}")
        print(f"headline shape small={small}: worst o {rep['o_worst']}, max-abs o {rep['o'][0]:.3e} rem {rep['rem'][0]:.3e}, "
              f"rel-L2 dq {rep['dq'][1]:.2e} dk {rep['dk'][1]:.2e} dv {rep['dv'][1]:.2e}")
        for t in got:
            assert torch.isfinite(t.float()).all()


@pytest.mark.parametrize("d", [128, 64])
def test_rows_of_other_sequences_cannot_leak_in(sb, cuda_device, d):
    """The tensor-core kernels load K/V (backward: Q/dO) tiles that reach past the end of their sequence, into the next
    sequence or into whatever lies behind the last one.  One whole sequence and the unused tail of the packed batch are
    filled with NaN and Inf here: every other sequence must come out finite and unchanged (a zero weight times a
    foreign NaN must never reach an accumulator), in both modes of the backward."""
    dtype = torch.bfloat16
    lengths = [100, 200, 77, 130, 321]          # none a multiple of 64: every sequence ends inside a tile
    total = sum(lengths) + 90                   # 90 tokens behind the last sequence belong to nobody
    q, k, v, do, drem = H.make_inputs((3, total, d), dtype, seed=90 + d)
    cu = cu_of(lengths)
    want = H.oracle_varlen(*[t[:, :sum(lengths)] for t in (q, k, v, do, drem)], cu)
    starts = [0] + cu.tolist()
    poisoned = 2
    a, b = starts[poisoned], starts[poisoned + 1]
    bad = [t.clone() for t in (q, k, v, do, drem)]
    for i, t in enumerate(bad):
        t[:, a:b] = float("nan") if i % 2 == 0 else float("inf")
        t[:, sum(lengths):] = float("inf") if i % 2 == 0 else float("nan")
    for small in (False, True):
        with sb.small_backward_workspace(small):
            got = H.run_varlen(sb, *bad, cu, cuda_device, max_seqlens=max(lengths))
        for s in range(len(lengths)):
            if s == poisoned:
                continue
            lo, hi = starts[s], starts[s + 1]
            H.assert_parity([t[:, lo:hi] for t in got], [t[:, lo:hi] for t in want], dtype,
                            f"sequence {s} beside a poisoned one, small={small}")
        for t in got:
            assert torch.all(t[:, sum(lengths):] == 0)


@pytest.mark.parametrize("mode", ["stored", "recompute"])
def test_backward_head_chunks(sb, cuda_device, mode):
    """The backward works through the heads in chunks when its scratch would exceed the budget.  With the budget
    lowered so that only one or two heads fit, the result must be bitwise what the unchunked call gives."""
    from stickbreaking_attention_b200 import ops
    lengths = [300, 129, 512]
    ins = H.make_inputs((5, sum(lengths), 128), torch.bfloat16, seed=77)
    cu = cu_of(lengths)
    with sb.small_backward_workspace(mode == "recompute"):
        whole = H.run_varlen(sb, *ins, cu, cuda_device, max_seqlens=512)
        # scratch per head: stored tiles 64 KiB per tile pair, boundary records 4 KiB; this batch has at most
        # (8 + 3 tiles) * (4 + 1) / 2 pair slots per head
        per_head = 28 * (65536 if mode == "stored" else 4096)
        for heads_per_chunk in (2, 1):
            old = ops.set_backward_scratch_budget(per_head * heads_per_chunk + per_head // 2)
            try:
                chunked = H.run_varlen(sb, *ins, cu, cuda_device, max_seqlens=512)
            finally:
                ops.set_backward_scratch_budget(old)
            for x, y, name in zip(whole, chunked, ("o", "rem", "dq", "dk", "dv")):
                assert torch.equal(x, y), f"{name}, {heads_per_chunk} head(s) per chunk"
    H.assert_parity(whole, H.oracle_varlen(*ins, cu), torch.bfloat16, "chunked backward")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_return_attention(sb, cuda_device, dtype):
    """The optional W output (the reference's `return_attention`, sb_varlen_fwd.py:195-202, 421-425) against the
    oracle's attention matrix, sequence by sequence; o and rem are unchanged by asking for it."""
    from stickbreaking_attention_b200 import ops
    from oracle import sb_oracle as O
    lengths = [70, 1, 33, 130]
    q, k, v, _, _ = H.make_inputs((2, sum(lengths), 64), dtype, seed=12)
    cu = cu_of(lengths).to(cuda_device)
    qd, kd, vd = (t.to(cuda_device) for t in (q, k, v))
    o, rem, _, w = ops.varlen_fwd(qd, kd, vd, cu, max(lengths), 0.125, return_attention=True)
    o2, rem2, _ = ops.varlen_fwd(qd, kd, vd, cu, max(lengths), 0.125)
    assert w.shape == (2, sum(lengths), max(lengths)) and w.dtype == torch.float32
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert H.max_abs(o, o2) <= tol and H.max_abs(rem, rem2) <= tol
    w = w.cpu()
    start = 0
    for n in lengths:
        _, _, att = O._row_block(q[:, start:start + n].float(), k[:, start:start + n].float(), v[:, start:start + n].float(),
                                 0, 0.125, False)
        assert H.max_abs(w[:, start:start + n, :n], att) <= 1e-5
        assert torch.all(w[:, start:start + n, n:] == 0)
        assert H.max_abs(1 - w[:, start:start + n].sum(-1), rem[:, start:start + n].float().cpu()) <= tol
        start += n
    # fixed-length form
    o4, rem4, _, w4 = ops.attn_fwd(qd[None, :, :130], kd[None, :, :130], vd[None, :, :130], 0.125, return_attention=True)
    _, _, att = O._row_block(q[:, :130].float(), k[:, :130].float(), v[:, :130].float(), 0, 0.125, False)
    assert H.max_abs(w4[0].cpu(), att) <= 1e-5


@pytest.mark.parametrize("d", [128, 64, 40])
def test_backward_modes_agree(sb, cuda_device, d):
    """Default backward (the dQ kernel stores its A / dz tiles, dK/dV are GEMMs over them) against the small-workspace
    backward (dK/dV recomputed from boundary values): both within the bound of the oracle and close to each other."""
    lengths = [700, 129, 1, 1333, 64, 512]
    ins = H.make_inputs((3, sum(lengths), d), torch.bfloat16, seed=11)
    cu = cu_of(lengths)
    want = H.oracle_varlen(*ins, cu)
    stored = H.run_varlen(sb, *ins, cu, cuda_device, max_seqlens=max(lengths))
    with sb.small_backward_workspace():
        recomputed = H.run_varlen(sb, *ins, cu, cuda_device, max_seqlens=max(lengths))
    H.assert_parity(stored, want, torch.bfloat16, "stored tiles")
    H.assert_parity(recomputed, want, torch.bfloat16, "recomputed tiles")
    for a, b, name in zip(stored, recomputed, ("o", "rem", "dq", "dk", "dv")):
        assert H.rel_l2(a, b) <= 4e-3, name


@pytest.mark.parametrize("ac", [False, True])
@pytest.mark.parametrize("dtype,d", [(torch.bfloat16, 128), (torch.bfloat16, 64), (torch.float16, 96),
                                     (torch.bfloat16, 50), (torch.float32, 64)])
def test_fused_rem_v_varlen(sb, cuda_device, dtype, d, ac):
    """out = o + rem * v in one operator (forward epilogue, backward fold) against the oracle's o, rem and gradients
    combined on the CPU; N(0, 0.5^2) inputs keep |out| below 2, where a bf16 step is still inside the bound."""
    lengths = [300, 1, 129, 700, 64, 257]
    q, k, v, dout, _ = H.make_inputs((3, sum(lengths), d), dtype, seed=20 + d, std=0.5)
    cu = cu_of(lengths, True)
    got = H.run_fused(sb, q, k, v, dout, cuda_device, cu, max_seqlens=max(lengths), zero_start=True,
                      attend_current=ac)
    want = H.oracle_fused(q, k, v, dout, cu, zero_start=True, attend_current=ac)
    H.assert_fused_parity(got, want, dtype, "fused varlen")


def test_fused_rem_v_matches_unfused_and_leaves_tail_zero(sb, cuda_device):
    """The fused operator against the two-output operator followed by the callers' arithmetic, both modes of the
    backward, with tokens past the last sequence end (their rows of out and of the gradients stay zero)."""
    lengths, total = [500, 130, 1000], 1700
    q, k, v, dout, _ = H.make_inputs((2, total, 128), torch.bfloat16, seed=31, std=0.5)
    cu = cu_of(lengths)
    want = H.oracle_fused(q[:, :1630], k[:, :1630], v[:, :1630], dout[:, :1630], cu)
    for small in (False, True):
        with sb.small_backward_workspace(small):
            got = H.run_fused(sb, q, k, v, dout, cuda_device, cu, max_seqlens=1000, zero_start=False)
        H.assert_fused_parity([t[:, :1630] for t in got], want, torch.bfloat16, f"fused small={small}")
        for t in got:
            assert torch.all(t[:, 1630:] == 0)
    qd, kd, vd = (t.to(cuda_device).requires_grad_(True) for t in (q, k, v))
    o, rem = sb.sb_attn_varlen(qd, kd, vd, cu.to(cuda_device), 1000, zero_start=False)
    out2 = o + rem[..., None] * vd
    grads2 = torch.autograd.grad(out2, (qd, kd, vd), dout.to(cuda_device))
    for a, b in zip(got, (out2,) + grads2):
        assert H.rel_l2(a[:, :1630], b.detach().cpu()[:, :1630]) <= 1e-2


@pytest.mark.parametrize("shape,dtype", [((2, 3, 384, 128), torch.bfloat16), ((1, 2, 300, 64), torch.float16),
                                         ((1, 2, 200, 32), torch.float32)])
def test_fused_rem_v_fixed(sb, cuda_device, shape, dtype):
    q, k, v, dout, _ = H.make_inputs(shape, dtype, seed=41, std=0.5)
    got = H.run_fused(sb, q, k, v, dout, cuda_device)
    H.assert_fused_parity(got, H.oracle_fused(q, k, v, dout), dtype, "fused fixed")


@pytest.mark.parametrize("backend", ["aot_eager", "inductor"])
def test_torch_compile_fullgraph(sb, cuda_device, backend):
    """torch.compile(fullgraph=True) traces the public functions as one functional operator each (fake implementation
    and autograd formula registered), and the compiled step returns exactly what eager mode returns."""
    lengths = [300, 724]
    q, k, v, do, drem = (t.to(cuda_device) for t in H.make_inputs((4, 1024, 128), torch.bfloat16, seed=7, std=0.5))
    cu = cu_of(lengths, True).to(cuda_device)
    q4, k4, v4 = (t.reshape(2, 2, 1024, 128) for t in (q, k, v))

    def step(q, k, v, q4, k4, v4):
        o, rem = sb.sb_attn_varlen(q, k, v, cu, 724)
        out = sb.sb_attn_varlen_fused(q, k, v, cu, 724)
        o4, rem4 = sb.sb_attn(q4, k4, v4)
        return o, rem, out, o4, rem4

    def run(fn):
        ins = [t.clone().requires_grad_(True) for t in (q, k, v, q4, k4, v4)]
        outs = fn(*ins)
        ups = (do, drem, do, do.reshape(2, 2, 1024, 128), drem.reshape(2, 2, 1024))
        return outs, torch.autograd.grad(outs, ins, ups)

    torch._dynamo.reset()
    want_o, want_g = run(step)
    got_o, got_g = run(torch.compile(step, backend=backend, fullgraph=True))
    for a, b in zip(got_o + got_g, want_o + want_g):
        assert torch.equal(a, b)


def test_functional_operator_opcheck(sb, cuda_device):
    """torch.library.opcheck: schema, fake implementation, autograd registration and AOT dispatch of the operator
    that torch.compile sees."""
    q, k, v, _, _ = (t.to(cuda_device) for t in H.make_inputs((2, 384, 64), torch.bfloat16, seed=9, std=0.5))
    cu = cu_of([100, 284]).to(cuda_device)
    args = (q.requires_grad_(), k.requires_grad_(), v.requires_grad_(), cu, 284, 0.125, False, False, False)
    torch.library.opcheck(torch.ops.stickbreaking_attention_b200.fwd.default, args)
    args4 = tuple(t.detach().reshape(1, 2, 384, 64).requires_grad_() for t in (q, k, v)) + (None, 0, 0.125, True, False, True)
    torch.library.opcheck(torch.ops.stickbreaking_attention_b200.fwd.default, args4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_varlen_forms_agree(sb, cuda_device, dtype):
    """zero_start / int32 / missing max_seqlens / empty sequences are the same computation."""
    lengths = [40, 0, 200, 17]
    ins = H.make_inputs((2, sum(lengths), 64), dtype, seed=3)
    base = H.run_varlen(sb, *ins, cu_of(lengths), cuda_device, max_seqlens=200)
    H.assert_parity(base, H.oracle_varlen(*ins, cu_of([40, 200, 17])), dtype, "forms")
    for kwargs, cu in [(dict(zero_start=True), cu_of(lengths, True)),
                       (dict(zero_start=True, max_seqlens=256), cu_of(lengths, True, torch.int32)),
                       (dict(max_seqlens=None), cu_of(lengths, dtype=torch.int32))]:
        other = H.run_varlen(sb, *ins, cu, cuda_device, **kwargs)
        for a, b in zip(base, other):
            assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_tokens_after_last_sequence_are_zero(sb, cuda_device, dtype):
    lengths = [70, 50]
    ins = H.make_inputs((2, 150, 64), dtype, seed=4)
    got = H.run_varlen(sb, *ins, cu_of(lengths), cuda_device)
    want = H.oracle_varlen(*[t[:, :120] for t in ins], cu_of(lengths))
    H.assert_parity([t[:, :120] for t in got], want, dtype, "tail")
    for t in got:
        assert torch.all(t[:, 120:] == 0)


@pytest.mark.parametrize("ac", [False, True])
@pytest.mark.parametrize("shape", [(2, 3, 256, 64), (1, 7, 500, 50), (2, 2, 512, 32), (1, 2, 300, 16),
                                   (1, 2, 1024, 128), (4, 1, 130, 128)])
def test_fixed_reference_grid_bf16(sb, cuda_device, shape, ac):
    """Shapes drawn from the reference's own test grid (tests/test_attn.py:37-43) with its input
    recipe, checked the way it checks (o + rem*v and its gradients, max-abs < 0.05) and to this
    build's tighter tolerances."""
    dtype = torch.bfloat16
    q, k, v, do, _ = H.make_inputs(shape, dtype, seed=1337, recipe="reference")
    drem = (do.float() * v.float()).sum(-1).to(dtype)         # d(o + rem*v)/d rem
    got = H.run_fixed(sb, q, k, v, do, drem, cuda_device, attend_current=ac)
    want = H.oracle_fixed(q, k, v, do, drem, attend_current=ac)
    H.assert_parity(got, want, dtype, f"fixed{shape}")
    folded = got[0].float() + got[1].float()[..., None] * v.float()
    folded_ref = want[0] + want[1][..., None] * v.float()
    assert H.max_abs(folded, folded_ref) < 0.05
    for a, b in zip(got[2:4], want[2:4]):
        assert H.max_abs(a, b) < 0.05


@pytest.mark.parametrize("dtype", DTYPES)
def test_fixed_matches_varlen_layout(sb, cuda_device, dtype):
    """(B,H,T,d) through sb_attn == the same sequences packed through sb_attn_varlen, bitwise."""
    B, Hh, T, d = 3, 2, 192, 128
    q, k, v, do, drem = H.make_inputs((B, Hh, T, d), dtype, seed=9)
    fixed = H.run_fixed(sb, q, k, v, do, drem, cuda_device)
    pack = lambda t: t.transpose(0, 1).reshape(Hh, B * T, *t.shape[3:])
    packed = H.run_varlen(sb, *(pack(t) for t in (q, k, v, do, drem)), cu_of([T] * B), cuda_device)
    for a, b in zip(fixed, packed):
        assert torch.equal(pack(a), b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_strided_views_and_scale(sb, cuda_device, dtype):
    """(T,H,d) storage viewed as (H,T,d), as the reference benchmarks pass it
    (benchmarks/varlen.py:43-45), and a non-default inv_temp."""
    lengths = [100, 156]
    T, Hh, d = 256, 3, 64
    gen = torch.Generator().manual_seed(5)
    q, k, v, do = (torch.randn(T, Hh, d, generator=gen).to(dtype).permute(1, 0, 2) for _ in range(4))
    drem = torch.randn(Hh, T, generator=gen).to(dtype)
    got = H.run_varlen(sb, q, k, v, do, drem, cu_of(lengths), cuda_device, inv_temp=0.2)
    want = H.oracle_varlen(q, k, v, do, drem, cu_of(lengths), inv_temp=0.2)
    H.assert_parity(got, want, dtype, "strided")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_backward_is_bitwise_deterministic(sb, cuda_device, dtype):
    lengths = [700, 324]
    ins = H.make_inputs((4, 1024, 128), dtype, seed=6)
    a = H.run_varlen(sb, *ins, cu_of(lengths), cuda_device)
    b = H.run_varlen(sb, *ins, cu_of(lengths), cuda_device)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_long_sequence_bf16(sb, cuda_device):
    """One 4096-token sequence, d=128 (the reference's varlen test shape, tests/test_varlen.py:68-74)."""
    dtype = torch.bfloat16
    q, k, v, do, _ = H.make_inputs((3, 4096, 128), dtype, seed=1337, recipe="reference")
    drem = (do.float() * v.float()).sum(-1).to(dtype)
    cu = cu_of([4096])
    got = H.run_varlen(sb, q, k, v, do, drem, cu, cuda_device, max_seqlens=4096)
    want = H.oracle_varlen(q, k, v, do, drem, cu)
    H.assert_parity(got, want, dtype, "L4096")


def test_tensor_core_path_is_taken(sb, cuda_device):
    """bf16/fp16 with head_dim 64 or 128 must run the tcgen05 kernels, fp32 the CUDA-core ones."""
    for d in (64, 128):
        for dtype in (torch.bfloat16, torch.float16):
            assert sb.kernel_path(torch.empty(2, 256, d, dtype=dtype, device=cuda_device)) == 1
    assert sb.kernel_path(torch.empty(2, 256, 64, dtype=torch.float32, device=cuda_device)) == 0


@pytest.mark.parametrize("d", [64, 128])
def test_tensor_core_and_cuda_core_paths_agree(sb, cuda_device, d):
    dtype = torch.bfloat16
    lengths = [257, 640, 127]
    ins = H.make_inputs((2, sum(lengths), d), dtype, seed=8)
    fast = H.run_varlen(sb, *ins, cu_of(lengths), cuda_device)
    with sb.force_simt():
        slow = H.run_varlen(sb, *ins, cu_of(lengths), cuda_device)
    for name, a, b in zip(("o", "rem"), fast, slow):
        assert H.max_abs(a, b) <= 2e-2, name
    for name, a, b in zip(("dq", "dk", "dv"), fast[2:], slow[2:]):
        assert H.rel_l2(a, b) <= 5e-2, name


@pytest.mark.parametrize("ac", [False, True])
@pytest.mark.parametrize("dtype,d", [(torch.bfloat16, 64), (torch.float16, 32), (torch.bfloat16, 40)])
def test_both_forward_kernels_for_small_heads(sb, cuda_device, dtype, d, ac):
    """Head sizes up to 64 run the two-tiles-per-block forward kernel while max_seqlens <= 1024 and the 256-row kernel
    above: the same batch through both (the bound is the caller's, so a larger one is legal) against the oracle, and
    against each other -- both do the same arithmetic in the same order, so the outputs are equal bit for bit."""
    lengths = [1, 33, 96, 97, 128, 129, 255, 256, 257, 383, 500, 1000, 1024, 31, 640]
    ins = H.make_inputs((3, sum(lengths), d), dtype, seed=41 + d, std=1.0)
    cu = cu_of(lengths)
    short = H.run_varlen(sb, *ins, cu, cuda_device, attend_current=ac, max_seqlens=max(lengths))
    long_ = H.run_varlen(sb, *ins, cu, cuda_device, attend_current=ac, max_seqlens=4096)
    want = H.oracle_varlen(*ins, cu, attend_current=ac)
    H.assert_parity(short, want, dtype, "two tiles per block")
    H.assert_parity(long_, want, dtype, "256-row items")
    assert torch.equal(short[0], long_[0]) and torch.equal(short[1], long_[1])


@pytest.mark.parametrize("mode", ["stored", "recompute"])
@pytest.mark.parametrize("d,dtype", [(128, torch.bfloat16), (64, torch.bfloat16), (96, torch.float16)])
def test_skipping_exact_zeros_changes_no_bit(sb, cuda_device, d, dtype, mode):
    """With N(0, 1) inputs the product of (1 - beta) underflows to exactly 0 about a hundred keys before the query; the
    kernels then skip the arithmetic whose results are exact zeros.  Forced to do it all the same
    (SB_FLAG_DENSE_ROW_PASS), they must return the same bits: o, rem and all three gradients."""
    import contextlib
    lengths = [1500, 700, 300, 2100]
    ins = H.make_inputs((3, sum(lengths), d), dtype, seed=23 + d, std=1.0)
    cu = cu_of(lengths)
    small = sb.small_backward_workspace() if mode == "recompute" else contextlib.nullcontext()
    with small:
        fast = H.run_varlen(sb, *ins, cu, cuda_device, max_seqlens=max(lengths))
        with sb.dense_row_pass():
            dense = H.run_varlen(sb, *ins, cu, cuda_device, max_seqlens=max(lengths))
    for name, a, b in zip(("o", "rem", "dq", "dk", "dv"), fast, dense):
        assert torch.equal(a, b), name
    H.assert_parity(fast, H.oracle_varlen(*ins, cu), dtype, "zeros skipped")


# ---- error behaviour: failures are made on the host, never by faulting the device -----------------------

def test_bad_cu_seqlens_is_reported_not_executed(sb, cuda_device):
    q = torch.randn(2, 64, 64, device=cuda_device)
    sb.check_status(cuda_device)
    for cu, kwargs in [(torch.tensor([40, 30]), dict(zero_start=False)),          # decreasing
                       (torch.tensor([40, 100]), dict(zero_start=False)),         # beyond the tokens
                       (torch.tensor([5, 40, 64]), dict(zero_start=True)),        # leading element not 0
                       (torch.tensor([40, 64]), dict(zero_start=False, max_seqlens=30))]:
        qd = q.clone().requires_grad_(True)
        o, rem = sb.sb_attn_varlen(qd, q, q, cu.to(cuda_device), **kwargs)
        dq, = torch.autograd.grad((o, rem), (qd,), (torch.ones_like(o), torch.ones_like(rem)))
        with pytest.raises(sb._cabi.SbError):
            sb.check_status(cuda_device)
        # nothing was computed, and nobody can mistake the outputs for results: every row is NaN
        for t in (o, rem, dq):
            assert torch.isnan(t).all()
    sb.check_status(cuda_device)   # cleared


def test_argument_errors(sb, cuda_device):
    q = torch.randn(2, 64, 64, device=cuda_device)
    with pytest.raises(ValueError):
        sb.sb_attn_varlen(q.cpu(), q.cpu(), q.cpu(), torch.tensor([64]))
    with pytest.raises(ValueError):
        sb.sb_attn_varlen(q, q[:, :32], q, torch.tensor([64], device=cuda_device), zero_start=False)
    with pytest.raises(ValueError):
        sb.sb_attn_varlen(q.double(), q.double(), q.double(), torch.tensor([64], device=cuda_device), zero_start=False)
    with pytest.raises(ValueError):
        sb.sb_attn(q, q, q)


def test_cuda_graph_replay_matches_eager(sb, cuda_device):
    """Forward and backward enqueue only (no allocation of their own, no synchronisation, no host reads), so a step can
    be captured in a CUDA graph and replayed: the replay on new inputs must equal an eager call bit for bit."""
    dtype = torch.bfloat16
    lengths = [700, 129, 1333, 64]
    cu = cu_of(lengths).to(cuda_device)
    ins_a = [t.to(cuda_device) for t in H.make_inputs((4, sum(lengths), 128), dtype, seed=71, std=1.0)]
    ins_b = [t.to(cuda_device) for t in H.make_inputs((4, sum(lengths), 128), dtype, seed=72, std=1.0)]
    static = [t.clone() for t in ins_a]

    def step(q, k, v, do, drem):
        q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
        o, rem = sb.sb_attn_varlen(q, k, v, cu, max(lengths), zero_start=False)
        return (o, rem) + torch.autograd.grad((o, rem), (q, k, v), (do, drem))

    side = torch.cuda.Stream(device=cuda_device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):   # warm-up outside the capture: kernel attributes, tensor-map cache, allocator pools
            step(*static)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step(*static)
    for ins in (ins_b, ins_a):
        for dst, src in zip(static, ins):
            dst.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        want = step(*ins)
        for name, a, b in zip(("o", "rem", "dq", "dk", "dv"), outs, want):
            assert torch.equal(a, b), name
    sb.check_status(cuda_device)
