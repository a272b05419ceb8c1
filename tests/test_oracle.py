"""The CPU oracle against the reference's own outputs (golden vectors) and against itself."""
import itertools

import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import sb_oracle as O

OUT_KEYS = ("o", "rem", "dq", "dk", "dv")


def cu(lengths):
    return torch.tensor(lengths).cumsum(0)


@pytest.mark.parametrize("ac", [0, 1])
def test_dense_matches_reference_tiny_varlen(ac):
    g = load_golden(f"tiny_varlen_ac{ac}")
    got = O.varlen_dense_grads(g["q"], g["k"], g["v"], cu(g["lengths"]), g["do"], g["drem"],
                               attend_current=bool(ac))
    for key, val in zip(OUT_KEYS, got):
        assert torch.allclose(val, g[key], rtol=1e-5, atol=2e-6), key


@pytest.mark.parametrize("ac", [0, 1])
def test_dense_matches_reference_tiny_fixed(ac):
    g = load_golden(f"tiny_fixed_ac{ac}")
    got = O.fixed_dense_grads(g["q"], g["k"], g["v"], g["do"], g["drem"], attend_current=bool(ac))
    for key, val in zip(OUT_KEYS, got):
        assert torch.allclose(val, g[key], rtol=1e-5, atol=2e-6), key


@pytest.mark.parametrize("ac", [0, 1])
def test_dense_matches_reference_recipe(ac):
    g = load_golden(f"recipe_varlen_ac{ac}")
    q, k, v, do, drem = (g[n].float() for n in ("q", "k", "v", "do", "drem"))
    got = O.varlen_dense_grads(q, k, v, cu(g["lengths"]), do, drem, attend_current=bool(ac))
    for key, val in zip(OUT_KEYS, got):
        assert torch.allclose(val, g[key], rtol=1e-5, atol=2e-6), key


def c1_inputs():
    torch.manual_seed(0)
    lengths = [128, 256, 64, 512]
    shape = (4, sum(lengths), 64)
    q, k, v, do = (torch.randn(shape) for _ in range(4))
    drem = torch.randn(shape[:2])
    return lengths, q, k, v, do, drem


def test_c1_config_matches_reference():
    """BASELINE config 1 (H=4, d=64, lengths [128,256,64,512], seed 0): inputs regenerate to the
    stored checksums and the oracle reproduces the stored rows of the reference's outputs."""
    g = load_golden("c1")
    lengths, q, k, v, do, drem = c1_inputs()
    assert lengths == g["lengths"]
    sums = torch.tensor([float(t.double().sum()) for t in (q, k, v, do, drem)], dtype=torch.float64)
    assert torch.allclose(sums, g["input_sums"], rtol=0, atol=1e-9)
    stride = int(g["row_stride"])
    got = O.varlen_dense_grads(q, k, v, cu(lengths), do, drem)
    for key, val in zip(OUT_KEYS, got):
        assert torch.allclose(val[:, ::stride], g[key], rtol=1e-5, atol=5e-6), key


@pytest.mark.parametrize("ac,block", list(itertools.product([False, True], [7, 64, 1024])))
def test_rowblocked_matches_dense(ac, block):
    gen = torch.Generator().manual_seed(5)
    lengths = [1, 130, 64, 257, 3]
    shape = (3, sum(lengths), 32)
    q, k, v, do = (torch.randn(shape, generator=gen) for _ in range(4))
    drem = torch.randn(shape[:2], generator=gen)
    want = O.varlen_dense_grads(q.double(), k.double(), v.double(), cu(lengths), do.double(),
                                drem.double(), attend_current=ac)
    got = O.varlen_rowblocked_grads(q, k, v, cu(lengths), do, drem, attend_current=ac, block=block,
                                    dtype=torch.float64)
    for key, a, b in zip(OUT_KEYS, got, want):
        assert torch.allclose(a, b, rtol=1e-6, atol=1e-6), key
    fo, fr = O.varlen_rowblocked(q, k, v, cu(lengths), attend_current=ac, block=block)
    assert torch.allclose(fo.double(), want[0], atol=1e-5)
    assert torch.allclose(fr.double(), want[1], atol=1e-5)


def test_zero_start_and_scale():
    gen = torch.Generator().manual_seed(6)
    lengths = [9, 20]
    q, k, v = (torch.randn(2, 29, 8, generator=gen) for _ in range(3))
    a = O.varlen_dense(q, k, v, torch.tensor([9, 29]))
    b = O.varlen_dense(q, k, v, torch.tensor([0, 9, 29]), zero_start=True)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    # a logit scale is the same as scaling q
    c = O.varlen_dense(q, k, v, torch.tensor([9, 29]), scale=0.5)
    d = O.varlen_dense(q * (0.5 * 8 ** 0.5), k, v, torch.tensor([9, 29]))
    assert torch.allclose(c[0], d[0], atol=1e-6) and torch.allclose(c[1], d[1], atol=1e-6)


def test_structural_known_answers():
    """First token of every sequence sees nothing when it may not attend to itself: o = 0,
    rem = 1; rem is the product of (1 - beta) and stays in [0, 1] up to rounding."""
    gen = torch.Generator().manual_seed(7)
    lengths = [4, 31, 2]
    q, k, v = (torch.randn(2, 37, 16, generator=gen) for _ in range(3))
    o, rem = O.varlen_dense(q, k, v, cu(lengths))
    for start in (0, 4, 35):
        assert torch.all(o[:, start] == 0) and torch.all(rem[:, start] == 1)
    assert rem.min() > -1e-6 and rem.max() <= 1
    z = torch.einsum("hid,hjd->hij", q[:, :4], k[:, :4]) / 4.0
    prod = torch.stack([torch.prod(1 - torch.sigmoid(z[:, i, :i]), -1) for i in range(4)], 1)
    assert torch.allclose(rem[:, :4], prod, atol=1e-6)


def test_flop_convention():
    assert O.flops([128, 256, 64, 512], 4, 64, "fwd") == pytest.approx(0.178e9, rel=2e-3)
    assert O.flops([2048] * 8, 16, 128) == pytest.approx(481.0e9, rel=1e-3)
