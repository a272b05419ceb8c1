"""Shared helpers of the GPU parity tests: run the CUDA path and the CPU oracle on the same inputs."""
import math

import torch

from oracle import sb_oracle as O

# Tolerances of the path (stated by the build target): against the oracle run in fp32 on the same
# seeded inputs, bf16/fp16 I/O within 2e-2 max-abs on o and rem and 5e-2 relative L2 on dq/dk/dv;
# fp32 I/O within 1e-4 on everything.
TOL = {
    torch.float32: dict(out=1e-4, grad_rel=1e-4),
    torch.bfloat16: dict(out=2e-2, grad_rel=5e-2),
    torch.float16: dict(out=2e-2, grad_rel=5e-2),
}


def make_inputs(shape, dtype, seed, recipe="normal", std=1.0):
    """'normal': N(0, std^2); 'reference': the reference tests' shifted recipe (tests/test_varlen.py:83-89)."""
    gen = torch.Generator().manual_seed(seed)
    if recipe == "reference":
        v = 0.25 * torch.randn(shape, generator=gen)
        q = 0.25 * (torch.randn(shape, generator=gen) + 1)
        k = 0.25 * (torch.randn(shape, generator=gen) - 1)
    else:
        q, k, v = (std * torch.randn(shape, generator=gen) for _ in range(3))
    do = torch.randn(shape, generator=gen)
    drem = torch.randn(shape[:-1], generator=gen)
    return tuple(t.to(dtype) for t in (q, k, v, do, drem))


def rel_l2(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-20))


def max_abs(a, b):
    return float((a.double().cpu() - b.double().cpu()).abs().max()) if a.numel() else 0.0


def run_varlen(sb, q, k, v, do, drem, cu, device, *, zero_start=False, max_seqlens=None, inv_temp=None,
               attend_current=False):
    qd, kd, vd = (t.to(device).requires_grad_(True) for t in (q, k, v))
    o, rem = sb.sb_attn_varlen(qd, kd, vd, cu.to(device), max_seqlens, inv_temp=inv_temp,
                               zero_start=zero_start, attend_current=attend_current)
    dq, dk, dv = torch.autograd.grad((o, rem), (qd, kd, vd), (do.to(device), drem.to(device)))
    return tuple(t.detach().cpu() for t in (o, rem, dq, dk, dv))


def run_fixed(sb, q, k, v, do, drem, device, *, inv_temp=None, attend_current=False):
    qd, kd, vd = (t.to(device).requires_grad_(True) for t in (q, k, v))
    o, rem = sb.sb_attn(qd, kd, vd, inv_temp=inv_temp, attend_current=attend_current)
    dq, dk, dv = torch.autograd.grad((o, rem), (qd, kd, vd), (do.to(device), drem.to(device)))
    return tuple(t.detach().cpu() for t in (o, rem, dq, dk, dv))


def oracle_varlen(q, k, v, do, drem, cu, *, zero_start=False, inv_temp=None, attend_current=False):
    f = lambda t: t.float()
    lengths = O.seq_bounds(cu, zero_start)
    if max(e - s for s, e in lengths) <= 2048:
        return O.varlen_dense_grads(f(q), f(k), f(v), cu, f(do), f(drem), scale=inv_temp,
                                    attend_current=attend_current, zero_start=zero_start)
    return O.varlen_rowblocked_grads(f(q), f(k), f(v), cu, f(do), f(drem), scale=inv_temp,
                                     attend_current=attend_current, zero_start=zero_start)


def oracle_fixed(q, k, v, do, drem, *, inv_temp=None, attend_current=False):
    f = lambda t: t.float()
    return O.fixed_dense_grads(f(q), f(k), f(v), f(do), f(drem), scale=inv_temp, attend_current=attend_current)


def ulp_16bit(x, dtype):
    """Spacing of `dtype` (bf16: 8 significand bits, fp16: 11) at the magnitude of each element of the fp32 tensor x."""
    bits = {torch.bfloat16: 7, torch.float16: 10}[dtype]
    e = torch.floor(torch.log2(x.abs().double().clamp_min(2.0 ** -24)))
    return torch.pow(2.0, e - bits)


def out_bound(want, dtype):
    """Elementwise bound on |got - oracle| for o and rem.  The stated tolerance is a max-abs one, but an output tensor
    stored in a 16-bit type cannot be closer to the fp32 oracle than its own spacing allows: once |o| reaches 4 a bf16
    step is 0.031.  So the bound is the stated max-abs tolerance or one unit in the last place of the oracle value in
    the output dtype, whichever is larger (for |o| < 4 in bf16, and everywhere in fp32, that is the stated tolerance)."""
    tol = torch.full_like(want, TOL[dtype]["out"], dtype=torch.float64)
    if dtype in (torch.bfloat16, torch.float16):
        tol = torch.maximum(tol, ulp_16bit(want, dtype))
    return tol


def worst_output_error(got, want, dtype):
    """(max of |got - want| / bound, the element's |got - want|, oracle value, oracle rounded to dtype, got)."""
    a, b = got.double().cpu(), want.double().cpu()
    ratio = (a - b).abs() / out_bound(want.cpu(), dtype)
    i = int(torch.argmax(ratio))
    bf, af = b.flatten()[i], a.flatten()[i]
    return float(ratio.flatten()[i]), float((af - bf).abs()), float(bf), float(bf.to(dtype).double()), float(af)


def assert_parity(got, want, dtype, what=""):
    tol = TOL[dtype]
    names = ("o", "rem", "dq", "dk", "dv")
    report = {}
    for name, a, b in zip(names, got, want):
        assert torch.isfinite(a.float()).all(), f"{what}: {name} has non-finite values"
        report[name] = (max_abs(a, b), rel_l2(a, b))
    for name, a, b in zip(names[:2], got[:2], want[:2]):
        ratio, err, ref, ref_rounded, val = worst_output_error(a, b, dtype)
        report[name + "_worst"] = dict(err=err, oracle=ref, oracle_rounded=ref_rounded, got=val)
        assert ratio <= 1.0, (f"{what}: {name} off by {err:.3e} at oracle value {ref:.6g} (rounded to the output dtype: "
                              f"{ref_rounded:.6g}, got {val:.6g}); bound max({tol['out']}, 1 ulp)")
    for name in ("dq", "dk", "dv"):
        assert report[name][1] <= tol["grad_rel"], f"{what}: {name} rel-L2 {report[name][1]:.3e} > {tol['grad_rel']}"
    return report


def oracle_fused(q, k, v, dout, cu=None, **kw):
    """Oracle for out = o + rem[..., None] * v (what the reference's callers compute, tests/test_varlen.py:101) and
    the gradients of q, k, v for an upstream gradient of `out`: d_o = d_out, d_rem = <d_out, v>, dv += rem * d_out."""
    vf, gf = v.float(), dout.float()
    drem = (gf * vf).sum(-1)
    if cu is None:
        o, rem, dq, dk, dv = oracle_fixed(q, k, v, gf, drem, **kw)
    else:
        o, rem, dq, dk, dv = oracle_varlen(q, k, v, gf, drem, cu, **kw)
    return o + rem[..., None] * vf, dq, dk, dv + rem[..., None] * gf


def run_fused(sb, q, k, v, dout, device, cu=None, **kw):
    qd, kd, vd = (t.to(device).requires_grad_(True) for t in (q, k, v))
    if cu is None:
        out = sb.sb_attn_fused(qd, kd, vd, **kw)
    else:
        out = sb.sb_attn_varlen_fused(qd, kd, vd, cu.to(device), **kw)
    dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), dout.to(device))
    return tuple(t.detach().cpu() for t in (out, dq, dk, dv))


def assert_fused_parity(got, want, dtype, what=""):
    tol = TOL[dtype]
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        assert torch.isfinite(a.float()).all(), f"{what}: {name} has non-finite values"
        if name == "out":
            assert max_abs(a, b) <= tol["out"], f"{what}: out max-abs {max_abs(a, b):.3e} > {tol['out']}"
        else:
            assert rel_l2(a, b) <= tol["grad_rel"], f"{what}: {name} rel-L2 {rel_l2(a, b):.3e} > {tol['grad_rel']}"
