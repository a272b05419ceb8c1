"""Length sweep of the two operators against FlashAttention-2 (+ rotary embedding on its side).

Same experiment as the reference's `benchmarks/varlen.py:75-124` and `benchmarks/attn.py:43-91`: batch 4, 12 heads,
head_dim 128, bf16, lengths 4096..16384, forward + backward, inputs allocated token-major ((T, H, d) or (B, T, H, d))
and handed to the operators as permuted views, the FlashAttention side paying for rotary position embedding of q and
k because stick-breaking attention needs none.  Timing is by CUDA events (median of `--rep` runs after `--warmup`).

    python -m stickbreaking_attention_b200.benchmarks --op varlen
    python -m stickbreaking_attention_b200.benchmarks --op attn --fwd-only
    python -m stickbreaking_attention_b200.benchmarks --op fused --batch 8 --heads 16 --lengths 2048

Rows printed: length, ms of this package, ms of FlashAttention-2 (or why it is unavailable), ms of the reference's
Triton operator when a `stickbreaking_attention` package that is not this one can be imported and compiles here.
"""
import argparse
import importlib
import json
import math
import statistics
import sys

import torch


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def _rope_tables(positions, dim, dtype, base=10000.0):
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, device=positions.device, dtype=torch.float32) / dim))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def _time_ms(fn, warmup, rep):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(rep):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)


def _with_backward(fn, inputs, do, bwd):
    if not bwd:
        return fn

    def step():
        o = fn()
        torch.autograd.grad(o, inputs=inputs, grad_outputs=do)
    return step


def _reference_ops():
    """The reference's own Triton operators, if a package of that name other than this one is importable."""
    try:
        mod = importlib.import_module("stickbreaking_attention")
        if "stickbreaking_attention_b200" in (getattr(mod, "__file__", "") or ""):
            return None, "not installed"
        return mod, None
    except Exception as e:  # noqa: BLE001 - reported, not hidden
        return None, f"{type(e).__name__}: {e}".splitlines()[0][:120]


def _try(label, make, warmup, rep):
    try:
        return round(_time_ms(make(), warmup, rep), 3)
    except Exception as e:  # noqa: BLE001 - a comparator that cannot run is reported as such
        torch.cuda.synchronize()
        return f"unavailable ({type(e).__name__}: {str(e).splitlines()[0][:100]})" if str(e) else f"unavailable ({type(e).__name__})"


def bench_varlen(length, batch, heads, dim, dtype, bwd, warmup, rep):
    from . import sb_attn_varlen
    dev = torch.device("cuda:0")
    torch.manual_seed(1337)
    total = batch * length
    lengths = torch.full((batch,), length, device=dev, dtype=torch.int32)
    q, k, v = (torch.randn(total, heads, dim, device=dev, dtype=dtype).requires_grad_() for _ in range(3))
    do = torch.randn(heads, total, dim, device=dev, dtype=dtype)
    ends = torch.cumsum(lengths, 0)
    scale = 1.0 / math.sqrt(dim)

    def ours():
        def f():
            o, _ = sb_attn_varlen(q.permute(1, 0, 2), k.permute(1, 0, 2), v.permute(1, 0, 2), ends, length,
                                  inv_temp=scale, zero_start=False)
            return o
        return _with_backward(f, (q, k, v), do, bwd)

    def flash():
        from flash_attn import flash_attn_varlen_func
        pos = torch.arange(length, device=dev).repeat(batch)
        cu = torch.nn.functional.pad(ends, (1, 0)).to(torch.int32)

        def f():
            cos, sin = _rope_tables(pos, dim, dtype)
            cos, sin = cos[:, None, :], sin[:, None, :]
            qr = q * cos + _rotate_half(q) * sin
            kr = k * cos + _rotate_half(k) * sin
            o = flash_attn_varlen_func(qr, kr, v, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=length,
                                       max_seqlen_k=length, causal=True)
            return o.permute(1, 0, 2)
        return _with_backward(f, (q, k, v), do, bwd)

    def reference():
        mod, why = _reference_ops()
        if mod is None:
            raise RuntimeError(why)
        ref_op = importlib.import_module("stickbreaking_attention.sb_varlen").sb_attn_varlen

        def f():
            o, _ = ref_op(q.permute(1, 0, 2), k.permute(1, 0, 2), v.permute(1, 0, 2), cu_seqlens=ends,
                          max_seqlens=length, inv_temp=scale, zero_start=False)
            return o
        return _with_backward(f, (q, k, v), do, bwd)

    return {"length": length, "sb_b200_ms": _try("ours", ours, warmup, rep),
            "flash_attn2_rope_ms": _try("flash", flash, warmup, rep),
            "reference_triton_ms": _try("reference", reference, warmup, max(rep // 4, 1))}


def bench_fused(length, batch, heads, dim, dtype, bwd, warmup, rep):
    """`o + rem[..., None] * v` (the step every caller of the reference takes next, `tests/test_varlen.py:101`):
    the two-output operator followed by torch arithmetic, against the fused operator."""
    from . import sb_attn_varlen, sb_attn_varlen_fused
    dev = torch.device("cuda:0")
    torch.manual_seed(1337)
    total = batch * length
    q, k, v = (torch.randn(heads, total, dim, device=dev, dtype=dtype).requires_grad_() for _ in range(3))
    do = torch.randn(heads, total, dim, device=dev, dtype=dtype)
    ends = torch.arange(1, batch + 1, device=dev, dtype=torch.int32) * length

    def two_step():
        def f():
            o, rem = sb_attn_varlen(q, k, v, ends, length, zero_start=False)
            return o + rem[..., None] * v
        return _with_backward(f, (q, k, v), do, bwd)

    def fused():
        return _with_backward(lambda: sb_attn_varlen_fused(q, k, v, ends, length, zero_start=False), (q, k, v), do, bwd)

    return {"length": length, "sb_b200_ms": _try("fused", fused, warmup, rep),
            "two_step_ms": _try("two_step", two_step, warmup, rep)}


def bench_attn(length, batch, heads, dim, dtype, bwd, warmup, rep):
    from . import sb_attn
    dev = torch.device("cuda:0")
    torch.manual_seed(1337)
    q, k, v = (torch.randn(batch, length, heads, dim, device=dev, dtype=dtype).requires_grad_() for _ in range(3))
    do = torch.randn(batch, length, heads, dim, device=dev, dtype=dtype)
    scale = 1.0 / math.sqrt(dim)

    def ours():
        def f():
            o, _ = sb_attn(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), inv_temp=scale)
            return o.permute(0, 2, 1, 3)
        return _with_backward(f, (q, k, v), do, bwd)

    def flash():
        from flash_attn import flash_attn_func
        pos = torch.arange(length, device=dev)

        def f():
            cos, sin = _rope_tables(pos, dim, dtype)
            cos, sin = cos[None, :, None, :], sin[None, :, None, :]
            qr = q * cos + _rotate_half(q) * sin
            kr = k * cos + _rotate_half(k) * sin
            return flash_attn_func(qr, kr, v, causal=True)
        return _with_backward(f, (q, k, v), do, bwd)

    def reference():
        mod, why = _reference_ops()
        if mod is None:
            raise RuntimeError(why)
        ref_op = importlib.import_module("stickbreaking_attention.sb_attn").sb_attn

        def f():
            o, _ = ref_op(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), inv_temp=scale)
            return o.permute(0, 2, 1, 3)
        return _with_backward(f, (q, k, v), do, bwd)

    return {"length": length, "sb_b200_ms": _try("ours", ours, warmup, rep),
            "flash_attn2_rope_ms": _try("flash", flash, warmup, rep),
            "reference_triton_ms": _try("reference", reference, warmup, max(rep // 4, 1))}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--op", choices=("varlen", "attn", "fused"), default="varlen")
    ap.add_argument("--lengths", type=int, nargs="+", default=[4096, 8192, 12288, 16384])
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--fwd-only", action="store_true")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rep", type=int, default=20)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        sys.exit("benchmarks need a CUDA device")
    fn = {"varlen": bench_varlen, "attn": bench_attn, "fused": bench_fused}[a.op]
    flop_c = 2 if a.fwd_only else 7
    for length in a.lengths:
        row = fn(length, a.batch, a.heads, a.head_dim, torch.bfloat16, not a.fwd_only, a.warmup, a.rep)
        if isinstance(row["sb_b200_ms"], float):
            flops = flop_c * a.head_dim * a.heads * a.batch * float(length) ** 2
            row["sb_b200_tflops"] = round(flops / row["sb_b200_ms"] / 1e9, 1)
        row.update(op=a.op, batch=a.batch, heads=a.heads, head_dim=a.head_dim, bwd=not a.fwd_only)
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
