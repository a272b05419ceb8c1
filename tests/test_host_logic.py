"""Host-side logic that needs no GPU: argument checks, workspace sizing, kernel selection, sharding plans."""
import ctypes

import pytest
import torch

from stickbreaking_attention_b200 import _cabi, shard
import stickbreaking_attention_b200 as sb


def params(dtype=1, batch=1, heads=4, d=128, tokens=4096, num_seq=2, max_seqlen=0, flags=0, stride_t=None):
    p = _cabi.SbParams()
    p.struct_bytes = ctypes.sizeof(_cabi.SbParams)
    p.dtype, p.batch, p.heads, p.head_dim, p.tokens = dtype, batch, heads, d, tokens
    p.num_seq, p.max_seqlen, p.flags = num_seq, max_seqlen, flags
    p.cu_seqlens = 256 if num_seq else None
    st = d if stride_t is None else stride_t
    for name in ("q", "k", "v"):
        setattr(p, name, _cabi.SbTensor(4096, heads * tokens * st, tokens * st, st))
    return p


def test_cpu_tensors_are_rejected_not_computed():
    q = torch.zeros(2, 8, 16)
    with pytest.raises(ValueError, match="CUDA"):
        sb.sb_attn_varlen(q, q, q, torch.tensor([8]), zero_start=False)
    with pytest.raises(ValueError, match="CUDA"):
        sb.sb_attn(q[None], q[None], q[None])


def test_kernel_selection():
    lib = _cabi.load()
    assert lib.sb_kernel_path(params(dtype=0)) == _cabi.SB_PATH_SIMT            # fp32 -> CUDA cores
    assert lib.sb_kernel_path(params(dtype=1, d=50)) == _cabi.SB_PATH_SIMT      # irregular head_dim
    assert lib.sb_kernel_path(params(dtype=1, flags=_cabi.SB_FLAG_FORCE_SIMT)) == _cabi.SB_PATH_SIMT
    for d in (64, 128):
        for dtype in (1, 2):
            assert lib.sb_kernel_path(params(dtype=dtype, d=d)) == _cabi.SB_PATH_TCGEN05
    assert lib.sb_kernel_path(params(dtype=1, d=128, stride_t=129)) == _cabi.SB_PATH_SIMT  # rows not 16-B aligned


def test_invalid_parameters():
    lib = _cabi.load()
    for bad in (params(dtype=7), params(heads=0), params(d=0), params(d=512), params(batch=2),
                params(num_seq=0, batch=1, tokens=-1), params(max_seqlen=-3)):
        assert lib.sb_kernel_path(bad) == -1
        assert lib.sb_last_error() != b""
    p = params(num_seq=0, batch=2)   # fixed-length batch is fine
    p.cu_seqlens = None
    assert lib.sb_kernel_path(p) in (0, 1)


def test_workspace_grows_with_the_backward_boundaries():
    lib = _cabi.load()
    small = lib.sb_workspace_bytes(params(tokens=4096, max_seqlen=512), 1)
    big = lib.sb_workspace_bytes(params(tokens=4096), 1)
    assert lib.sb_workspace_bytes(params(), 0) < small < big
    # one 131072-token sequence, 16 heads: boundary scratch is capped by chunking over heads
    huge = lib.sb_workspace_bytes(params(heads=16, tokens=131072, num_seq=1, max_seqlen=131072), 1)
    assert huge < 10 * 2 ** 30


def test_head_ranges_cover_all_heads():
    for heads, world in [(16, 8), (7, 4), (3, 8), (32, 1)]:
        spans = [shard.head_range(heads, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == heads
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("by", ["tokens", "work"])
def test_contiguous_segments_partition_the_batch(by):
    gen = torch.Generator().manual_seed(0)
    lengths = torch.randint(64, 4096, (41,), generator=gen).tolist()
    for world in (1, 2, 4, 8):
        segs = shard.contiguous_segments(lengths, world, by)
        assert len(segs) == world and segs[0][0] == 0 and segs[-1][1] == len(lengths)
        assert all(a[1] == b[0] for a, b in zip(segs, segs[1:]))
        assert shard.imbalance(lengths, [range(a, b) for a, b in segs], by) < 1.6
    assert shard.contiguous_segments([5, 5], 4)[2:] == [(2, 2), (2, 2)]


def test_lpt_beats_contiguous_on_skewed_lengths():
    lengths = [16384, 64, 64, 4000, 3000, 128, 8000, 500, 700, 900, 64, 2000]
    parts = shard.lpt_assignment(lengths, 4)
    assert sorted(i for p in parts for i in p) == list(range(len(lengths)))
    segs = shard.contiguous_segments(lengths, 4, "work")
    assert shard.imbalance(lengths, parts) <= shard.imbalance(lengths, [range(a, b) for a, b in segs])


def test_slice_packed_round_trip():
    lengths = [3, 5, 2, 7]
    x = torch.arange(2 * 17 * 4).reshape(2, 17, 4)
    (sl,), lens, idx = shard.slice_packed([x], lengths, [1, 2])
    assert lens == [5, 2] and torch.equal(sl, x[:, 3:10]) and idx.tolist() == list(range(3, 10))
    (sl,), lens, idx = shard.slice_packed([x], lengths, [0, 3])
    assert lens == [3, 7] and torch.equal(sl, torch.cat([x[:, :3], x[:, 10:]], 1))
    (sl,), lens, idx = shard.slice_packed([x], lengths, [])
    assert sl.shape[1] == 0 and lens == []


def test_dropin_alias():
    import sys
    sb.install_as_dropin("stickbreaking_attention_alias_for_test")
    from stickbreaking_attention_alias_for_test.sb_varlen import sb_attn_varlen
    from stickbreaking_attention_alias_for_test.sb_attn import sb_attn
    assert sb_attn_varlen is sb.sb_attn_varlen and sb_attn is sb.sb_attn
    for key in [k for k in sys.modules if k.startswith("stickbreaking_attention_alias_for_test")]:
        del sys.modules[key]


def test_benchmark_sweep_host_side():
    """Rotary tables of the FlashAttention comparator and the no-device refusal of the sweep."""
    import pytest
    from stickbreaking_attention_b200 import benchmarks
    cos, sin = benchmarks._rope_tables(torch.arange(5), 8, torch.float32)
    assert cos.shape == (5, 8) and torch.allclose(cos[0], torch.ones(8)) and torch.allclose(sin[0], torch.zeros(8))
    x = torch.randn(5, 8)
    rot = x * cos + benchmarks._rotate_half(x) * sin            # a rotation: norms of the (i, i+4) pairs are kept
    assert torch.allclose(rot[:, :4] ** 2 + rot[:, 4:] ** 2, x[:, :4] ** 2 + x[:, 4:] ** 2, atol=1e-5)
    if not torch.cuda.is_available():
        with pytest.raises(SystemExit):
            benchmarks.main(["--op", "attn", "--lengths", "256"])


def test_functional_operator_traces_without_a_device():
    """What torch.compile relies on: the functional operator has a shape-only implementation, so a trace with fake
    tensors records one call of it and the right output shapes, dtypes and strides without running any kernel."""
    from torch.fx.experimental.proxy_tensor import make_fx
    from stickbreaking_attention_b200 import ops
    q = torch.randn(40, 3, 16).permute(1, 0, 2)          # (heads, tokens, d) view of token-major storage
    cu = torch.tensor([0, 15, 40])

    def f(q, k, v, cu):
        return ops.functional_fwd(q, k, v, cu, None, 0.25, leading_zero=True)

    gm = make_fx(f, tracing_mode="fake")(q, q, q, cu)
    calls = [n for n in gm.graph.nodes if n.op == "call_function" and "stickbreaking_attention_b200.fwd" in str(n.target)]
    assert len(calls) == 1
    o, rem, log_rem = (n.meta["val"] for n in gm.graph.find_nodes(op="output")[0].args[0])
    assert o.shape == q.shape and o.stride() == q.stride() and o.dtype == q.dtype
    assert rem.shape == q.shape[:-1] and log_rem.shape == q.shape[:-1] and log_rem.dtype == torch.float64


def test_switches_are_per_thread_and_travel_as_flags():
    """The context managers set C-ABI flag bits for the calling thread only; autograd hands them to its own thread
    through the saved context, so another thread must not see them."""
    import threading
    from stickbreaking_attention_b200 import _cabi, ops
    import stickbreaking_attention_b200 as sb
    assert ops.switch_flags() == 0
    seen = {}
    with sb.dense_row_pass(), sb.small_backward_workspace():
        assert ops.switch_flags() == _cabi.SB_FLAG_DENSE_ROW_PASS | _cabi.SB_FLAG_BWD_RECOMPUTE
        t = threading.Thread(target=lambda: seen.setdefault("other", ops.switch_flags()))
        t.start()
        t.join()
        with sb.force_simt():
            assert ops.switch_flags() & _cabi.SB_FLAG_FORCE_SIMT
        assert not ops.switch_flags() & _cabi.SB_FLAG_FORCE_SIMT
    assert seen["other"] == 0 and ops.switch_flags() == 0
