#!/usr/bin/env python
"""Benchmark of the stick-breaking attention hot path: sb_attn_varlen forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c2s|c3|c4|c5|c5s]

One step = one forward + backward pass of ``sb_attn_varlen`` over one synthetic batch.  The default
workload is the configuration the headline metric is quoted on: 16 heads, head_dim 128, 8 sequences of
2048 tokens (16384 packed tokens), q/k/v ~ N(0,1) in bf16, dO ~ N(0,1).  With N > 1 (one process per
GPU under torchrun) every rank runs its own batch of that shape: the path shards by independent
(head, sequence) pairs with no collective, so scaling is "weak" and ``value`` is the sum over ranks of
the algorithmic FLOPs divided by the slowest rank's device time.

Printed by rank 0, one JSON line:
  value      TFLOP/s of the whole job, inputs resident in HBM, CUDA-event timed, max over ranks; the K-step timed
             loop is repeated (``timing.repeats``) and the median repetition is the one reported
  e2e        same metric through the public Python operator with pinned HOST buffers: the H2D copies of
             q, k, v, dO, dRem and the D2H copies of o, rem, dq, dk, dv are inside the timed region (every step
             copies all of them; the copies of neighbouring steps overlap the compute on separate streams)
  roofline   the dominant kernel against the measured dense bf16 tensor peak
  cpu_baseline  the reference's own sb_ref.stickbreaking on the host cores (from the reference installation under
             baseline/_ref when it is there, else this repository's port of it), bounded sample, rank 0, N == 1
  sharded    the long-context workload split by heads and the skewed packed workload split by sequences across the
             N ranks (strong scaling: the total work is fixed), each plan with its slowest and mean rank time, and a
             bitwise comparison of the gathered shards (NCCL, outside the timed region) with an unsharded run

FLOP convention (causal): forward 2*L^2*d per head per sequence, backward 2.5x that.

``--impl reference`` times the reference's CPU implementation of the path on the host cores instead: every
step runs the whole workload (all heads, all sequences, split per sequence as the reference's tests do).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from one ncu capture of this workload.  The figures belong
# to the kernel sources whose digest is recorded with them: after any change to the kernels they are stale, and
# `roofline.traffic` is reported as null until a new capture is entered here.
NCU_TRAFFIC = {"kernel_sources_sha256_16": "b83484319ccfd8fa",
               "bytes": {"c2": {"fwd": 492.3e6, "bwd_dq": 1466.0e6, "bwd_dkv": 1406.4e6}, "c5s": {"fwd": 2386.8e6}}}


def kernel_sources_digest():
    import hashlib
    csrc = os.path.join(ROOT, "stickbreaking_attention_b200", "csrc")
    h = hashlib.sha256()
    for name in sorted(os.listdir(csrc)):
        if name.endswith((".cu", ".cuh")):
            with open(os.path.join(csrc, name), "rb") as f:
                h.update(name.encode() + b"\0" + f.read())
    return h.hexdigest()[:16]


def ncu_traffic(workload_name, kernel):
    if NCU_TRAFFIC["kernel_sources_sha256_16"] != kernel_sources_digest():
        return None
    return NCU_TRAFFIC["bytes"].get(workload_name, {}).get(kernel)


# ---------------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------------
def workload(name: str, seed: int = 0):
    """Returns dict(heads, head_dim, lengths, std, zero_start, fwd_only, label)."""
    import numpy as np
    if name == "c2":
        return dict(heads=16, head_dim=128, lengths=[2048] * 8, std=1.0, zero_start=False, fwd_only=False,
                    label="16 heads x 8 sequences x 2048 tokens, head_dim 128, bf16, fwd+bwd")
    if name == "c2s":     # small stand-in used for profiler captures
        return dict(heads=8, head_dim=128, lengths=[2048] * 4, std=1.0, zero_start=False, fwd_only=False,
                    label="8 heads x 4 sequences x 2048 tokens, head_dim 128, bf16, fwd+bwd")
    if name == "c3":
        rng = np.random.default_rng(seed)
        lengths, total = [], 0
        while total < 65536:
            n = int(np.clip(rng.lognormal(np.log(1024.0), 1.0), 64, 16384))
            n = min(n, 65536 - total)
            lengths.append(n)
            total += n
        return dict(heads=32, head_dim=128, lengths=lengths, std=1.0, zero_start=True, fwd_only=False,
                    label="32 heads, 65536 tokens in lognormal-length sequences, head_dim 128, bf16, fwd+bwd")
    if name == "c4":
        return dict(heads=16, head_dim=128, lengths=[131072], std=0.5, zero_start=False, fwd_only=False,
                    label="16 heads x 1 sequence of 131072 tokens, head_dim 128, bf16, fwd+bwd")
    if name == "c5s":     # small stand-in of c5 used for profiler captures
        rng = np.random.default_rng(seed)
        lengths = rng.integers(128, 513, size=1024).tolist()
        return dict(heads=8, head_dim=64, lengths=lengths, std=1.0, zero_start=False, fwd_only=True,
                    label="8 heads, 1024 sequences of 128..512 tokens, head_dim 64, bf16, forward only")
    if name == "c5":
        rng = np.random.default_rng(seed)
        lengths = rng.integers(128, 513, size=4096).tolist()
        return dict(heads=32, head_dim=64, lengths=lengths, std=1.0, zero_start=False, fwd_only=True,
                    label="32 heads, 4096 sequences of 128..512 tokens, head_dim 64, bf16, forward only")
    raise SystemExit(f"unknown workload {name}")


def flops_of(w, mode):
    c = {"fwd": 2.0, "bwd": 5.0, "fwd_bwd": 7.0}[mode]
    return c * w["head_dim"] * w["heads"] * float(sum(n * n for n in w["lengths"]))


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            data = json.load(f)
        return {"bf16_tflops": float(data["bf16_tflops"]), "hbm_gbs": float(data["hbm_gbs"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"]))}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


# ---------------------------------------------------------------------------------------------------
# clock sampling (read-only NVML queries)
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                bits = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.004)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------------
# CPU arm: the reference's sb_ref.stickbreaking on the host cores
# ---------------------------------------------------------------------------------------------------
def load_reference_sb_ref():
    """The reference's own sb_ref module, loaded by file path from its installation under baseline/_ref (a pure
    torch file; nothing else of the reference is imported), or None when that installation is absent."""
    import importlib.util
    path = os.path.join(ROOT, "baseline", "_ref", "stickbreaking_attention", "sb_ref.py")
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location("_reference_sb_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def use_all_host_threads():
    try:   # torchrun pins OMP_NUM_THREADS=1; the CPU arm is meant to use every host core it may
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except Exception:
        pass
    return torch.get_num_threads()


def cpu_inputs(w, heads, seqs):
    lengths = w["lengths"][:seqs]
    gen = torch.Generator().manual_seed(0)
    shape = (heads, sum(lengths), w["head_dim"])
    q, k, v = (w["std"] * torch.randn(shape, generator=gen) for _ in range(3))
    do = torch.randn(shape, generator=gen)
    drem = torch.randn(shape[:2], generator=gen)
    return lengths, q, k, v, do, drem


def cpu_step(ref, w, lengths, q, k, v, do, drem):
    """One forward + backward of the workload slice on the CPU, fp32.  With the reference module: its dense function
    per sequence with the mask and cumulative-weight matrices its tests build (tests/test_varlen.py:10-27 of the
    reference), gradients by autograd for upstream gradients of both outputs.  Sequences too long for the dense
    L x L matrices, or no reference installation: this repository's port (row-blocked where needed)."""
    from oracle import sb_oracle as O
    cu = torch.tensor(lengths).cumsum(0)
    if ref is None or max(lengths) > 4096:
        fn = O.varlen_dense_grads if max(lengths) <= 4096 else O.varlen_rowblocked_grads
        fn(q, k, v, cu, do, drem)
        return "port"
    start = 0
    for n in lengths:
        sl = slice(start, start + n)
        qs, ks, vs = (t[None, :, sl].detach().clone().requires_grad_(True) for t in (q, k, v))
        cm = torch.ones(n, n).tril(-1)
        mask = torch.ones(n, n).triu(0).bool()
        o, rem = ref.stickbreaking(qs, ks, vs, mask, cm)
        torch.autograd.grad((o, rem), (qs, ks, vs), (do[None, :, sl], drem[None, :, sl]))
        start += n
    return "reference"


def cpu_sample(w, heads, seqs, reps):
    """Times `reps` CPU steps over `heads` heads x the first `seqs` sequences; returns
    (best seconds, TFLOP/s under the causal convention, description, kind)."""
    ref = load_reference_sb_ref()
    use_all_host_threads()
    lengths, q, k, v, do, drem = cpu_inputs(w, heads, seqs)
    best, kind = float("inf"), "port"
    for _ in range(reps):
        t0 = time.perf_counter()
        kind = cpu_step(ref, w, lengths, q, k, v, do, drem)
        best = min(best, time.perf_counter() - t0)
    fl = 7.0 * w["head_dim"] * heads * float(sum(n * n for n in lengths))
    whole = heads == w["heads"] and seqs >= len(w["lengths"])
    desc = (("the whole workload" if whole else
             f"{heads} of {w['heads']} heads x the first {len(lengths)} of {len(w['lengths'])} sequence(s)")
            + f" ({sum(lengths)} tokens), fp32, forward + autograd backward, best of {reps}")
    return best, fl / best / 1e12, desc, kind


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ref = load_reference_sb_ref()
    threads = use_all_host_threads()
    heads, seqs = w["heads"], len(w["lengths"])      # every step is the whole workload ...
    if max(w["lengths"]) > 4096:
        seqs = 1
    lengths, q, k, v, do, drem = cpu_inputs(w, heads, seqs)
    times, kind = [], "port"
    total = args.warmup + args.steps
    i = 0
    while i < total:
        t0 = time.perf_counter()
        kind = cpu_step(ref, w, lengths, q, k, v, do, drem)
        dt = time.perf_counter() - t0
        # ... unless the first step shows that W + K such steps would not end within the time allowed: then the
        # steps go on with as many heads as fit it (the per-head work is identical; the sample line says what ran)
        if i == 0 and heads > 1 and dt * total > args.reference_budget_s:
            heads = max(1, int(heads * args.reference_budget_s / (dt * total)))
            lengths, q, k, v, do, drem = cpu_inputs(w, heads, seqs)
            continue
        if i >= args.warmup:
            times.append(dt)
        i += 1
    mean = sum(times) / len(times)
    fl = 7.0 * w["head_dim"] * heads * float(sum(n * n for n in lengths))
    value = fl / mean / 1e12
    whole = heads == w["heads"] and seqs == len(w["lengths"])
    desc = (("every step is the whole workload: " if whole else "every step is a part of the workload: ")
            + f"{heads} of {w['heads']} heads x {seqs} of {len(w['lengths'])} sequence(s), {sum(lengths)} tokens, fp32, "
            f"forward + autograd backward, split per sequence")
    line = {
        "impl": "reference", "metric": "sb_attn_varlen fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["label"], "name": args.workload, "sample_per_step": desc,
                   "host_cores": os.cpu_count(), "torch_threads": threads,
                   "function": ("stickbreaking_attention/sb_ref.py:stickbreaking of the installed reference"
                                if kind == "reference" else "this repository's port of sb_ref.stickbreaking")},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
def make_batch(w, device, seed):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    T = sum(w["lengths"])
    shape = (w["heads"], T, w["head_dim"])
    host = {}
    for name in ("q", "k", "v"):
        host[name] = (w["std"] * torch.randn(shape, generator=gen)).to(torch.bfloat16).pin_memory()
    host["do"] = torch.randn(shape, generator=gen).to(torch.bfloat16).pin_memory()
    host["drem"] = torch.randn(shape[:2], generator=gen).to(torch.bfloat16).pin_memory()
    ends = torch.tensor(w["lengths"], dtype=torch.int32).cumsum(0).to(torch.int32)
    cu = torch.cat([torch.zeros(1, dtype=torch.int32), ends]) if w["zero_start"] else ends
    return host, cu.to(device)


def event_time_ms(fn, iters):
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters


def kernel_breakdown(sb, w, dev_t, cu, max_len, iters=5):
    """Average device time of each kernel group, timed alone through the C ABI with CUDA events on the
    launching stream: forward, backward dQ kernel, backward dK/dV kernel."""
    from stickbreaking_attention_b200 import _cabi, ops
    lib = _cabi.load()
    q, k, v, do, drem = (dev_t[n] for n in ("q", "k", "v", "do", "drem"))
    ends = cu[1:] if w["zero_start"] else cu
    o = torch.empty_like(q)
    rem = torch.empty(q.shape[:2], dtype=q.dtype, device=q.device)
    log_rem = torch.empty(q.shape[:2], dtype=torch.float64, device=q.device)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    status = torch.zeros(4, dtype=torch.int32, device=q.device)
    prm = _cabi.SbParams()
    ops._fill(prm, fixed=False, q=q, k=k, v=v, cu_seqlens=ends, max_seqlens=max_len,
              logit_scale=w["head_dim"] ** -0.5, attend_current=False, leading_zero=w["zero_start"])
    prm.o = _cabi.tensor_arg(o, False)
    prm.rem, prm.log_rem = rem.data_ptr(), log_rem.data_ptr()
    prm.d_o = _cabi.tensor_arg(do, False)
    prm.d_rem = drem.data_ptr()
    prm.dq, prm.dk, prm.dv = (_cabi.tensor_arg(t, False) for t in (dq, dk, dv))
    need = max(lib.sb_workspace_bytes(prm, 1), lib.sb_workspace_bytes(prm, 0))
    ws = torch.empty(need, dtype=torch.uint8, device=q.device)
    prm.workspace, prm.workspace_bytes, prm.status = ws.data_ptr(), ws.numel(), status.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    base_flags = prm.flags

    def call(fn, flags):
        prm.flags = base_flags | flags
        rc = fn(prm, stream)
        if rc != 0:
            raise RuntimeError(lib.sb_last_error().decode())

    call(lib.sb_fwd, 0)
    call(lib.sb_bwd, 0)
    torch.cuda.synchronize()
    out = {"fwd": event_time_ms(lambda: call(lib.sb_fwd, 0), iters)}
    if not w["fwd_only"]:
        out["bwd_dq"] = event_time_ms(lambda: call(lib.sb_bwd, _cabi.SB_FLAG_BWD_SKIP_DKV), iters)
        out["bwd_dkv"] = event_time_ms(lambda: call(lib.sb_bwd, _cabi.SB_FLAG_BWD_SKIP_DQ), iters)
    path = lib.sb_kernel_path(prm)
    return out, path


def run_gpu_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    distributed = world > 1
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    import stickbreaking_attention_b200 as sb

    host, cu = make_batch(w, device, seed=1234 + rank)
    dev_t = {n: t.to(device, non_blocking=True) for n, t in host.items()}
    max_len = max(w["lengths"])
    fwd_only = w["fwd_only"]
    mode = "fwd" if fwd_only else "fwd_bwd"

    def step_resident():
        q, k, v = (dev_t[n].requires_grad_(not fwd_only) for n in ("q", "k", "v"))
        o, rem = sb.sb_attn_varlen(q, k, v, cu, max_len, zero_start=w["zero_start"])
        if fwd_only:
            return o, rem
        return torch.autograd.grad((o, rem), (q, k, v), (dev_t["do"], dev_t["drem"]))

    out_host = {}
    # End to end, as a training loop would drive it: three streams and two sets of device input buffers, so that the
    # host->device copy of step i+1 and the device->host copy of step i-1 run while step i computes.  Every step still
    # copies all of its inputs from pinned host memory and all of its results back, inside the timed region.
    s_in, s_cmp, s_out = (torch.cuda.Stream(device=device) for _ in range(3))
    dev_in = [{n: torch.empty_like(t, device=device) for n, t in host.items()} for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    for ev in in_free:
        ev.record()
    e2e_state = {"i": 0}

    def step_e2e():
        b = e2e_state["i"] % 2
        e2e_state["i"] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[b])          # the step that last used this buffer set has finished with it
            for n, t in host.items():
                dev_in[b][n].copy_(t, non_blocking=True)
            in_ready[b].record(s_in)
        with torch.cuda.stream(s_cmp):
            s_cmp.wait_event(in_ready[b])
            q, k, v = (dev_in[b][n].detach().requires_grad_(not fwd_only) for n in ("q", "k", "v"))
            o, rem = sb.sb_attn_varlen(q, k, v, cu, max_len, zero_start=w["zero_start"])
            results = {"o": o, "rem": rem}
            if not fwd_only:
                dq, dk, dv = torch.autograd.grad((o, rem), (q, k, v), (dev_in[b]["do"], dev_in[b]["drem"]))
                results.update(dq=dq, dk=dk, dv=dv)
            in_free[b].record(s_cmp)
            done = torch.cuda.Event()
            done.record(s_cmp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for name, t in results.items():
                t = t.detach()
                if name not in out_host:
                    out_host[name] = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                t.record_stream(s_out)
                out_host[name].copy_(t, non_blocking=True)
            copied = torch.cuda.Event()
            copied.record(s_out)
        torch.cuda.current_stream().wait_event(copied)   # the timing events sit on the current stream

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step, steps, warmup, repeats):
        """`repeats` repetitions of the `steps`-long loop, each bracketed by a barrier and a device synchronisation and
        timed with CUDA events; every repetition's time is the max over ranks.  Returns per-step ms of all
        repetitions, the launches of one repetition and the clocks seen under load."""
        for _ in range(warmup):
            step()
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        per_step, launches = [], 0
        with ClockSampler(local_rank) as clocks:
            for _ in range(repeats):
                barrier()
                launches0 = sb.kernel_launches()
                start.record()
                for _ in range(steps):
                    step()
                stop.record()
                barrier()
                launches = sb.kernel_launches() - launches0
                per_step.append(start.elapsed_time(stop) / steps)
        if distributed:
            t = torch.tensor(per_step, device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            per_step = t.tolist()
        return per_step, launches, clocks.summary()

    def host_time_us(step, calls=20):
        """Host time of one un-synchronised forward + backward call: what the Python and C layers cost per step."""
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(calls):
            step()
        dt = time.perf_counter() - t0
        torch.cuda.synchronize()
        return dt / calls * 1e6

    repeats = max(1, args.repeats)
    ms_reps, launches, clocks = timed(step_resident, args.steps, max(args.warmup, 3), repeats)
    ms_step = statistics.median(ms_reps)
    sb.check_status(device)
    # The same step with the per-score arithmetic forced for every score (SB_FLAG_DENSE_ROW_PASS): by default the row
    # passes form only the running log-sum where the weights are exact zeros for a whole warp -- with N(0, 1) inputs that
    # is most of every sequence -- and this figure says what that is worth (every MMA runs either way).
    def step_dense():
        with sb.dense_row_pass():
            return step_resident()
    dense_reps, _, _ = timed(step_dense, args.steps, 3, min(repeats, 3))
    ms_dense = statistics.median(dense_reps)
    host_us = host_time_us(step_resident)
    e2e_steps = max(3, min(args.steps, 20))
    e2e_reps, _, _ = timed(step_e2e, e2e_steps, 3, min(repeats, 3))
    ms_e2e = statistics.median(e2e_reps)

    fl = flops_of(w, mode)
    value = fl * world / (ms_step * 1e-3) / 1e12
    e2e_value = fl * world / (ms_e2e * 1e-3) / 1e12
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = sum(t.numel() * t.element_size() for t in out_host.values())

    line = None
    if rank == 0:
        peaks, peak_kind = load_peaks()
        kern, path = kernel_breakdown(sb, w, dev_t, cu, max_len)
        alg = {"fwd": flops_of(w, "fwd"), "bwd_dq": 0.6 * flops_of(w, "bwd"), "bwd_dkv": 0.4 * flops_of(w, "bwd")}
        kernels = {name: {"ms": ms, "tflops": alg[name] / (ms * 1e-3) / 1e12} for name, ms in kern.items()}
        top = max(kern, key=lambda n: kern[n])
        achieved = kernels[top]["tflops"]
        roofline = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": peaks["bf16_tflops"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                    "traffic": ncu_traffic(args.workload, top),
                    "peak_source": f"{peak_kind} dense bf16 (burst)", "kernels": kernels,
                    "step_frac_of_peak": value / world / peaks["bf16_tflops"],
                    "kernel_path": "tcgen05" if path == 1 else "cuda-core"}
        if fwd_only:
            # forward-only workloads with a low arithmetic intensity sit under the HBM roof: q, k, v read once, o, rem
            # and log_rem written once are the algorithmic bytes
            tokens, esz = sum(w["lengths"]), 2
            alg_bytes = w["heads"] * tokens * (4 * w["head_dim"] * esz + esz + 8)
            if fl / alg_bytes < peaks["bf16_tflops"] * 1e12 / (peaks["hbm_gbs"] * 1e9):
                gbs = alg_bytes / (kern["fwd"] * 1e-3) / 1e9
                roofline.update({"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                 "frac": gbs / peaks["hbm_gbs"], "peak_source": f"{peak_kind} HBM copy",
                                 "algorithmic_bytes": alg_bytes})
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            heads = min(4, w["heads"])
            seqs = len(w["lengths"]) if max(w["lengths"]) <= 4096 else 1
            sec, tfl, desc, kind = cpu_sample(w, heads, seqs, 2)
            cpu = {"value": tfl, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
                   "sample": desc, "seconds": sec, "host_cores": os.cpu_count()}
        line = {
            "metric": "sb_attn_varlen fwd+bwd TFLOP/s" if not fwd_only else "sb_attn_varlen fwd TFLOP/s",
            "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["label"], "name": args.workload, "tokens_per_gpu": sum(w["lengths"]),
                       "sequences_per_gpu": len(w["lengths"]), "heads": w["heads"], "head_dim": w["head_dim"],
                       "parallelism": f"{world} independent shard(s), no collective",
                       "l2": "q,k,v,dO and the outputs of one step exceed the 126 MB L2; no flush between steps",
                       "flop_convention": "causal: fwd 2*L^2*d per head per sequence, bwd 2.5x"},
            "tokens_per_s": sum(w["lengths"]) * world / (ms_step * 1e-3),
            "timing": {"repeats": repeats, "ms_per_step_median": ms_step, "ms_per_step_min": min(ms_reps),
                       "ms_per_step_max": max(ms_reps), "host_us_per_step": host_us,
                       "note": "each repetition: barrier, K steps between CUDA events, barrier; max over ranks; "
                               "value uses the median repetition; host_us_per_step is the wall time the Python and C "
                               "layers take to enqueue one forward + backward (rank 0, no synchronisation)"},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e, "steps": e2e_steps, "repeats": len(e2e_reps),
                    "pinned_gb_per_s_per_rank": (h2d + d2h) / (ms_e2e * 1e-3) / 1e9,
                    "overlap": "h2d of step i+1 and d2h of step i-1 run on their own streams while step i computes"},
            "dense_row_pass": {"value": fl * world / (ms_dense * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_dense,
                               "repeats": len(dense_reps),
                               "note": "same step with SB_FLAG_DENSE_ROW_PASS: the row passes evaluate every score, also "
                                       "where a whole warp's weights are exact zeros (bit-identical results)"},
            "gpu_launches": launches * repeats,
            "gpu_launches_per_repetition": launches,
            "clocks": clocks,
            "roofline": roofline,
            "cpu_baseline": cpu,
        }
    if not args.no_sharded and args.workload == "c2":
        sharded = run_sharded(sb, device, rank, world, dist if distributed else None)
        if line is not None:
            line["sharded"] = sharded
    if distributed:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# the same total work split across the ranks (strong scaling); no collective inside any timed region
# ---------------------------------------------------------------------------------------------------
def run_sharded(sb, device, rank, world, dist, steps=3):
    """Long-context workload (one 131072-token sequence, 16 heads) split by heads, and the skewed packed workload
    (65536 tokens in lognormal-length sequences, 32 heads) split by sequences under three plans: contiguous
    token-balanced runs, contiguous runs balanced by sum of L^2, and longest-first assignment of whole sequences.
    Every rank builds the full inputs from the same seed on its own GPU, keeps its shard and runs the ordinary
    operator on it.  Times: CUDA events per rank, max and mean over ranks.  Afterwards, outside any timed region, the
    shards' results are gathered over NCCL and rank 0 compares them bitwise with an unsharded run."""
    from stickbreaking_attention_b200 import shard

    def full_inputs(w, seed):
        gen = torch.Generator(device=device).manual_seed(seed)
        T = sum(w["lengths"])
        shape = (w["heads"], T, w["head_dim"])
        t = {}
        for name in ("q", "k", "v"):
            t[name] = (w["std"] * torch.randn(shape, generator=gen, device=device)).to(torch.bfloat16)
        t["do"] = torch.randn(shape, generator=gen, device=device).to(torch.bfloat16)
        t["drem"] = torch.randn(shape[:2], generator=gen, device=device).to(torch.bfloat16)
        return t

    def run_op(t, lengths, n_steps):
        """(outputs of the last step, ms per step) of forward + backward over the packed tensors in t."""
        if not lengths or t["q"].shape[0] == 0:
            return None, 0.0
        cu = torch.tensor(lengths, dtype=torch.int32).cumsum(0).to(torch.int32).to(device)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        outs = None
        for i in range(n_steps + 2):          # two warm-up steps
            if i == 2:
                torch.cuda.synchronize()
                start.record()
            q, k, v = (t[n].detach().requires_grad_(True) for n in ("q", "k", "v"))
            o, rem = sb.sb_attn_varlen(q, k, v, cu, max(lengths), zero_start=False)
            dq, dk, dv = torch.autograd.grad((o, rem), (q, k, v), (t["do"], t["drem"]))
            outs = {"o": o.detach(), "rem": rem.detach(), "dq": dq, "dk": dk, "dv": dv}
        stop.record()
        torch.cuda.synchronize()
        return outs, start.elapsed_time(stop) / n_steps

    def rank_times(ms):
        if dist is None:
            return [ms]
        t = torch.zeros(world, device=device, dtype=torch.float64)
        t[rank] = ms
        dist.all_reduce(t)
        return t.tolist()

    def summarise(w, times, extra):
        slow = max(times)
        fl = flops_of(w, "fwd_bwd")
        out = {"ms_max": slow, "ms_mean": sum(times) / len(times), "ms_per_rank": times,
               "tokens_per_s": sum(w["lengths"]) / (slow * 1e-3), "tflops": fl / (slow * 1e-3) / 1e12}
        out.update(extra)
        return out

    result = {"scaling": "strong", "ranks": world, "steps": steps}

    # ---- one long sequence, split by heads
    w4 = workload("c4")
    full = full_inputs(w4, 4242)
    h0, h1 = shard.head_range(w4["heads"], world, rank)
    mine = {n: x[h0:h1] for n, x in full.items()}
    if dist is not None:
        dist.barrier()
    outs, ms = run_op(mine, w4["lengths"], steps)
    times = rank_times(ms)
    verify = None
    if dist is not None:
        gathered = {n: shard.all_gather_heads(x, w4["heads"]) for n, x in outs.items()}
        if rank == 0:
            pick = [0, w4["heads"] - 1]
            ref_outs, _ = run_op({n: x[pick].contiguous() for n, x in full.items()}, w4["lengths"], 1)
            verify = all(torch.equal(gathered[n][pick], ref_outs[n]) for n in ref_outs)
        del gathered
    result["long_context_by_heads"] = summarise(
        w4, times, {"workload": w4["label"], "heads_per_rank": h1 - h0, "plan": "shard.head_range",
                    "backward": "recomputing dK/dV kernel (one head's stored tiles, 34 GB, exceed the default 8 GiB "
                                "scratch budget)", "gathered_equals_unsharded": verify})
    # the same split with the backward's scratch budget raised to 40 GiB, where the GPU has the memory to spare: one
    # head's tiles then fit and the stored-tiles kernels run, head by head
    free_bytes, _ = torch.cuda.mem_get_info(device)
    roomy = free_bytes > (60 << 30)
    if dist is not None:
        flag = torch.tensor([int(roomy)], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        roomy = bool(flag.item())
    if roomy:
        old_budget = sb.set_backward_scratch_budget(40 << 30)
        try:
            if dist is not None:
                dist.barrier()
            _, ms = run_op(mine, w4["lengths"], steps)
        finally:
            sb.set_backward_scratch_budget(old_budget)
        result["long_context_by_heads_scratch_40GiB"] = summarise(
            w4, rank_times(ms), {"heads_per_rank": h1 - h0, "backward": "stored-tiles kernels, one head per chunk"})
    del full, mine, outs
    torch.cuda.empty_cache()

    # ---- skewed packed batch, split by sequences
    w3 = workload("c3")
    lengths = w3["lengths"]
    full = full_inputs(w3, 4343)
    whole_outs = None
    if dist is not None and rank == 0:
        whole_outs, _ = run_op(full, lengths, 1)
    plans = {
        "contiguous_by_tokens": [list(range(a, b)) for a, b in shard.contiguous_segments(lengths, world, by="tokens")],
        "contiguous_by_work": [list(range(a, b)) for a, b in shard.contiguous_segments(lengths, world, by="work")],
        "lpt_by_work": shard.lpt_assignment(lengths, world, by="work"),
    }
    result["skewed_by_sequences"] = {"workload": w3["label"], "sequences": len(lengths),
                                     "longest": max(lengths), "plans": {}}
    for name, parts in plans.items():
        seqs = parts[rank]
        tensors, my_lengths, index = shard.slice_packed([full[n] for n in ("q", "k", "v", "do", "drem")], lengths, seqs)
        mine = dict(zip(("q", "k", "v", "do", "drem"), (x.contiguous() for x in tensors)))
        if dist is not None:
            dist.barrier()
        outs, ms = run_op(mine, my_lengths, steps)
        times = rank_times(ms)
        verify = None
        if dist is not None:
            ok = True
            for n in ("o", "rem", "dq", "dk", "dv"):
                # a rank whose plan gave it no sequence still takes part in the gather, with zero tokens
                local = outs[n] if outs is not None else full["drem" if n == "rem" else "q"][:, :0]
                gathered = shard.all_gather_tokens(local, index, sum(lengths))
                if rank == 0:
                    ok = ok and torch.equal(gathered, whole_outs[n])
                del gathered
            verify = ok if rank == 0 else None
        result["skewed_by_sequences"]["plans"][name] = summarise(
            w3, times, {"imbalance_tokens": shard.imbalance(lengths, parts, by="tokens"),
                        "imbalance_work": shard.imbalance(lengths, parts, by="work"),
                        "sequences_per_rank": [len(p) for p in parts], "gathered_equals_unsharded": verify})
        del mine, outs
    del full, whole_outs
    torch.cuda.empty_cache()
    return result


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sharded", action="store_true", help="skip the sharded workloads (profiler runs)")
    ap.add_argument("--repeats", type=int, default=10, help="repetitions of the timed K-step loop")
    ap.add_argument("--reference-budget-s", type=float, default=1200.0,
                    help="--impl reference: wall-clock allowance for the W + K steps; the whole workload runs per step "
                         "unless the first step shows that it would not fit")
    ap.add_argument("--small-workspace", action="store_true",
                    help="backward recomputes the attention tiles in the dK/dV kernel instead of storing them")
    args = ap.parse_args()
    w = workload(args.workload)
    if args.impl == "reference":
        run_reference_arm(args, w)
    elif args.small_workspace:
        import stickbreaking_attention_b200 as sb
        with sb.small_backward_workspace():
            run_gpu_arm(args, w)
    else:
        run_gpu_arm(args, w)


if __name__ == "__main__":
    main()
