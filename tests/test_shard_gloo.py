"""The multi-GPU partitioning (N > 1) exercised with two gloo ranks on CPU.

Each rank takes its slice (heads, or whole sequences), computes it (the CPU oracle stands in for
the CUDA operator here: this test is about the partition and the verification gather, not the
kernels) and the gathered result must equal the unpartitioned computation."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from stickbreaking_attention_b200 import shard
        from oracle import sb_oracle as O
        gen = torch.Generator().manual_seed(0)
        lengths = [33, 7, 64, 20, 5]
        H, T, d = 3, sum(lengths), 16
        q, k, v = (torch.randn(H, T, d, generator=gen) for _ in range(3))
        cu = torch.tensor(lengths).cumsum(0)
        full_o, full_rem = O.varlen_dense(q, k, v, cu)
        if mode == "heads":
            h0, h1 = shard.head_range(H, world, rank)
            o, rem = O.varlen_dense(q[h0:h1], k[h0:h1], v[h0:h1], cu)
            got_o = shard.all_gather_heads(o, H)
            got_rem = shard.all_gather_heads(rem, H)
        else:
            if mode == "segments":
                a, b = shard.contiguous_segments(lengths, world, "tokens")[rank]
                ids = list(range(a, b))
            else:
                ids = shard.lpt_assignment(lengths, world)[rank]
            (qs, ks, vs), lens, index = shard.slice_packed([q, k, v], lengths, ids)
            o, rem = O.varlen_dense(qs, ks, vs, torch.tensor(lens).cumsum(0)) if lens else \
                (qs.clone(), qs[..., 0].clone())
            got_o = shard.all_gather_tokens(o, index, T)
            got_rem = shard.all_gather_tokens(rem, index, T)
        ok = torch.allclose(got_o, full_o, atol=1e-6) and torch.allclose(got_rem, full_rem, atol=1e-6)
        dist.barrier()
        open(os.path.join(out_dir, f"rank{rank}.{'ok' if ok else 'bad'}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["heads", "segments", "lpt"])
def test_partition_and_gather_world2(tmp_path, mode):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), mode, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["rank0.ok", "rank1.ok"]
