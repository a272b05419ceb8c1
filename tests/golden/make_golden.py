"""Regenerates the golden vectors in this folder from the UNMODIFIED reference oracle.

Run where the reference checkout is available::

    python tests/golden/make_golden.py /path/to/stickbreaking-attention

It loads ``stickbreaking_attention/sb_ref.py`` from that checkout by file path (nothing else of
the reference is imported), builds masks and per-sequence splits the way the reference's own tests
do (``tests/test_varlen.py:10-41``, ``tests/test_attn.py:10-32``), and stores inputs, outputs and
autograd gradients.  Nothing from this repository's oracle or kernels takes part, so the stored
numbers are the reference's own.

Cases
-----
tiny_varlen_ac{0,1}   H=2 d=16 lengths [5,17,1,33], N(0,1) fp32, full tensors
tiny_fixed_ac{0,1}    B=2 H=2 T=24 d=50, the reference tests' input recipe, full tensors
recipe_varlen_ac{0,1} H=1 d=128 one sequence of 160, the reference tests' recipe, bf16-rounded inputs
                      (inputs stored as bf16 bit patterns)
c1                    H=4 d=64 lengths [128,256,64,512], torch.manual_seed(0), N(0,1) fp32
                      (inputs are regenerated from the seed; their checksums and every 16th
                      token row of each output are stored)
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    path = os.path.join(root, "stickbreaking_attention", "sb_ref.py")
    spec = importlib.util.spec_from_file_location("_reference_sb_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.stickbreaking


def ref_varlen(stickbreaking, q, k, v, lengths, attend_current):
    longest = max(lengths)
    cm = torch.ones(longest, longest).tril(-1).to(q)
    mask = torch.ones(longest, longest).triu(0 if not attend_current else 1).bool()
    outs, rems = [], []
    for qc, kc, vc in zip(q.split(lengths, 1), k.split(lengths, 1), v.split(lengths, 1)):
        n = qc.size(1)
        o, rem = stickbreaking(qc[None], kc[None], vc[None], mask[:n, :n], cm[:n, :n])
        outs.append(o[0])
        rems.append(rem[0])
    return torch.cat(outs, 1), torch.cat(rems, 1)


def ref_fixed(stickbreaking, q, k, v, attend_current):
    length = q.shape[-2]
    cm = torch.ones(length, length).tril(-1).to(q)
    mask = torch.ones(length, length).triu(1 if attend_current else 0).bool()
    return stickbreaking(q, k, v, mask, cm)


def with_grads(fn, q, k, v, do, drem):
    q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
    o, rem = fn(q, k, v)
    dq, dk, dv = torch.autograd.grad((o, rem), (q, k, v), (do, drem))
    return dict(o=o.detach(), rem=rem.detach(), dq=dq, dk=dk, dv=dv)


def recipe(shape, gen):
    """Input recipe of the reference tests (tests/test_varlen.py:83-89)."""
    v = 0.25 * torch.randn(shape, generator=gen)
    q = 0.25 * (torch.randn(shape, generator=gen) + 1)
    k = 0.25 * (torch.randn(shape, generator=gen) - 1)
    return q, k, v


def save(name, **arrays):
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        **{key: (val.numpy() if torch.is_tensor(val) else np.asarray(val))
                           for key, val in arrays.items()})


def main(root):
    sb = load_reference(root)
    torch.set_num_threads(4)

    for ac in (False, True):
        gen = torch.Generator().manual_seed(11)
        lengths = [5, 17, 1, 33]
        shape = (2, sum(lengths), 16)
        q, k, v, do = (torch.randn(shape, generator=gen) for _ in range(4))
        drem = torch.randn(shape[:2], generator=gen)
        out = with_grads(lambda a, b, c: ref_varlen(sb, a, b, c, lengths, ac), q, k, v, do, drem)
        save(f"tiny_varlen_ac{int(ac)}", q=q, k=k, v=v, do=do, drem=drem,
             lengths=np.array(lengths), **out)

        gen = torch.Generator().manual_seed(12)
        shape = (2, 2, 24, 50)
        q, k, v = recipe(shape, gen)
        do = torch.randn(shape, generator=gen)
        drem = torch.randn(shape[:3], generator=gen)
        out = with_grads(lambda a, b, c: ref_fixed(sb, a, b, c, ac), q, k, v, do, drem)
        save(f"tiny_fixed_ac{int(ac)}", q=q, k=k, v=v, do=do, drem=drem, **out)

        gen = torch.Generator().manual_seed(1337)
        lengths = [160]
        shape = (1, 160, 128)
        q, k, v = (t.bfloat16().float() for t in recipe(shape, gen))
        do = torch.randn(shape, generator=gen).bfloat16().float()
        drem = torch.randn(shape[:2], generator=gen).bfloat16().float()
        out = with_grads(lambda a, b, c: ref_varlen(sb, a, b, c, lengths, ac), q, k, v, do, drem)
        bits = {key: val.bfloat16().view(torch.int16) for key, val in
                dict(q=q, k=k, v=v, do=do, drem=drem).items()}
        save(f"recipe_varlen_ac{int(ac)}", lengths=np.array(lengths), **bits, **out)

    torch.manual_seed(0)
    lengths = [128, 256, 64, 512]
    shape = (4, sum(lengths), 64)
    q, k, v, do = (torch.randn(shape) for _ in range(4))
    drem = torch.randn(shape[:2])
    out = with_grads(lambda a, b, c: ref_varlen(sb, a, b, c, lengths, False), q, k, v, do, drem)
    sums = np.array([float(t.double().sum()) for t in (q, k, v, do, drem)])
    save("c1", lengths=np.array(lengths), input_sums=sums, row_stride=np.array(16),
         **{key: val[:, ::16] for key, val in out.items()})
    print("wrote golden vectors to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/stickbreaking-attention")
    main(sys.argv[1])
