"""Builds ``libsb_b200.so`` (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

Used by ``setup.py`` and by ``__graft_entry__.build()``; can be run directly::

    python stickbreaking_attention_b200/build.py [--force] [--verbose]

(by file path: importing the package itself already requires the built library).  Setting
``SB_TRACE=1`` in the environment compiles the kernels' event log in (``-DSB_TRACE``); normal builds
leave it out because even the untaken branches cost a few percent.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libsb_b200.so")
SOURCES = ("sb_api.cu", "sb_simt.cu", "sb_tc.cu", "sb_tc_fwd256.cu", "sb_tc_fwd128.cu", "sb_tc_bwd.cu")
HEADERS = ("sb_common.cuh", "sb_ptx.cuh", "sb_tc_common.cuh", "sb_tc_fwd_rows.cuh", "../../include/sb_b200.h")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-Xptxas", "-v",
)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC=/path/to/nvcc")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = find_nvcc()
    extra = ("-DSB_TRACE",) if os.environ.get("SB_TRACE") == "1" else ()
    obj_dir = os.path.join(PKG_DIR, "build")
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, h) for h in HEADERS]
    objs, procs = [], []
    for src in SOURCES:
        src_path = os.path.join(CSRC, src)
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [src_path, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", src_path, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(out)
        with open(os.path.join(obj_dir, src + ".ptxas.log"), "w") as f:
            f.write(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    if force or procs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
