"""Builds the sm_100a attention library in-tree with nvcc (no JIT cache).

    python -m fblt_b200.build            # fblt_b200/libfblt_attn.so
    python -m fblt_b200.build --verbose  # also prints ptxas register / shared-memory usage
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libfblt_attn.so"
SOURCES = ["status.cu", "head_l0.cu", "row_kernel.cu", "tile_kernel.cu", "tile5_kernel.cu", "unit5_kernel.cu", "gemm5_kernel.cu", "mha.cu", "decode_kernel.cu", "decisions.cu", "mask_dense.cu", "gather.cu",
           "api.cu", "session.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "fblt_attn.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel for sm_100a into one shared library. Returns its path."""
    if not force and not verbose and not _stale():
        return LIB
    objs = []
    procs = []
    for s in SOURCES:
        obj = CSRC / (Path(s).stem + ".o")
        cmd = [_nvcc(), *ARCH, "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-c", str(CSRC / s), "-o",
               str(obj)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {s}:\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("nvcc compilation failed")
    link = [_nvcc(), *ARCH, "-shared", "-o", str(LIB), *objs, "-lcudart", "-ldl"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    path = build(force=True, verbose="--verbose" in sys.argv)
    print(path)
