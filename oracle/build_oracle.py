"""Builds the oracle's native pieces. TEST INFRASTRUCTURE ONLY.

  oracle/liboracle_c.so         gcc, from oracle/route_oracle.c (always)
  oracle/_ref/libref_kernels.so nvcc sm_100a, from oracle/ref_kernels.cu + the reference's own
                                topk.cuh / preamble.cuh compiled where they lie (only when the
                                reference tree is present; the prebuilt file is used otherwise)

Usage: python oracle/build_oracle.py [reference_root]
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_SUBDIR = "xFused-NVFP4-Kernels/xMoE/xW4A16/sm120a"


def build_c() -> Path:
    out = HERE / "liboracle_c.so"
    src = HERE / "route_oracle.c"
    if not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-o", str(out), str(src), "-lm"], check=True)
    return out


def build_ref(reference_root: str = "/root/reference") -> Path | None:
    inc = Path(reference_root) / REF_SUBDIR
    out = HERE / "_ref" / "libref_kernels.so"
    if not (inc / "preamble.cuh").exists():
        return out if out.exists() else None
    out.parent.mkdir(exist_ok=True)
    src = HERE / "ref_kernels.cu"
    if not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-shared", "-Xcompiler", "-fPIC",
                        "-I", str(inc), "-o", str(out), str(src)], check=True)
    return out


if __name__ == "__main__":
    print(build_c())
    print(build_ref(*sys.argv[1:2]))
