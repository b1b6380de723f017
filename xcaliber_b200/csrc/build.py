"""Builds libxmoe_b200.so (sm_100a only) in-tree with nvcc.

Usage: python -m xcaliber_b200.csrc.build [--force] [--verbose]
One object per .cu (compiled in parallel), linked into xcaliber_b200/libxmoe_b200.so.
The library links the CUDA runtime statically and resolves the one driver symbol it
needs (tensor-map encoding) at run time, so it also loads on a machine without a GPU.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB = PKG / "libxmoe_b200.so"
SOURCES = ["router.cu", "act_quant.cu", "misc.cu", "ff1_nvfp4.cu", "ff1_nvfp4_prefill.cu", "ff1_nvfp4_pair.cu", "ff2_w4a16.cu", "ff2_w4a16_pair.cu", "ep_p2p.cu", "probe.cu", "gate.cu", "api.cu"]
HEADERS = ["common.cuh", "kernels.h", "tile_sched.cuh", "cluster.cuh", "nvfp4_quant.cuh", "../../include/xmoe_b200.h"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    obj_dir = CSRC / "build"
    obj_dir.mkdir(exist_ok=True)
    hdrs = [(CSRC / h).resolve() for h in HEADERS] + [Path(__file__)]
    jobs = []
    for src in SOURCES:
        obj = obj_dir / (src[:-3] + ".o")
        if force or _stale(obj, [CSRC / src] + hdrs):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            for cmd, res in zip(jobs, pool.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs)):
                if verbose or res.returncode:
                    sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
                if res.returncode:
                    raise RuntimeError(f"nvcc failed on {cmd[-3]}")
    objs = [obj_dir / (s[:-3] + ".o") for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
