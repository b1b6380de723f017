"""Builds libxmoe_b200.so (sm_100a only) in-tree with nvcc, and the PyTorch custom-op shim over it.

Usage: python -m xcaliber_b200.csrc.build [--force] [--verbose]
One object per .cu (compiled in parallel), linked into xcaliber_b200/libxmoe_b200.so.
The library links the CUDA runtime statically and resolves the one driver symbol it
needs (tensor-map encoding) at run time, so it also loads on a machine without a GPU.
torch_op.cpp (TORCH_LIBRARY registration, host code only) is compiled with g++ against the
installed torch into xcaliber_b200/libxmoe_torch_ops.so, which depends on libxmoe_b200.so
beside it ($ORIGIN).
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
TORCH_OPS_LIB = PKG / "libxmoe_torch_ops.so"
SOURCES = ["router.cu", "act_quant.cu", "misc.cu", "ff1_nvfp4.cu", "ff1_nvfp4_prefill.cu", "ff1_nvfp4_pair.cu", "ff2_w4a16.cu", "ff2_w4a16_pair.cu", "ep_p2p.cu", "probe.cu", "gate.cu", "decode_front.cu", "api.cu"]
HEADERS = ["common.cuh", "kernels.h", "tile_sched.cuh", "cluster.cuh", "nvfp4_quant.cuh", "router_core.cuh", "k_walk.h", "../../include/xmoe_b200.h"]
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
    build_torch_ops(force=force, verbose=verbose)
    return LIB


def build_torch_ops(force: bool = False, verbose: bool = False) -> Path:
    """g++ only: the shim holds no device code. Linked against the torch libraries by soname (they are
    already loaded when torch.ops.load_library opens the shim) and against libxmoe_b200.so in the same folder."""
    src = CSRC / "torch_op.cpp"
    if not (force or _stale(TORCH_OPS_LIB, [src, (CSRC / "../../include/xmoe_b200.h").resolve(), LIB, Path(__file__)])):
        return TORCH_OPS_LIB
    import torch
    from torch.utils import cpp_extension as ext

    cxx = os.environ.get("CXX", "g++")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-DTORCH_EXTENSION_NAME=libxmoe_torch_ops"]
    cmd += [f"-I{p}" for p in ext.include_paths("cuda")]
    cmd += [str(src), "-o", str(TORCH_OPS_LIB), f"-L{PKG}", "-lxmoe_b200", "-Wl,-rpath,$ORIGIN"]
    cmd += [f"-L{p}" for p in ext.library_paths("cuda") if Path(p).exists()]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("torch op shim failed to build")
    return TORCH_OPS_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
