"""Compile the CUDA sources of this package for sm_100a into one shared library.

    python -m sm120_nvfp4_b200.build            # builds sm120_nvfp4_b200/libb200_nvfp4.so

The library is built in-tree (it is git-ignored) and exports the C ABI declared in
include/b200_nvfp4.h plus the C++ API of include/sm120_nvfp4/. nvcc cross-compiles without a
GPU. cudart is linked statically; nothing else is linked (the driver entry point used to
encode tensor maps is fetched at run time).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OUT = PKG / "libb200_nvfp4.so"
SOURCES = ["gemm.cu", "gemm_splitk_static.cu", "gemm_host.cu", "moe_kernels.cu", "ep_kernels.cu", "fused_moe.cu", "host_common.cpp", "api.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v",
              f"-I{ROOT / 'include'}", f"-I{CSRC}"]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.hpp")) + list((ROOT / "include").rglob("*.h*"))
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    jobs = []
    for name in SOURCES:
        src = CSRC / name
        obj = objdir / (name + ".o")
        if force or _stale(obj, [src, *headers]):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        flags = list(NVCC_FLAGS)
        if src.name == "api.cpp":  # the C++ API symbols are part of the public surface
            flags[flags.index("-fPIC,-fvisibility=hidden")] = "-fPIC"
        cmd = [_nvcc(), *flags, "-x", "cu", "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        return src.name, res.stderr

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        for name, log in pool.map(compile_one, jobs):
            (objdir / (name + ".ptxas.log")).write_text(log)
            if verbose:
                print(f"== {name}\n{log}")
    objs = [objdir / (n + ".o") for n in SOURCES]
    if force or jobs or _stale(OUT, objs):
        cmd = [_nvcc(), "-shared", "-o", str(OUT), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
