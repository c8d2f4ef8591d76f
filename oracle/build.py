"""Build the CPU oracle (and, where the reference checkout exists, the
reference-derived checker) as shared libraries.

TEST INFRASTRUCTURE ONLY - see the header of nvfp4_oracle.c.

    python oracle/build.py            # liboracle.so (+ _ref/libref_shim.so if possible)

Outputs:
  oracle/liboracle.so          gcc build of nvfp4_oracle.c (-fopenmp, no FMA contraction)
  oracle/_ref/libref_shim.so   g++ build of ref_shim.cpp against the reference's own
                               src/fused_moe/scale_layout.cuh and CUTLASS / CUDA headers;
                               only built when the reference tree and the headers exist.
  oracle/_ref/libref_bindings.so  the reference's torch bindings of this path compiled unchanged
                               against this repository's C++ headers and linked to its library
                               (build_ref_bindings).
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
# the reference checkout: NVFP4_REFERENCE_DIR, else a directory named "reference" beside this repository
REFERENCE = Path(os.environ.get("NVFP4_REFERENCE_DIR", HERE.parent.parent / "reference"))


def _newer(target: Path, *sources: Path) -> bool:
    return target.exists() and all(target.stat().st_mtime >= s.stat().st_mtime for s in sources)


def build_oracle(force: bool = False) -> Path:
    src = HERE / "nvfp4_oracle.c"
    out = HERE / "liboracle.so"
    if not force and _newer(out, src):
        return out
    cmd = ["gcc", "-O3", "-march=native", "-fopenmp", "-ffp-contract=off", "-fvisibility=hidden",
           "-shared", "-fPIC", "-o", str(out), str(src), "-lm"]
    subprocess.run(cmd, check=True)
    return out


def _cutlass_include() -> Path | None:
    """CUTLASS headers bundled with the flashinfer package (located without importing it)."""
    import importlib.util
    candidates = list(sys.path)
    try:
        spec = importlib.util.find_spec("flashinfer")
        if spec is not None and spec.origin:
            candidates.insert(0, str(Path(spec.origin).resolve().parent.parent))
    except Exception:
        pass
    for p in candidates:
        base = Path(p) / "flashinfer" / "data" / "cutlass" / "include"
        if (base / "cutlass" / "float8.h").exists():
            return base
    return None


def build_ref(force: bool = False) -> Path | None:
    """Returns the path of the built shim, or None when it cannot be built here."""
    out = HERE / "_ref" / "libref_shim.so"
    src = HERE / "ref_shim.cpp"
    layout = REFERENCE / "src" / "fused_moe" / "scale_layout.cuh"
    if not layout.exists():
        return out if out.exists() else None
    cutlass = _cutlass_include()
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    if cutlass is None or not (cuda_inc / "cuda_fp4.h").exists():
        return out if out.exists() else None
    if not force and _newer(out, src, layout):
        return out
    out.parent.mkdir(exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O1", "-shared", "-fPIC", "-w", "-x", "c++",
           f"-I{REFERENCE / 'src'}", f"-I{REFERENCE / 'include'}", f"-I{cutlass}", f"-I{cuda_inc}",
           "-o", str(out), str(src)]
    subprocess.run(cmd, check=True)
    return out


REF_BINDING_SOURCES = ("gemm_ops.cu", "grouped_gemm_ops.cpp", "fused_moe_ops.cpp")


def build_ref_bindings(force: bool = False) -> Path | None:
    """The reference's own torch bindings for this path (bindings/gemm_ops.cu, grouped_gemm_ops.cpp,
    fused_moe_ops.cpp), compiled unchanged from where they lie against THIS repository's
    include/sm120_nvfp4/*.hpp and linked against sm120_nvfp4_b200/libb200_nvfp4.so. The result,
    oracle/_ref/libref_bindings.so, registers the reference's torch ops (sm120_nvfp4::gemm, ...)
    with the reference's argument checks, running on this library's kernels: the drop-in claim
    made executable. Returns the built library, an earlier build when the reference tree is not
    there, or None."""
    out = HERE / "_ref" / "libref_bindings.so"
    srcs = [REFERENCE / "bindings" / name for name in REF_BINDING_SOURCES]
    if not all(s.exists() for s in srcs):
        return out if out.exists() else None
    root = HERE.parent
    lib = root / "sm120_nvfp4_b200" / "libb200_nvfp4.so"
    if not lib.exists():
        return None
    headers = list((root / "include").rglob("*.h*"))
    if not force and _newer(out, *srcs, *headers):   # linked dynamically: a rebuilt library needs no relink
        return out
    import sysconfig
    import torch
    from torch.utils import cpp_extension
    out.parent.mkdir(exist_ok=True)
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    inc = [f"-I{root / 'include'}", *(f"-I{q}" for q in cpp_extension.include_paths()), f"-I{cuda / 'include'}",
           f"-I{sysconfig.get_paths()['include']}"]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    procs, objs = [], []
    for src in srcs:
        obj = out.parent / (src.name + ".o")
        objs.append(obj)
        cmd = ["g++", "-std=c++17", "-O1", "-fPIC", "-w", abi, "-x", "c++", *inc, "-c", str(src), "-o", str(obj)]
        procs.append(subprocess.Popen(cmd))
    for pr in procs:
        if pr.wait() != 0:
            raise RuntimeError("compiling the reference bindings against this repository's headers failed")
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    cmd = ["g++", "-shared", "-o", str(out), *map(str, objs), f"-L{lib.parent}", "-lb200_nvfp4",
           "-Wl,-rpath,$ORIGIN/../../sm120_nvfp4_b200", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda",
           "-lc10", "-lc10_cuda", f"-Wl,-rpath,{torch_lib}", f"-L{cuda / 'lib64'}", "-lcudart",
           "-Wl,--no-undefined"]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
    print(build_ref_bindings(force="--force" in sys.argv))
