"""Build the CPU oracle (and, where the reference checkout exists, the
reference-derived checker) as shared libraries.

TEST INFRASTRUCTURE ONLY - see the header of nvfp4_oracle.c.

    python oracle/build.py            # liboracle.so (+ _ref/libref_shim.so if possible)

Outputs:
  oracle/liboracle.so          gcc build of nvfp4_oracle.c (-fopenmp, no FMA contraction)
  oracle/_ref/libref_shim.so   g++ build of ref_shim.cpp against the reference's own
                               src/fused_moe/scale_layout.cuh and CUTLASS / CUDA headers;
                               only built when the reference tree and the headers exist.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REFERENCE = Path(os.environ.get("NVFP4_REFERENCE_DIR", "/root/reference"))


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


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
