"""Builds tests/cpp/api_check.cpp against the public C++ headers and the in-tree library and
runs it: the host-only checks here, the known-answer device checks under the gpu marker."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
SRC = ROOT / "tests" / "cpp" / "api_check.cpp"
OUT = ROOT / "tests" / "cpp" / "_build" / "api_check"


def _build() -> Path:
    from sm120_nvfp4_b200 import build as libbuild
    lib = libbuild.build()
    deps = [SRC, lib, *(ROOT / "include").rglob("*.h*")]
    if OUT.exists() and all(OUT.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    cmd = ["g++", "-std=c++17", "-O1", f"-I{ROOT / 'include'}", f"-I{cuda / 'include'}", str(SRC), "-o", str(OUT),
           f"-L{lib.parent}", "-lb200_nvfp4", f"-Wl,-rpath,{lib.parent}", f"-L{cuda / 'lib64'}", "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    return OUT


def _run(mode: str):
    exe = _build()
    res = subprocess.run([str(exe), mode], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "PASS" in res.stdout, res.stdout + res.stderr


def test_cpp_api_host_checks():
    _run("host")


@pytest.mark.gpu
def test_cpp_api_device_known_answers():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    _run("device")
