"""Compiles the C++ host mirror (sharpnet_b200/host/sharpnet_tensor.hpp) and its test program with g++
and runs it on the GPU: the C ABI driven from compiled code, as the C# P/Invoke shim would drive it."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _compile(built_library, out):
    lib_dir = os.path.dirname(built_library)
    cmd = ["g++", "-std=c++17", "-O2", os.path.join(ROOT, "tests", "cpp", "test_host_mirror.cpp"), "-I", f"{CUDA}/include",
           "-L", lib_dir, "-L", f"{CUDA}/lib64", "-lsharpnet_b200", "-lcudart", f"-Wl,-rpath,{lib_dir}",
           f"-Wl,-rpath,{CUDA}/lib64", "-o", out]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    return out


def test_cpp_host_mirror_compiles(built_library, tmp_path):
    _compile(built_library, str(tmp_path / "test_host_mirror"))


@pytest.mark.gpu
def test_cpp_host_mirror_runs(built_library, tmp_path, wrapper):
    exe = _compile(built_library, str(tmp_path / "test_host_mirror"))
    proc = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert proc.stdout.strip().splitlines()[-1].startswith("OK"), proc.stdout   # libraries may print a banner first
