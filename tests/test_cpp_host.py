"""The C++ host-side mirror (include/systemds_cla.hpp): compiles against the C ABI; on a GPU box the program runs
every product and compares with a dense evaluation; without a GPU it must fail loudly (no CPU path)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "test_host_mirror.cpp")
EXE = os.path.join(ROOT, "tests", "cpp", "test_host_mirror.bin")
LIBDIR = os.path.join(ROOT, "systemds_b200")


def build():
    cmd = ["g++", "-std=c++17", "-O1", SRC, "-o", EXE, f"-L{LIBDIR}", "-lsystemds_cla", f"-Wl,-rpath,{LIBDIR}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    return EXE


def test_cpp_mirror_builds_and_has_no_cpu_path():
    import torch
    exe = build()
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present; covered by the gpu test")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 3, r.stdout + r.stderr  # CLA_ERR_CUDA reported through DMLCompressionException
    assert "no usable CUDA device" in r.stdout


@pytest.mark.gpu
def test_cpp_mirror_products_on_gpu():
    exe = build()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "MISMATCH" not in r.stdout
