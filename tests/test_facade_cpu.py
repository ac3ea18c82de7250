"""The header-only C++ layer compiles with g++ against the C ABI and keeps the reference's
exception behaviour on the host (no GPU needed: every compute call must fail loudly here)."""
import os
import subprocess

import pytest
import torch

import small_llm_b200 as sl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.is_available(), reason="host-only behaviour")
def test_cpp_facade_compiles_and_fails_loudly_without_gpu(tmp_path):
    libdir = os.path.dirname(sl.lib_path())
    exe = str(tmp_path / "facade_cpu")
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "facade_cpu.cpp"),
                    "-o", exe, "-L", libdir, "-lsllm_b200", f"-Wl,-rpath,{libdir}"], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "no CUDA device" in r.stdout
