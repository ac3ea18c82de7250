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


def test_model_constructor_initialises_like_the_reference(tmp_path, golden_dir):
    """Model(config) after Tensor::seed(7): every parameter bit-equal with the reference constructor's (golden
    hashes written by tests/golden/make_golden.py from the unmodified reference: embedding first, then per block
    q k v out gate up down, out / down with std 0.02 / sqrt(2 L), gains 1)."""
    import hashlib
    import numpy as np
    libdir = os.path.dirname(sl.lib_path())
    exe, out = str(tmp_path / "facade_init"), str(tmp_path / "w.bin")
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "facade_init.cpp"),
                    "-o", exe, "-L", libdir, "-lsllm_b200", f"-Wl,-rpath,{libdir}"], check=True)
    subprocess.run([exe, out, "7"], check=True)
    g = np.load(os.path.join(golden_dir, "model_init_ref.npz"))
    with open(out, "rb") as f:
        n = int(np.frombuffer(f.read(4), np.uint32)[0])
        assert n == len(g["names"]) == 20
        for i in range(n):
            nl = int(np.frombuffer(f.read(4), np.uint32)[0])
            name = f.read(nl).decode()
            ne = int(np.frombuffer(f.read(8), np.uint64)[0])
            data = np.frombuffer(f.read(4 * ne), np.float32)
            assert name == str(g["names"][i])
            assert np.array_equal(data[:4], g["head"][i]), name
            assert hashlib.sha256(data.tobytes()).hexdigest() == str(g["sha"][i]), name


def test_cpp_balanced_assignment_matches_python(tmp_path):
    """include/sllm_serving.hpp compiles on its own, and its balancedAssignment deals sequences exactly as the Python
    host layer's (small_llm_b200.shard.balanced_assignment) does."""
    import numpy as np
    from small_llm_b200.shard import balanced_assignment
    libdir = os.path.dirname(sl.lib_path())
    exe = str(tmp_path / "serving_cpu")
    subprocess.run(["g++", "-std=c++17", "-O1", "-pthread", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "serving_cpu.cpp"), "-o", exe, "-L", libdir, "-lsllm_b200",
                    f"-Wl,-rpath,{libdir}"], check=True)
    rng = np.random.default_rng(3)
    for world, n in ((1, 5), (2, 7), (3, 10), (8, 64)):
        lens = rng.integers(1, 1537, size=n)
        r = subprocess.run([exe, str(world)] + [str(int(x)) for x in lens], capture_output=True, text=True, check=True)
        got = [[int(t) for t in line.split()] for line in r.stdout.strip("\n").split("\n")]
        assert got == [p.tolist() for p in balanced_assignment(lens, world)]
