"""The C++ serving components (include/sllm_serving.hpp) on a GPU: a program compiled against the headers runs a
ContinuousBatcher and a ShardedInference (two engines on two host threads); every request's tokens must equal what
the oracle generates for that request alone."""
import os
import subprocess

import numpy as np
import pytest

import small_llm_b200 as sl
from oracle.binding import OracleModel, uniforms
from tests.helpers import MID

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _read(f):
    n = int(np.frombuffer(f.read(8), dtype=np.uint64)[0])
    return np.frombuffer(f.read(4 * n), dtype=np.uint32)


def _prompt(r):
    return np.array([(r * 131 + i * 7919 + 13) % 1000 for i in range(5 + 7 * r)], dtype=np.uint32)


def _same_stream(got, ref, o, what, near_ties):
    """Equal streams; or equal up to a step at which the two tokens' reference logits differ by less than 1e-5 of the
    row's largest logit: the engine's fp32 logits equal the oracle's only up to summation order (2e-5), which can swap
    two neighbours of the sampler's descending order.  Such a step is recorded and ends the comparison."""
    if np.array_equal(got, ref):
        return
    n = min(len(got), len(ref))
    diff = np.nonzero(got[:n] != ref[:n])[0]
    assert diff.size, (what, len(got), len(ref))
    i = int(diff[0])
    lg = o.forward(ref[:i], 1, i)[0, -1]
    assert abs(float(lg[got[i]]) - float(lg[ref[i]])) <= 1e-5 * float(np.abs(lg).max()), (what, i, int(got[i]), int(ref[i]))
    near_ties.append((what, i))


def test_cpp_batcher_and_sharding_match_oracle(tmp_path):
    import torch
    cfg = MID
    o = OracleModel(cfg)
    o.init_normal(12, 0.1)
    ckpt = str(tmp_path / "w.bin")
    o.save_checkpoint(ckpt, 0, 0)
    libdir = os.path.dirname(sl.lib_path())
    exe, res = str(tmp_path / "serving_gpu"), str(tmp_path / "out.bin")
    subprocess.run(["g++", "-std=c++17", "-O1", "-pthread", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "serving_gpu.cpp"), "-o", exe, "-L", libdir, "-lsllm_b200",
                    f"-Wl,-rpath,{libdir}"], check=True)
    eos = 700
    devices = "0,1" if torch.cuda.device_count() >= 2 else "0,0"
    r = subprocess.run([exe, ckpt, res, str(cfg.vocab), str(cfg.context), str(cfg.layers), str(cfg.d_model), str(cfg.heads),
                        str(cfg.ffn), str(eos), devices], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    budgets = [30, 22, 4, 17, 9, 25, 12]
    near_ties = []
    with open(res, "rb") as f:
        for i, n in enumerate(budgets):                          # continuous batching, sampled
            got = _read(f)
            ref = o.generate(_prompt(i), n, 0.9, 0.9, 1.1, us=uniforms(70 + i, n), eos=eos)
            _same_stream(got, ref, o, ("batcher", i), near_ties)
        for i in range(5):                                       # sharded, greedy
            got = _read(f)
            assert np.array_equal(got, o.generate(_prompt(10 + i), 12, 0.0, 1.0, 1.0, eos=eos)), ("sharded greedy", i)
        for i in range(5):                                       # sharded, sampled with supplied draws
            got = _read(f)
            ref = o.generate(_prompt(10 + i), 12, 0.8, 0.95, 1.15, us=uniforms(90 + i, 12), eos=eos)
            _same_stream(got, ref, o, ("sharded sampled", i), near_ties)
    assert len(near_ties) <= 2, near_ties
