"""The header-only C++ layer (the reference's class names over the C ABI) on a GPU: a small program loads a
checkpoint, calls Model::forward, Inference::generateTokenIds and ChatSession::sayIds; its results are
compared with the oracle."""
import os
import subprocess

import numpy as np
import pytest

import small_llm_b200 as sl
from oracle.binding import OracleModel
from tests.helpers import MID, rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _read(f, dtype):
    n = int(np.frombuffer(f.read(8), dtype=np.uint64)[0])
    return np.frombuffer(f.read(4 * n), dtype=dtype)


def test_cpp_facade_on_gpu_matches_oracle(tmp_path):
    cfg = MID
    o = OracleModel(cfg)
    o.init_normal(12, 0.1)
    ckpt = str(tmp_path / "w.bin")
    o.save_checkpoint(ckpt, 3, 4)
    libdir = os.path.dirname(sl.lib_path())
    exe, res = str(tmp_path / "facade_gpu"), str(tmp_path / "out.bin")
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "facade_gpu.cpp"),
                    "-o", exe, "-L", libdir, "-lsllm_b200", f"-Wl,-rpath,{libdir}"], check=True)
    eos = 1000
    r = subprocess.run([exe, ckpt, res, str(cfg.vocab), str(cfg.context), str(cfg.layers), str(cfg.d_model), str(cfg.heads),
                        str(cfg.ffn), str(eos - 256)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    ids = np.array([(i * 7919 + 13) % 500 for i in range(2 * 37)], dtype=np.uint32)
    with open(res, "rb") as f:
        logits = _read(f, np.float32).reshape(2, 37, cfg.vocab)
        loss = float(np.frombuffer(f.read(4), dtype=np.float32)[0])
        sampled = _read(f, np.uint32)
        reply1 = _read(f, np.uint32)
        reply2 = _read(f, np.uint32)
    assert rel_err(logits, o.forward(ids, 2, 37)) <= 2e-5                      # fp32 weights
    from oracle.binding import cross_entropy
    targets = np.array([-1 if i % 5 == 0 else int(ids[(i + 1) % ids.size]) for i in range(ids.size)], dtype=np.int32)
    assert abs(loss - cross_entropy(o.forward(ids, 2, 37).reshape(74, cfg.vocab), targets, int((targets >= 0).sum()))) <= 2e-5
    ref = o.generate(ids[:21], 30, 0.8, 0.9, 1.2, seed=77, eos=eos)
    assert np.array_equal(sampled, ref)
    user, asst, end = eos + 1, eos + 2, eos + 3
    ctx1 = np.concatenate([[user], ids[:9], [end, asst]]).astype(np.uint32)
    g1 = o.generate(ctx1, 12, 0.0, 1.0, 1.0, eos=eos, stop=end)
    r1 = g1[ctx1.size:]
    r1 = r1[:-1] if r1[-1] in (eos, end) else r1
    assert np.array_equal(reply1, r1)
    ctx2 = np.concatenate([ctx1, r1, [end], [user], ids[9:20], [end, asst]]).astype(np.uint32)
    g2 = o.generate(ctx2, 12, 0.0, 1.0, 1.0, eos=eos, stop=end)
    r2 = g2[ctx2.size:]
    r2 = r2[:-1] if r2[-1] in (eos, end) else r2
    assert np.array_equal(reply2, r2)
