"""Bit-for-bit pin of the C oracle against the reference compiled from its own sources.

Runs wherever oracle/_ref/libsllm_ref.so exists (built by `make -C oracle ref` from the reference
tree); skipped elsewhere -- the golden vectors cover that case.
"""
import os

import numpy as np
import pytest

from oracle.binding import Config, OracleModel, RefModel, prompt_ids, ref_available

pytestmark = pytest.mark.skipif(not ref_available(), reason="reference library not built on this machine")

CFGS = [
    Config(vocab=512, context=64, layers=2, d_model=64, heads=2, ffn=96),
    Config(vocab=256, context=32, layers=3, d_model=48, heads=3, ffn=40, theta=500.0, eps=1e-6),   # odd sizes
]


@pytest.mark.parametrize("cfg", CFGS)
def test_weights_forward_checkpoint_bit_equal(cfg, tmp_path):
    o, r = OracleModel(cfg), RefModel(cfg)
    o.init_normal(11, 0.1)
    r.init_normal(11, 0.1)
    for (n1, a), (n2, b) in zip(o.params(), r.params()):
        assert n1 == n2 and np.array_equal(a, b)
    T = cfg.context
    ids = prompt_ids(4, 3 * T, cfg.vocab)
    assert np.array_equal(o.forward(ids, 3, T), r.forward(ids, 3, T))
    # single-token and empty-batch edges
    assert np.array_equal(o.forward(ids[:1], 1, 1), r.forward(ids[:1], 1, 1))
    # the oracle's checkpoint writer produces what the reference's loader accepts, bit for bit
    path = str(tmp_path / "ck.bin")
    o.save_checkpoint(path, 5, 6)
    r2 = RefModel(cfg)
    assert r2.load_checkpoint(path) == (5, 6)
    for (_, a), (_, b) in zip(o.params(), r2.params()):
        assert np.array_equal(a, b)
    o2 = OracleModel(cfg)
    assert o2.load_checkpoint(path) == (5, 6)
    for (_, a), (_, b) in zip(o.params(), o2.params()):
        assert np.array_equal(a, b)


def test_reference_errors(tmp_path):
    cfg = CFGS[0]
    r, o = RefModel(cfg), OracleModel(cfg)
    with pytest.raises(RuntimeError, match="exceeds context_length"):
        r.forward(np.zeros(cfg.context + 1, np.uint32), 1, cfg.context + 1)
    with pytest.raises(RuntimeError, match="exceeds context_length"):
        o.forward(np.zeros(cfg.context + 1, np.uint32), 1, cfg.context + 1)
    with pytest.raises(RuntimeError, match="zero tokens"):
        r.generate_tokens(np.zeros(0, np.uint32), 3, 0.7, 0.8, 1.1, 1)
    with pytest.raises(RuntimeError, match="zero tokens"):
        o.generate(np.zeros(0, np.uint32), 3, 0.7, 0.8, 1.1, seed=1)
    path = str(tmp_path / "ck.bin")
    o.save_checkpoint(path)
    data = open(path, "rb").read()
    open(path, "wb").write(data[:-10])                       # cut inside the last tensor
    with pytest.raises(RuntimeError, match="truncated"):
        r.load_checkpoint(path)
    with pytest.raises(RuntimeError, match="truncated"):
        o.load_checkpoint(path)
    open(path, "wb").write(data[: len(data) // 2])           # cut mid-file: the next name reads empty
    with pytest.raises(RuntimeError, match="expected parameter"):
        r.load_checkpoint(path)
    with pytest.raises(RuntimeError):
        o.load_checkpoint(path)
    other = OracleModel(CFGS[1])
    other.save_checkpoint(path)
    with pytest.raises(RuntimeError, match="parameter count differs"):
        r.load_checkpoint(path)
    with pytest.raises(RuntimeError, match="parameter count differs"):
        o.load_checkpoint(path)


@pytest.mark.parametrize("opts", [(0.8, 0.95, 1.15, 2), (0.7, 0.8, 1.1, 1234), (1.3, 0.5, 1.0, 7), (0.2, 0.999, 2.0, 8)])
def test_token_loop_equals_reference_loop(opts):
    """Inference::generateTokens (reference, own RNG) vs the restated loop fed the same draws."""
    t, p, pen, seed = opts
    cfg = CFGS[0]
    o, r = OracleModel(cfg), RefModel(cfg)
    o.init_normal(3, 0.2)
    r.init_normal(3, 0.2)
    prompt = prompt_ids(seed, 9, cfg.vocab)
    a = r.generate_tokens(prompt, 90, t, p, pen, seed, eos_merges=cfg.vocab - 6 - 256)
    b = o.generate(prompt, 90, t, p, pen, eos=cfg.vocab - 6, seed=seed)
    assert np.array_equal(a, b)


def test_reference_greedy_quirk():
    """temperature <= 0 in the reference computes an argmax but never appends it."""
    cfg = CFGS[0]
    r = RefModel(cfg)
    r.init_normal(3, 0.2)
    prompt = prompt_ids(1, 6, cfg.vocab)
    assert np.array_equal(r.generate_tokens(prompt, 5, 0.0, 0.9, 1.0, 1, eos_merges=250), prompt)


def test_cross_entropy_bit_equal():
    """ops::cross_entropy (src/ops/cross_entropy.cpp:14-54): all positions, masked positions with num_valid,
    a single row, peaked and flat rows."""
    from oracle.binding import cross_entropy
    cfg = CFGS[0]
    r = RefModel(cfg)
    rng = np.random.default_rng(3)
    logits = (rng.normal(0, 3.0, size=(37, cfg.vocab))).astype(np.float32)
    logits[5] = 0.0
    logits[6, 17] = 60.0
    targets = rng.integers(0, cfg.vocab, size=37).astype(np.int32)
    a, b = cross_entropy(logits, targets), r.cross_entropy(logits, targets)
    assert np.float32(a) == np.float32(b)
    masked = targets.copy()
    masked[::3] = -1
    nv = int((masked >= 0).sum())
    assert np.float32(cross_entropy(logits, masked, nv)) == np.float32(r.cross_entropy(logits, masked, nv))
    assert np.float32(cross_entropy(logits[:1], targets[:1])) == np.float32(r.cross_entropy(logits[:1], targets[:1]))
