"""Regenerates the golden vectors in this folder from the UNMODIFIED reference.

Run where the reference tree is available (it is compiled, where it lies, by
`make -C oracle ref`):   python tests/golden/make_golden.py

Everything written here comes out of the reference's own Model::forward,
Inference::generateTokens, Tensor::randomNormal and load_checkpoint_weights (through
oracle/ref_shim.cpp); nothing is computed by this repository's code.
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.binding import Config, RefModel, build_ref, prompt_ids  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
SMALL = Config(vocab=512, context=64, layers=2, d_model=64, heads=2, ffn=96)
SMALL_EOS_MERGES = 512 - 6 - 256          # Tokenizer::getEosToken() = 256 + merges = 506


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def small():
    r = RefModel(SMALL)
    r.init_normal(0, 0.02)
    w_sha = [sha(a) for _, a in r.params()]
    names = [n for n, _ in r.params()]
    r.init_normal(3, 0.2)                  # peaked logits: exercises top-p and the penalty
    ids = prompt_ids(1, 2 * 24, SMALL.vocab)
    logits = r.forward(ids, 2, 24)
    prompt = prompt_ids(5, 8, SMALL.vocab)
    streams = {}
    for seed, (t, p, pen, n) in {2: (0.8, 0.95, 1.15, 100), 1234: (0.7, 0.8, 1.1, 40), 3: (0.7, 0.8, 1.1, 80)}.items():
        streams[f"stream_seed{seed}"] = r.generate_tokens(prompt, n, t, p, pen, seed, eos_merges=SMALL_EOS_MERGES)
        streams[f"opts_seed{seed}"] = np.array([t, p, pen, n], dtype=np.float64)
    np.savez_compressed(os.path.join(OUT, "small_ref.npz"), ids=ids, logits=logits, prompt=prompt,
                        weight_names=np.array(names), weight_sha_seed0=np.array(w_sha), **streams)


def c1_probe():
    """100.3M config, seed-0 N(0,0.02) weights, the first 24 ids of the seed-1 prompt."""
    cfg = Config()
    r = RefModel(cfg)
    r.init_normal(0, 0.02)
    T = 24
    ids = prompt_ids(1, 128)[:T]
    logits = r.forward(ids, 1, T)[0]                      # [T, V]
    probe = prompt_ids(99, 512)                           # fixed probe columns
    top = np.argsort(-logits, axis=1, kind="stable")[:, :8].astype(np.uint32)
    emb = r.param(0)[1]
    np.savez_compressed(os.path.join(OUT, "c1_ref_probe.npz"), ids=ids, probe_cols=probe,
                        probe_logits=logits[:, probe], top_ids=top,
                        top_vals=np.take_along_axis(logits, top.astype(np.int64), axis=1),
                        row_absmax=np.abs(logits).max(axis=1), row_sum=logits.astype(np.float64).sum(axis=1),
                        emb_row0=emb[0].copy(), emb_sha=np.array(sha(emb)),
                        last_param_sha=np.array(sha(r.param(r.num_params() - 2)[1])))


def cross_entropy_vectors():
    """ops::cross_entropy of the small model's own logits (next-token targets) and of a masked variant."""
    r = RefModel(SMALL)
    r.init_normal(3, 0.2)
    ids = prompt_ids(1, 2 * 24, SMALL.vocab)
    logits = r.forward(ids, 2, 24).reshape(48, SMALL.vocab)
    targets = np.roll(ids.reshape(2, 24), -1, axis=1).reshape(-1).astype(np.int32)     # next id, wrapping inside a row
    masked = targets.copy()
    masked[::4] = -1
    nv = int((masked >= 0).sum())
    np.savez_compressed(os.path.join(OUT, "ce_ref.npz"), ids=ids, targets=targets, masked=masked,
                        loss_all=np.float32(r.cross_entropy(logits, targets)),
                        loss_masked=np.float32(r.cross_entropy(logits, masked, nv)))


def model_init():
    """The reference's own initial weights: Tensor::seed(7), then Model::Model (embedding, then per block q k v out
    gate up down, out/down with std 0.02/sqrt(2L); src/model.cpp:15-29, src/nn/attention.cpp:39-45,
    src/nn/swiglu.cpp:17-22)."""
    r = RefModel(SMALL, ctor_seed=7)
    ps = r.params()
    np.savez_compressed(os.path.join(OUT, "model_init_ref.npz"), names=np.array([n for n, _ in ps]),
                        sha=np.array([sha(a) for _, a in ps]), head=np.stack([a.reshape(-1)[:4] for _, a in ps]),
                        std=np.array([float(a.std()) for _, a in ps]))


def attention_op():
    """ops::attention (src/ops/attention.cpp:143-184) on random q, k, v: [1, 2 heads, 200 positions, 32]."""
    import ctypes as C
    r = RefModel(SMALL)
    rng = np.random.default_rng(11)
    H, T, hd = 2, 200, 32
    q, k, v = (rng.normal(0, 1.0, (1, H, T, hd)).astype(np.float32) for _ in range(3))
    out = np.empty_like(q)
    f32p = C.POINTER(C.c_float)
    rc = r.lib.ref_op_attention(q.ctypes.data_as(f32p), k.ctypes.data_as(f32p), v.ctypes.data_as(f32p), 1, H, T, hd,
                                out.ctypes.data_as(f32p))
    assert rc == 0
    np.savez_compressed(os.path.join(OUT, "attention_op_ref.npz"), q=q, k=k, v=v, out=out)


if __name__ == "__main__":
    if build_ref() is None:
        sys.exit("reference tree not available; golden vectors can only be regenerated where it is")
    small()
    c1_probe()
    cross_entropy_vectors()
    model_init()
    attention_op()
    print("golden vectors written to", OUT)
