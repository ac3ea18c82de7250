"""Shared helpers of the GPU parity tests: build an oracle model and an engine with the same weights
(exchanged through a checkpoint file in the reference's layout, as a user of the reference would)."""
from __future__ import annotations

import os
import tempfile

import numpy as np

from oracle.binding import Config, OracleModel
from small_llm_b200 import Engine, EngineOptions, ModelConfig

SMALL = Config(vocab=512, context=64, layers=2, d_model=64, heads=2, ffn=96)
SMALL_EOS = 506
MID = Config(vocab=1024, context=256, layers=3, d_model=128, heads=4, ffn=200)      # 4 KV pages: split-K path
ODD = Config(vocab=256, context=96, layers=2, d_model=48, heads=3, ffn=40, theta=500.0, eps=1e-6)
FULL = Config()
# BASELINE config 5's layer shape (d=1536, 24 heads x 64, SwiGLU 4096) with 2 layers and a small vocabulary
WIDE = Config(vocab=2048, context=192, layers=2, d_model=1536, heads=24, ffn=4096)


def to_model_config(c: Config) -> ModelConfig:
    return ModelConfig(vocab_size=c.vocab, context_length=c.context, num_layers=c.layers, d_model=c.d_model,
                       num_heads=c.heads, ffn_hidden=c.ffn, rope_theta=c.theta, kRmsNormEps=c.eps)


def make_pair(cfg: Config, seed: int, stddev: float, fp32: bool, max_batch: int = 1, via_checkpoint: bool = True,
              **opts) -> tuple[OracleModel, Engine]:
    o = OracleModel(cfg)
    o.init_normal(seed, stddev)
    eng = Engine(to_model_config(cfg), EngineOptions(max_batch=max_batch, fp32_weights=fp32, **opts))
    if via_checkpoint:
        fd, path = tempfile.mkstemp(suffix=".bin", dir=os.environ.get("TMPDIR", "/tmp"))
        os.close(fd)
        try:
            o.save_checkpoint(path, 3, 4)
            st = eng.load_checkpoint(path)
            assert (st.step, st.data_position) == (3, 4)
        finally:
            os.unlink(path)
    else:
        for name, arr in o.params():
            eng.set_param(name, arr)
    return o, eng


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """max|got-ref| / max|ref| per row, worst row."""
    got = got.reshape(-1, got.shape[-1]); ref = ref.reshape(-1, ref.shape[-1])
    return float((np.abs(got - ref).max(axis=1) / np.abs(ref).max(axis=1)).max())
