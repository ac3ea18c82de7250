"""CPU-side checks of the drop-in boundary: the library loads, exports every symbol that
include/sllm.h declares, fills defaults as the reference's structs do, and refuses to compute
without a GPU (no fallback)."""
import ctypes as C
import os
import re

import pytest

import small_llm_b200 as sl
from small_llm_b200 import api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_symbols_all_exported():
    hdr = open(os.path.join(ROOT, "include", "sllm.h")).read()
    declared = set(re.findall(r"\b(sllm_[a-z_0-9]+)\s*\(", hdr))
    assert declared, "no declarations found"
    assert declared == set(api.ABI_SYMBOLS)
    lib = sl.load_library()
    for name in declared:
        assert hasattr(lib, name), name


def test_defaults_match_reference_structs():
    lib = sl.load_library()
    c = api._ModelConfig()
    lib.sllm_default_model_config(C.byref(c))
    d = sl.ModelConfig()
    assert (c.vocab_size, c.context_length, c.num_layers, c.d_model, c.num_heads, c.ffn_hidden) == \
        (d.vocab_size, d.context_length, d.num_layers, d.d_model, d.num_heads, d.ffn_hidden) == \
        (32768, 2048, 16, 640, 10, 1728)
    assert c.rope_theta == 10000.0 and abs(c.rms_eps - 1e-5) < 1e-12
    assert d.totalParams() == 100_291_200 and d.head_dim() == 64
    s = api._Sampling()
    lib.sllm_default_sampling(C.byref(s))
    o = sl.SamplingOptions()
    assert abs(s.temperature - 0.7) < 1e-7 and abs(s.top_p - 0.8) < 1e-7 and abs(s.repetition_penalty - 1.1) < 1e-7
    assert (s.seed, s.stop_token, s.eos_token) == (o.seed, o.stop_token, 32762) == (1234, -1, 32762)


def test_bad_configs_rejected_before_any_device_work():
    with pytest.raises(ValueError, match="d_model must equal num_heads"):
        sl.Engine(sl.ModelConfig(d_model=100, num_heads=3))
    with pytest.raises(ValueError, match="context length must be greater than zero"):
        sl.Engine(sl.ModelConfig(context_length=0))
    with pytest.raises(ValueError, match="head_dim"):
        sl.Engine(sl.ModelConfig(d_model=96, num_heads=1))


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(sl.SllmError, match="no CUDA device"):
        sl.Engine(sl.ModelConfig())
