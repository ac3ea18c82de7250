"""small_llm_b200: B200-native token loop for small-llm (prefill, KV-cached decode, sampling).

The product is the shared library ``libsllm_b200.so`` (hand-written sm_100a kernels behind the C ABI
of ``include/sllm.h``).  This package is the Python host layer over that ABI: classes with the
reference's names (``ModelConfig``, ``Model``, ``Inference``, ``SamplingOptions``,
``load_checkpoint_weights``) that forward to the library through ctypes.  There is no CPU path: every
call that computes raises when the library or a Blackwell GPU is missing.
"""
from .api import (Engine, EngineOptions, Inference, Model, ModelConfig, SamplingOptions, SllmError, TrainState,
                  lib_path, load_checkpoint_weights, load_library)

__all__ = ["Engine", "EngineOptions", "Inference", "Model", "ModelConfig", "SamplingOptions", "SllmError",
           "TrainState", "lib_path", "load_checkpoint_weights", "load_library"]
