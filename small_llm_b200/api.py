"""ctypes host layer over include/sllm.h, mirroring the reference's C++ inference API.

Reference interface mirrored here (paths inside the small-llm tree):
  ModelConfig          include/config.h:6-47
  SamplingOptions      include/inference.h:9-15
  Model                include/model.h:23-50      (forward, parameters, config; inference half only)
  Inference            include/inference.h:17-27  (generateTokens; generate/generateChat need a tokenizer)
  load_checkpoint_weights / TrainState   include/checkpoint.h:9-17
Exceptions follow the reference: ValueError for std::invalid_argument, RuntimeError for
std::runtime_error / std::logic_error.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

OK, ERR_INVALID, ERR_IO, ERR_CUDA, ERR_CAPACITY, ERR_DEVICE_WAIT, ERR_NONFINITE, ERR_STATE = range(8)

u32p = C.POINTER(C.c_uint32)
u64p = C.POINTER(C.c_uint64)
f32p = C.POINTER(C.c_float)
f64p = C.POINTER(C.c_double)


class SllmError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.code = code


def lib_path() -> str:
    return os.path.join(_HERE, "libsllm_b200.so")


class _ModelConfig(C.Structure):
    _fields_ = [("vocab_size", C.c_uint64), ("context_length", C.c_uint64), ("num_layers", C.c_uint64),
                ("d_model", C.c_uint64), ("num_heads", C.c_uint64), ("ffn_hidden", C.c_uint64),
                ("rope_theta", C.c_float), ("rms_eps", C.c_float)]


class _EngineOptions(C.Structure):
    _fields_ = [("max_batch", C.c_uint32), ("weight_dtype", C.c_uint32), ("kv_pages", C.c_uint64),
                ("max_chunk_tokens", C.c_uint32), ("device", C.c_int32), ("use_graph", C.c_uint32),
                ("reserved", C.c_uint32)]


class _Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("repetition_penalty", C.c_float),
                ("eos_token", C.c_uint32), ("stop_token", C.c_int64), ("seed", C.c_uint64)]


class _Stats(C.Structure):
    _fields_ = [("weight_bytes", C.c_uint64), ("kv_bytes", C.c_uint64), ("scratch_bytes", C.c_uint64),
                ("kv_pages_total", C.c_uint64), ("kv_pages_free", C.c_uint64), ("launches", C.c_uint64),
                ("decode_steps", C.c_uint64), ("last_step_ms", C.c_float), ("reserved", C.c_uint32),
                ("prefill_tokens", C.c_uint64)]


# every symbol include/sllm.h declares; tests check that the library exports all of them
ABI_SYMBOLS = [
    "sllm_default_model_config", "sllm_default_engine_options", "sllm_default_sampling", "sllm_last_error",
    "sllm_engine_create", "sllm_engine_destroy", "sllm_engine_stats", "sllm_engine_stream", "sllm_num_params",
    "sllm_param_info", "sllm_set_param", "sllm_load_checkpoint", "sllm_forward_logits", "sllm_reset",
    "sllm_prefill", "sllm_sample", "sllm_decode_step", "sllm_get_step_logits", "sllm_get_tokens",
    "sllm_set_step_logits", "sllm_force_token", "sllm_truncate", "sllm_generate", "sllm_decode_loop", "sllm_k_attn_decode", "sllm_k_attn_decode_static",
    "sllm_eval_loss", "sllm_slot_assign", "sllm_slot_append", "sllm_slot_release", "sllm_get_finished", "sllm_num_live",
    "sllm_k_wait_probe", "sllm_kv_write", "sllm_kv_read", "sllm_decode_loop_timed",
    "sllm_engine_make_current",
]


def load_library(path: str | None = None):
    """Loads libsllm_b200.so; raises (no fallback) when it has not been built."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    p = path or lib_path()
    if not os.path.exists(p):
        raise FileNotFoundError(f"{p} is missing: build it with `python -m small_llm_b200.build` "
                                "(this package has no CPU or PyTorch fallback)")
    lib = C.CDLL(p)
    E = C.c_void_p
    lib.sllm_default_model_config.argtypes = [C.POINTER(_ModelConfig)]
    lib.sllm_default_engine_options.argtypes = [C.POINTER(_EngineOptions)]
    lib.sllm_default_sampling.argtypes = [C.POINTER(_Sampling)]
    lib.sllm_last_error.restype = C.c_char_p
    lib.sllm_last_error.argtypes = [E]
    lib.sllm_engine_create.argtypes = [C.POINTER(_ModelConfig), C.POINTER(_EngineOptions), C.POINTER(E)]
    lib.sllm_engine_destroy.argtypes = [E]
    lib.sllm_engine_stats.argtypes = [E, C.POINTER(_Stats)]
    lib.sllm_engine_stream.restype = C.c_void_p
    lib.sllm_engine_stream.argtypes = [E]
    lib.sllm_num_params.restype = C.c_uint32
    lib.sllm_num_params.argtypes = [E]
    lib.sllm_param_info.argtypes = [E, C.c_uint32, C.c_char_p, u64p, u32p]
    lib.sllm_set_param.argtypes = [E, C.c_char_p, f32p, u64p, C.c_uint32]
    lib.sllm_load_checkpoint.argtypes = [E, C.c_char_p, u64p, u64p]
    lib.sllm_forward_logits.argtypes = [E, u32p, C.c_uint64, C.c_uint64, f32p]
    lib.sllm_reset.argtypes = [E]
    lib.sllm_prefill.argtypes = [E, u32p, u32p, C.c_uint32]
    lib.sllm_sample.argtypes = [E, C.POINTER(_Sampling), f64p]
    lib.sllm_decode_step.argtypes = [E]
    lib.sllm_get_step_logits.argtypes = [E, C.c_uint32, f32p]
    lib.sllm_set_step_logits.argtypes = [E, C.c_uint32, f32p]
    lib.sllm_get_tokens.argtypes = [E, C.c_uint32, u32p, C.c_uint64, u64p]
    lib.sllm_force_token.argtypes = [E, C.c_uint32, C.c_uint32]
    lib.sllm_truncate.argtypes = [E, C.c_uint32, C.c_uint64]
    lib.sllm_generate.argtypes = [E, u32p, u32p, C.c_uint32, C.c_uint64, C.POINTER(_Sampling), f64p, u32p,
                                  C.c_uint64, u64p]
    lib.sllm_decode_loop.argtypes = [E, C.c_uint64, C.POINTER(_Sampling), f64p]
    i32p = C.POINTER(C.c_int32)
    lib.sllm_slot_assign.argtypes = [E, C.c_uint32, u32p, C.c_uint32]
    lib.sllm_slot_append.argtypes = [E, C.c_uint32, u32p, C.c_uint32]
    lib.sllm_eval_loss.argtypes = [E, u32p, C.POINTER(C.c_int32), C.c_uint64, C.c_uint64, C.c_uint64, C.POINTER(C.c_float)]
    lib.sllm_slot_release.argtypes = [E, C.c_uint32]
    lib.sllm_get_finished.argtypes = [E, i32p, C.c_uint32]
    lib.sllm_k_wait_probe.argtypes = [E, C.c_uint32]
    lib.sllm_engine_make_current.argtypes = [E]
    lib.sllm_decode_loop_timed.argtypes = [E, C.c_uint64, C.POINTER(_Sampling), f64p, f32p]
    lib.sllm_kv_write.argtypes = [E, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, f32p, f32p]
    lib.sllm_kv_read.argtypes = [E, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, f32p, f32p]
    lib.sllm_num_live.restype = C.c_uint32
    lib.sllm_num_live.argtypes = [E]
    for fn in (lib.sllm_k_attn_decode, lib.sllm_k_attn_decode_static):
        fn.argtypes = [E, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
    if path is None:
        _LIB = lib
    return lib


@dataclass
class ModelConfig:
    """include/config.h:6-47 -- same fields and defaults."""
    vocab_size: int = 32768
    context_length: int = 2048
    num_layers: int = 16
    d_model: int = 640
    num_heads: int = 10
    ffn_hidden: int = 1728
    rope_theta: float = 10000.0
    seed: int = 1234
    kRmsNormEps: float = 1e-5

    def head_dim(self) -> int:
        return self.d_model // self.num_heads

    def totalParams(self) -> int:
        per_layer = 4 * self.d_model * self.d_model + 3 * self.d_model * self.ffn_hidden + 2 * self.d_model
        return self.vocab_size * self.d_model + self.num_layers * per_layer + self.d_model


@dataclass
class SamplingOptions:
    """include/inference.h:9-15 -- same fields and defaults."""
    temperature: float = 0.7
    top_p: float = 0.8
    repetition_penalty: float = 1.1
    seed: int = 1234
    stop_token: int = -1


@dataclass
class EngineOptions:
    max_batch: int = 1
    fp32_weights: bool = False
    kv_pages: int = 0
    max_chunk_tokens: int = 0
    device: int = -1
    use_graph: bool = True


@dataclass
class TrainState:
    step: int = 0
    data_position: int = 0


def _raise(code: int, msg: str):
    if code == ERR_INVALID:
        raise ValueError(msg)
    raise SllmError(code, msg)


class Engine:
    """Thin object over the C ABI: one engine = one GPU."""

    def __init__(self, config: ModelConfig, options: EngineOptions | None = None):
        self.lib = load_library()
        self.config = config
        self.options = options or EngineOptions()
        c = _ModelConfig(config.vocab_size, config.context_length, config.num_layers, config.d_model,
                         config.num_heads, config.ffn_hidden, config.rope_theta, config.kRmsNormEps)
        o = _EngineOptions(self.options.max_batch, 1 if self.options.fp32_weights else 0, self.options.kv_pages,
                           self.options.max_chunk_tokens, self.options.device, 1 if self.options.use_graph else 0, 0)
        h = C.c_void_p()
        rc = self.lib.sllm_engine_create(C.byref(c), C.byref(o), C.byref(h))
        if rc:
            _raise(rc, self.lib.sllm_last_error(None).decode())
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.lib.sllm_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc: int):
        if rc:
            _raise(rc, self.lib.sllm_last_error(self.h).decode())

    # ---- weights ------------------------------------------------------------------------------
    def param_infos(self):
        out = []
        for i in range(self.lib.sllm_num_params(self.h)):
            name = C.create_string_buffer(64)
            dims = (C.c_uint64 * 2)()
            nd = C.c_uint32()
            self._ck(self.lib.sllm_param_info(self.h, i, name, dims, C.byref(nd)))
            out.append((name.value.decode(), tuple(int(dims[k]) for k in range(nd.value))))
        return out

    def set_param(self, name: str, value: np.ndarray):
        v = np.ascontiguousarray(value, dtype=np.float32)
        dims = (C.c_uint64 * 2)(*(list(v.shape) + [0])[:2])
        self._ck(self.lib.sllm_set_param(self.h, name.encode(), v.ctypes.data_as(f32p), dims, v.ndim))

    def load_checkpoint(self, path: str) -> TrainState:
        st, dp = C.c_uint64(), C.c_uint64()
        self._ck(self.lib.sllm_load_checkpoint(self.h, path.encode(), C.byref(st), C.byref(dp)))
        return TrainState(st.value, dp.value)

    # ---- model forward ------------------------------------------------------------------------
    def forward_logits(self, ids, B: int, T: int) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
        if ids.size != B * T:
            raise ValueError("Model::forward: token_ids.size() must equal batch_size * seq_len")
        out = np.empty((B, T, self.config.vocab_size), dtype=np.float32)
        self._ck(self.lib.sllm_forward_logits(self.h, ids.ctypes.data_as(u32p), B, T, out.ctypes.data_as(f32p)))
        return out

    # ---- token loop, step by step ---------------------------------------------------------------
    def reset(self):
        self._ck(self.lib.sllm_reset(self.h))

    def prefill(self, prompts):
        lens = np.array([len(p) for p in prompts], dtype=np.uint32)
        ids = np.ascontiguousarray(np.concatenate([np.asarray(p, dtype=np.uint32) for p in prompts]) if len(prompts)
                                   else np.zeros(0, np.uint32))
        self._ck(self.lib.sllm_prefill(self.h, ids.ctypes.data_as(u32p), lens.ctypes.data_as(u32p), len(prompts)))

    def _sampling(self, opt: SamplingOptions, eos: int) -> _Sampling:
        return _Sampling(opt.temperature, opt.top_p, opt.repetition_penalty, eos, opt.stop_token, opt.seed)

    def sample(self, opt: SamplingOptions, draws=None, eos: int = 32762):
        s = self._sampling(opt, eos)
        dp = None
        if draws is not None:
            draws = np.ascontiguousarray(draws, dtype=np.float64)
            dp = draws.ctypes.data_as(f64p)
        self._ck(self.lib.sllm_sample(self.h, C.byref(s), dp))

    def decode_step(self):
        self._ck(self.lib.sllm_decode_step(self.h))

    def step_logits(self, slot: int = 0) -> np.ndarray:
        out = np.empty(self.config.vocab_size, dtype=np.float32)
        self._ck(self.lib.sllm_get_step_logits(self.h, slot, out.ctypes.data_as(f32p)))
        return out

    def set_step_logits(self, slot: int, logits):
        v = np.ascontiguousarray(logits, dtype=np.float32)
        assert v.size == self.config.vocab_size
        self._ck(self.lib.sllm_set_step_logits(self.h, slot, v.ctypes.data_as(f32p)))

    def tokens(self, slot: int = 0) -> np.ndarray:
        cap = 2 * self.config.context_length + 2
        out = np.empty(cap, dtype=np.uint32)
        n = C.c_uint64()
        self._ck(self.lib.sllm_get_tokens(self.h, slot, out.ctypes.data_as(u32p), cap, C.byref(n)))
        return out[: n.value].copy()

    def force_token(self, slot: int, token: int):
        self._ck(self.lib.sllm_force_token(self.h, slot, token))

    def truncate(self, slot: int, n_tokens: int):
        self._ck(self.lib.sllm_truncate(self.h, slot, n_tokens))

    def decode_loop(self, n_steps: int, opt: SamplingOptions, draws=None, eos: int = 32762):
        s = self._sampling(opt, eos)
        dp = None
        if draws is not None:
            draws = np.ascontiguousarray(draws, dtype=np.float64)
            dp = draws.ctypes.data_as(f64p)
        self._ck(self.lib.sllm_decode_loop(self.h, n_steps, C.byref(s), dp))

    def decode_loop_timed(self, n_steps: int, opt: SamplingOptions, draws=None, eos: int = 32762) -> np.ndarray:
        """decode_loop with a CUDA event per iteration; returns the device time of every iteration in ms."""
        s = self._sampling(opt, eos)
        dp = None
        if draws is not None:
            draws = np.ascontiguousarray(draws, dtype=np.float64)
            dp = draws.ctypes.data_as(f64p)
        out = np.zeros(n_steps, dtype=np.float32)
        self._ck(self.lib.sllm_decode_loop_timed(self.h, n_steps, C.byref(s), dp, out.ctypes.data_as(f32p)))
        return out

    # ---- token loop in one call -------------------------------------------------------------------
    def generate(self, prompts, max_new: int, opt: SamplingOptions, draws=None, eos: int = 32762):
        """prompts: list of id sequences.  draws: [max_new][n_seq] float64 or None (seeded mode).
        Returns a list of uint32 arrays (prompt + continuation)."""
        n = len(prompts)
        lens = np.array([len(p) for p in prompts], dtype=np.uint32)
        ids = np.ascontiguousarray(np.concatenate([np.asarray(p, dtype=np.uint32) for p in prompts]) if n
                                   else np.zeros(0, np.uint32))
        stride = 2 * self.config.context_length + 2
        out = np.empty((max(n, 1), stride), dtype=np.uint32)
        out_lens = np.zeros(max(n, 1), dtype=np.uint64)
        s = self._sampling(opt, eos)
        dp = None
        if draws is not None:
            draws = np.ascontiguousarray(draws, dtype=np.float64)
            assert draws.size >= max_new * n
            dp = draws.ctypes.data_as(f64p)
        self._ck(self.lib.sllm_generate(self.h, ids.ctypes.data_as(u32p), lens.ctypes.data_as(u32p), n, max_new,
                                        C.byref(s), dp, out.ctypes.data_as(u32p), stride,
                                        out_lens.ctypes.data_as(u64p)))
        return [out[i, : int(out_lens[i])].copy() for i in range(n)]

    def slot_assign(self, slot: int, ids):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        self._ck(self.lib.sllm_slot_assign(self.h, slot, ids.ctypes.data_as(u32p), ids.size))

    def eval_loss(self, ids, targets, B: int, T: int, num_valid: int = 0) -> float:
        """ops::cross_entropy of the model's logits against targets [B*T] (negative = ignored), computed on the device."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
        targets = np.ascontiguousarray(targets, dtype=np.int32).reshape(-1)
        assert ids.size == B * T == targets.size
        out = C.c_float()
        self._ck(self.lib.sllm_eval_loss(self.h, ids.ctypes.data_as(u32p), targets.ctypes.data_as(C.POINTER(C.c_int32)),
                                         B, T, num_valid, C.byref(out)))
        return float(out.value)

    def slot_append(self, slot: int, ids):
        """Appends ids behind a live slot's tokens; only they run through the model (KV reuse across turns)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        self._ck(self.lib.sllm_slot_append(self.h, slot, ids.ctypes.data_as(u32p), ids.size))

    def slot_release(self, slot: int):
        self._ck(self.lib.sllm_slot_release(self.h, slot))

    def num_live(self) -> int:
        """Column count of the draw matrix sllm_decode_loop reads: highest slot that holds a sequence, plus one."""
        return int(self.lib.sllm_num_live(self.h))

    def finished(self, n: int) -> np.ndarray:
        out = np.zeros(n, dtype=np.int32)
        self._ck(self.lib.sllm_get_finished(self.h, out.ctypes.data_as(C.POINTER(C.c_int32)), n))
        return out

    def k_attn_decode(self, layer: int, n_tok: int, d_q: int, d_tok_slot: int, d_tok_pos: int, n_splits: int,
                      d_out: int, stream: int = 0, static_scratch: bool = False):
        """Launches the flash-decode attention kernel alone; every d_* is a device address."""
        fn = self.lib.sllm_k_attn_decode_static if static_scratch else self.lib.sllm_k_attn_decode
        self._ck(fn(self.h, layer, n_tok, d_q, d_tok_slot, d_tok_pos, n_splits, d_out, stream or None))

    def kv_write(self, layer: int, slot: int, pos0: int, k_rows, v_rows):
        """K / V rows [n_pos][d_model] fp32 into the slot's cache at positions pos0.. of `layer`."""
        k = np.ascontiguousarray(k_rows, dtype=np.float32)
        v = np.ascontiguousarray(v_rows, dtype=np.float32)
        assert k.shape == v.shape and k.shape[1] == self.config.d_model
        self._ck(self.lib.sllm_kv_write(self.h, layer, slot, pos0, k.shape[0], k.ctypes.data_as(f32p), v.ctypes.data_as(f32p)))

    def kv_read(self, layer: int, slot: int, pos0: int, n_pos: int):
        k = np.empty((n_pos, self.config.d_model), dtype=np.float32)
        v = np.empty_like(k)
        self._ck(self.lib.sllm_kv_read(self.h, layer, slot, pos0, n_pos, k.ctypes.data_as(f32p), v.ctypes.data_as(f32p)))
        return k, v

    def wait_probe(self, limit_us: int):
        """Diagnostic: one device thread waits limit_us on a barrier nobody arrives at; raises SllmError(ERR_DEVICE_WAIT)."""
        self._ck(self.lib.sllm_k_wait_probe(self.h, limit_us))

    def stats(self) -> dict:
        s = _Stats()
        self._ck(self.lib.sllm_engine_stats(self.h, C.byref(s)))
        return {k: getattr(s, k) for k, _ in _Stats._fields_}

    def stream(self) -> int:
        return int(self.lib.sllm_engine_stream(self.h) or 0)


class Model:
    """Model of include/model.h:23-50, inference half: construction allocates on the GPU
    (the reference's Model(cfg) + to(CUDA) + enable_bf16(true)); weights arrive through
    load_checkpoint_weights or set_parameter."""

    def __init__(self, config: ModelConfig, options: EngineOptions | None = None):
        self._config = config
        self.engine = Engine(config, options)

    def config(self) -> ModelConfig:
        return self._config

    def bf16(self) -> bool:
        return not self.engine.options.fp32_weights

    def parameters(self):
        """Registry order and names of src/model.cpp:106-131 as (name, shape) pairs."""
        return self.engine.param_infos()

    def set_parameter(self, name: str, value: np.ndarray):
        self.engine.set_param(name, value)

    def forward(self, token_ids, batch_size: int, seq_len: int) -> np.ndarray:
        """src/model.cpp:31-62: ids [B*T] -> logits [B,T,vocab] fp32."""
        ids = np.asarray(token_ids, dtype=np.uint32).reshape(-1)
        if ids.size != batch_size * seq_len:
            raise ValueError("Model::forward: token_ids.size() must equal batch_size * seq_len")
        if seq_len > self._config.context_length:
            raise ValueError("Model::forward: seq_len exceeds context_length")
        return self.engine.forward_logits(ids, batch_size, seq_len)


def load_checkpoint_weights(path: str, model: Model) -> TrainState:
    """src/checkpoint.cpp:57-102."""
    return model.engine.load_checkpoint(path)


class Inference:
    """Inference of include/inference.h:17-27 over token ids.

    generateTokens returns the ids (prompt + continuation) instead of decoded text: the tokenizer is
    outside this path.  With temperature <= 0 the reference computes the argmax but never appends it
    (src/inference.cpp:90-95,158-163); this class appends it, which is the evident intent.
    """

    def __init__(self, model: Model, eos_token: int = 32762):
        self.model = model
        self.eos = eos_token

    def generateTokens(self, tokens, max_new_tokens: int, opt: SamplingOptions | None = None, draws=None):
        opt = opt or SamplingOptions()
        tokens = np.asarray(tokens, dtype=np.uint32)
        if tokens.size == 0:
            raise ValueError("Inference::generate: prompt encoded to zero tokens")
        return self.model.engine.generate([tokens], max_new_tokens, opt, draws, self.eos)[0]
