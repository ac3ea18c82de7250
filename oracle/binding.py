"""ctypes bindings for the CPU oracle libraries -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Two libraries, same role (the checker, never the thing shipped or measured as the product):

* ``OracleModel``  -> oracle/libsllm_oracle.so, this repository's C restatement of the reference's
  CPU algorithm (sllm_oracle.c).  Always buildable (gcc only).
* ``RefModel``     -> oracle/_ref/libsllm_ref.so, the UNMODIFIED reference sources compiled behind
  ref_shim.cpp.  Present only where the reference tree was available at build time.

Only tests, the smoke check and the benchmark's cpu_baseline / reference legs import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libsllm_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libsllm_ref.so")
REF_FAST_SO = os.path.join(HERE, "_ref", "libsllm_ref_fast.so")
# Root of the small-llm tree: $SLLM_REF_DIR, else a checkout named "reference" beside this repository; empty when
# neither exists (then the reference build is skipped and only its committed golden vectors are used).
_SIBLING = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
REF_TREE = os.environ.get("SLLM_REF_DIR") or (_SIBLING if os.path.isdir(os.path.join(_SIBLING, "src")) else "")

u32p = C.POINTER(C.c_uint32)
u64p = C.POINTER(C.c_uint64)
f32p = C.POINTER(C.c_float)
f64p = C.POINTER(C.c_double)


def _ptr(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "sllm_oracle.c")
    if force or not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "oracle"], check=True, capture_output=True)
    return ORACLE_SO


def build_ref(force: bool = False) -> str | None:
    """Compile the reference's own sources where they lie; None when the tree is absent."""
    if REF_TREE and os.path.isdir(os.path.join(REF_TREE, "src")):
        shim = os.path.join(HERE, "ref_shim.cpp")
        if force or not os.path.exists(REF_SO) or os.path.getmtime(REF_SO) < os.path.getmtime(shim):
            subprocess.run(["make", "-C", HERE, "ref", f"REF={REF_TREE}"], check=True, capture_output=True)
    return REF_SO if os.path.exists(REF_SO) else None


def ref_available() -> bool:
    return os.path.exists(REF_SO)


@dataclass(frozen=True)
class Config:
    vocab: int = 32768
    context: int = 2048
    layers: int = 16
    d_model: int = 640
    heads: int = 10
    ffn: int = 1728
    theta: float = 10000.0
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.d_model // self.heads

    def as_u64(self) -> np.ndarray:
        return np.array([self.vocab, self.context, self.layers, self.d_model, self.heads, self.ffn], dtype=np.uint64)


class _OrcConfig(C.Structure):
    _fields_ = [("vocab", C.c_uint64), ("context", C.c_uint64), ("layers", C.c_uint64),
                ("d_model", C.c_uint64), ("heads", C.c_uint64), ("ffn", C.c_uint64),
                ("theta", C.c_float), ("eps", C.c_float)]


class _OrcSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("repetition_penalty", C.c_float),
                ("stop_token", C.c_int64), ("eos_token", C.c_uint32)]


_orc = None


def orc():
    global _orc
    if _orc is None:
        lib = C.CDLL(build_oracle())
        lib.orc_last_error.restype = C.c_char_p
        lib.orc_model_create.restype = C.c_void_p
        lib.orc_model_create.argtypes = [C.POINTER(_OrcConfig)]
        lib.orc_model_destroy.argtypes = [C.c_void_p]
        lib.orc_num_params.restype = C.c_uint32
        lib.orc_num_params.argtypes = [C.c_void_p]
        lib.orc_param.restype = f32p
        lib.orc_param.argtypes = [C.c_void_p, C.c_uint32, C.c_char_p, u64p, u32p]
        lib.orc_init_normal.argtypes = [C.c_void_p, C.c_uint32, C.c_float]
        lib.orc_save_checkpoint.argtypes = [C.c_void_p, C.c_char_p, C.c_uint64, C.c_uint64]
        lib.orc_load_checkpoint.argtypes = [C.c_void_p, C.c_char_p, u64p, u64p]
        lib.orc_forward.argtypes = [C.c_void_p, u32p, C.c_uint64, C.c_uint64, C.c_uint64, f32p]
        lib.orc_session_create.restype = C.c_void_p
        lib.orc_session_create.argtypes = [C.c_void_p]
        lib.orc_session_destroy.argtypes = [C.c_void_p]
        lib.orc_session_reset.argtypes = [C.c_void_p]
        lib.orc_session_len.restype = C.c_uint64
        lib.orc_session_len.argtypes = [C.c_void_p]
        lib.orc_session_feed.argtypes = [C.c_void_p, u32p, C.c_uint64, f32p, f32p]
        lib.orc_sample.restype = C.c_int64
        lib.orc_sample.argtypes = [f32p, C.c_uint64, u32p, C.c_uint64, C.c_float, C.c_float, C.c_float,
                                   C.c_double, f64p]
        lib.orc_greedy.restype = C.c_int64
        lib.orc_greedy.argtypes = [f32p, C.c_uint64, u32p, C.c_uint64, C.c_float, f32p]
        lib.orc_generate.argtypes = [C.c_void_p, u32p, C.c_uint64, C.c_uint64, C.POINTER(_OrcSampling),
                                     f32p, u32p, u64p]
        lib.orc_generate_seeded.argtypes = [C.c_void_p, u32p, C.c_uint64, C.c_uint64,
                                            C.POINTER(_OrcSampling), C.c_uint64, u32p, u64p]
        lib.orc_prompt_ids.argtypes = [C.c_uint32, C.c_uint64, C.c_uint32, u32p]
        lib.orc_uniforms.argtypes = [C.c_uint32, C.c_uint64, f32p]
        lib.orc_canonical64.argtypes = [C.c_uint64, C.c_uint64, f64p]
        lib.orc_cross_entropy.argtypes = [f32p, C.POINTER(C.c_int32), C.c_uint64, C.c_uint64, C.c_uint64]
        lib.orc_cross_entropy.restype = C.c_float
        _orc = lib
    return _orc


def prompt_ids(seed: int, n: int, vocab: int = 32768) -> np.ndarray:
    """ids = std::mt19937(seed)() & (vocab-1); vocab must be a power of two."""
    assert vocab & (vocab - 1) == 0
    out = np.empty(n, dtype=np.uint32)
    orc().orc_prompt_ids(seed, n, vocab - 1, _ptr(out, u32p))
    return out


def uniforms(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    orc().orc_uniforms(seed, n, _ptr(out, f32p))
    return out


def cross_entropy(logits: np.ndarray, targets: np.ndarray, num_valid: int = 0) -> float:
    """ops::cross_entropy restated: logits [n, V] fp32, targets [n] (negative = ignored position)."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    V = logits.shape[-1]
    targets = np.ascontiguousarray(targets, dtype=np.int32).reshape(-1)
    assert logits.size == targets.size * V
    return float(orc().orc_cross_entropy(_ptr(logits, f32p), targets.ctypes.data_as(C.POINTER(C.c_int32)), targets.size, V, num_valid))


def canonical64(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float64)
    orc().orc_canonical64(seed, n, _ptr(out, f64p))
    return out


def sample(logits: np.ndarray, history: np.ndarray, temperature: float, top_p: float, penalty: float,
           u: float) -> tuple[int, float]:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    history = np.ascontiguousarray(history, dtype=np.uint32)
    mg = C.c_double(0)
    tok = orc().orc_sample(_ptr(logits, f32p), logits.size, _ptr(history, u32p), history.size,
                           temperature, top_p, penalty, float(u), C.byref(mg))
    return int(tok), float(mg.value)


def greedy(logits: np.ndarray, history: np.ndarray, penalty: float = 1.0) -> tuple[int, float]:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    history = np.ascontiguousarray(history, dtype=np.uint32)
    mg = C.c_float(0)
    tok = orc().orc_greedy(_ptr(logits, f32p), logits.size, _ptr(history, u32p), history.size, penalty,
                           C.byref(mg))
    return int(tok), float(mg.value)


class OracleModel:
    """The C restatement (sllm_oracle.c)."""

    def __init__(self, cfg: Config):
        self.cfg = cfg
        self.lib = orc()
        c = _OrcConfig(cfg.vocab, cfg.context, cfg.layers, cfg.d_model, cfg.heads, cfg.ffn, cfg.theta, cfg.eps)
        self.h = self.lib.orc_model_create(C.byref(c))
        if not self.h:
            raise ValueError(self.lib.orc_last_error().decode())

    def close(self):
        if self.h:
            self.lib.orc_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc:
            raise RuntimeError(self.lib.orc_last_error().decode())

    def num_params(self) -> int:
        return self.lib.orc_num_params(self.h)

    def param(self, i: int) -> tuple[str, np.ndarray]:
        name = C.create_string_buffer(64)
        dims = (C.c_uint64 * 2)()
        nd = C.c_uint32()
        p = self.lib.orc_param(self.h, i, name, dims, C.byref(nd))
        shape = tuple(int(dims[k]) for k in range(nd.value))
        arr = np.ctypeslib.as_array(p, shape=shape)      # view into the model's storage
        return name.value.decode(), arr

    def params(self):
        return [self.param(i) for i in range(self.num_params())]

    def init_normal(self, seed: int, stddev: float = 0.02):
        self.lib.orc_init_normal(self.h, seed, stddev)

    def save_checkpoint(self, path: str, step: int = 0, data_pos: int = 0):
        self._check(self.lib.orc_save_checkpoint(self.h, path.encode(), step, data_pos))

    def load_checkpoint(self, path: str) -> tuple[int, int]:
        st, dp = C.c_uint64(), C.c_uint64()
        self._check(self.lib.orc_load_checkpoint(self.h, path.encode(), C.byref(st), C.byref(dp)))
        return st.value, dp.value

    def forward(self, ids: np.ndarray, B: int, T: int, row_from: int = 0) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
        assert ids.size == B * T
        out = np.empty((B, T - row_from, self.cfg.vocab), dtype=np.float32)
        self._check(self.lib.orc_forward(self.h, _ptr(ids, u32p), B, T, row_from, _ptr(out, f32p)))
        return out

    def generate(self, prompt, max_new, temperature, top_p, penalty, us=None, eos=32762, stop=-1,
                 seed=None) -> np.ndarray:
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.empty(prompt.size + max_new, dtype=np.uint32)
        n = C.c_uint64()
        opt = _OrcSampling(temperature, top_p, penalty, stop, eos)
        if seed is not None:
            rc = self.lib.orc_generate_seeded(self.h, _ptr(prompt, u32p), prompt.size, max_new, C.byref(opt),
                                              seed, _ptr(out, u32p), C.byref(n))
        else:
            up = None
            if us is not None:
                us = np.ascontiguousarray(us, dtype=np.float32)
                up = _ptr(us, f32p)
            rc = self.lib.orc_generate(self.h, _ptr(prompt, u32p), prompt.size, max_new, C.byref(opt), up,
                                       _ptr(out, u32p), C.byref(n))
        self._check(rc)
        return out[: n.value].copy()


class OracleSession:
    def __init__(self, model: OracleModel):
        self.m = model
        self.h = model.lib.orc_session_create(model.h)

    def close(self):
        if self.h:
            self.m.lib.orc_session_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset(self):
        self.m.lib.orc_session_reset(self.h)

    def feed(self, ids, all_rows: bool = False) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
        V = self.m.cfg.vocab
        if all_rows:
            out = np.empty((ids.size, V), dtype=np.float32)
            rc = self.m.lib.orc_session_feed(self.h, _ptr(ids, u32p), ids.size, None, _ptr(out, f32p))
        else:
            out = np.empty(V, dtype=np.float32)
            rc = self.m.lib.orc_session_feed(self.h, _ptr(ids, u32p), ids.size, _ptr(out, f32p), None)
        self.m._check(rc)
        return out


class RefModel:
    """The unmodified reference behind ref_shim.cpp (parity build by default)."""

    def __init__(self, cfg: Config, fast: bool = False, ctor_seed: int | None = None):
        """ctor_seed: Tensor::seed(ctor_seed) before Model::Model, i.e. the reference's own initial weights."""
        path = REF_FAST_SO if fast else REF_SO
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        lib = C.CDLL(path)
        lib.ref_last_error.restype = C.c_char_p
        lib.ref_model_create.restype = C.c_void_p
        lib.ref_model_create.argtypes = [u64p, C.c_float, C.c_float]
        lib.ref_model_destroy.argtypes = [C.c_void_p]
        lib.ref_model_init_normal.argtypes = [C.c_void_p, C.c_uint32, C.c_float]
        lib.ref_model_num_params.restype = C.c_uint32
        lib.ref_model_num_params.argtypes = [C.c_void_p]
        lib.ref_model_param.restype = f32p
        lib.ref_model_param.argtypes = [C.c_void_p, C.c_uint32, C.c_char_p, u64p, u32p]
        lib.ref_model_load_weights.argtypes = [C.c_void_p, C.c_char_p, u64p, u64p]
        lib.ref_model_forward.argtypes = [C.c_void_p, u32p, C.c_uint64, C.c_uint64, f32p]
        lib.ref_generate_tokens.argtypes = [C.c_void_p, u32p, C.c_uint64, C.c_uint64, C.c_float, C.c_float,
                                            C.c_float, C.c_uint64, C.c_int64, C.c_int, u32p, u64p]
        for name, nargs in (("ref_op_rmsnorm", None),):
            pass
        lib.ref_op_rmsnorm.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64, C.c_float, f32p]
        lib.ref_op_matmul.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, f32p]
        lib.ref_op_matmul_bt.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, f32p]
        lib.ref_op_rope.argtypes = [f32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, f32p]
        lib.ref_op_attention.argtypes = [f32p, f32p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, f32p]
        lib.ref_op_silu_mul.argtypes = [f32p, f32p, C.c_uint64, f32p]
        lib.ref_op_cross_entropy.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, C.POINTER(C.c_float)]
        self.lib = lib
        self.cfg = cfg
        c = cfg.as_u64()
        if ctor_seed is None:
            self.h = lib.ref_model_create(_ptr(c, u64p), cfg.theta, cfg.eps)
        else:
            lib.ref_model_create_seeded.restype = C.c_void_p
            lib.ref_model_create_seeded.argtypes = [u64p, C.c_float, C.c_float, C.c_uint32]
            self.h = lib.ref_model_create_seeded(_ptr(c, u64p), cfg.theta, cfg.eps, ctor_seed)
        if not self.h:
            raise ValueError(lib.ref_last_error().decode())

    def close(self):
        if self.h:
            self.lib.ref_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def init_normal(self, seed: int, stddev: float = 0.02):
        self._check(self.lib.ref_model_init_normal(self.h, seed, stddev))

    def num_params(self) -> int:
        return self.lib.ref_model_num_params(self.h)

    def param(self, i: int) -> tuple[str, np.ndarray]:
        name = C.create_string_buffer(64)
        dims = (C.c_uint64 * 4)()
        nd = C.c_uint32()
        p = self.lib.ref_model_param(self.h, i, name, dims, C.byref(nd))
        shape = tuple(int(dims[k]) for k in range(nd.value))
        return name.value.decode(), np.ctypeslib.as_array(p, shape=shape)

    def params(self):
        return [self.param(i) for i in range(self.num_params())]

    def load_checkpoint(self, path: str) -> tuple[int, int]:
        st, dp = C.c_uint64(), C.c_uint64()
        self._check(self.lib.ref_model_load_weights(self.h, path.encode(), C.byref(st), C.byref(dp)))
        return st.value, dp.value

    def forward(self, ids: np.ndarray, B: int, T: int) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
        out = np.empty((B, T, self.cfg.vocab), dtype=np.float32)
        self._check(self.lib.ref_model_forward(self.h, _ptr(ids, u32p), B, T, _ptr(out, f32p)))
        return out

    def cross_entropy(self, logits: np.ndarray, targets: np.ndarray, num_valid: int = 0) -> float:
        """The reference's ops::cross_entropy on host logits [n, V]; targets as it stores them (ids as floats)."""
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        V = logits.shape[-1]
        t = np.ascontiguousarray(targets, dtype=np.float32).reshape(-1)
        out = C.c_float()
        self._check(self.lib.ref_op_cross_entropy(_ptr(logits, f32p), _ptr(t, f32p), t.size, V, num_valid, C.byref(out)))
        return float(out.value)

    def generate_tokens(self, prompt, max_new, temperature, top_p, penalty, seed, stop=-1,
                        eos_merges=32506) -> np.ndarray:
        """The reference's Inference::generateTokens, unmodified (own mt19937_64 draws)."""
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.empty(prompt.size + max_new + 1, dtype=np.uint32)
        n = C.c_uint64()
        self._check(self.lib.ref_generate_tokens(self.h, _ptr(prompt, u32p), prompt.size, max_new, temperature,
                                                 top_p, penalty, seed, stop, eos_merges, _ptr(out, u32p),
                                                 C.byref(n)))
        return out[: n.value].copy()
