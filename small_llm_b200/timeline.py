"""Per-phase timeline of the batch-1 decode step, from in-kernel `globaltimer` stamps.

    python -m small_llm_b200.timeline [--tokens 40] [--prompt 256]

Builds a debug copy of the library with -DSLLM_TIMELINE (libsllm_b200_timeline.so, beside the normal one; the normal
build carries no stamps), runs the 100.3M model's sampled batch-1 decode (the benchmark's config 2) on the current GPU
and prints, for block 0 of the persistent decode kernel and of the sampler kernels, the median time between
consecutive stamps.  A stamp is two plain stores by one thread (the persistent kernel reserves its entries once per
launch), so the figures are within a few percent of the unstamped run; compare the token period printed last with
`bench.py --workload c2`.
"""
from __future__ import annotations

import argparse
import collections
import ctypes as C
import os
import subprocess

import numpy as np

from . import api, build

LABELS = {
    (401, 412): "dependency wait -> embedding row, first 1/rms",
    (425, 412): "x gather + gain product + 1/rms            (hand-off 1)",
    (412, 413): "QKV rows, RoPE, K/V append, publish",
    (413, 414): "q|k|v gather of the head                   (hand-off 2)",
    (414, 4141): "attention: scores of the warp's keys",
    (4141, 4142): "attention: softmax weights",
    (4142, 4143): "attention: value product",
    (4143, 4144): "attention: block barrier",
    (4144, 416): "attention: combine the 16 warps, publish",
    (416, 417): "partials gather                            (hand-off 3)",
    (417, 4171): "merge: weight per (head, key range)",
    (4171, 4172): "merge: block barrier",
    (4172, 4173): "merge: weighted sum",
    (4173, 418): "merge: block barrier",
    (418, 419): "out-projection rows, residual, publish",
    (419, 421): "x gather + gain product + 1/rms            (hand-off 4)",
    (421, 422): "gate/up rows, SiLU, publish",
    (422, 424): "hidden-unit gather                         (hand-off 5)",
    (424, 425): "down-projection rows, residual, publish",
    (425, 430): "final x gather + 1/rms",
    (430, 431): "tied head: vocabulary rows streamed through shared memory",
    (431, 432): "folded sampler kernels: penalised maxima, hand-off, weights, level-0 histogram",
    (430, 432): "tied head (no folded sampler work in this launch)",
    (432, 320): "kernel boundary -> k_samp_pick",
    (432, 300): "kernel boundary -> k_samp_max",
    (300, 310): "k_samp_max -> k_samp_hist",
    (320, 3201): "k_samp_pick: weights + level-0 histogram requested and stored",
    (3201, 3202): "k_samp_pick: block barrier, the slot's maximum",
    (3202, 322): "k_samp_pick: scan of the level-0 histogram",
    (322, 323): "k_samp_pick: top-p cut",
    (323, 324): "k_samp_pick: the draw",
    (324, 325): "k_samp_pick: token",
    (325, 321): "k_samp_pick: append, stop rules",
    (321, 401): "kernel boundary -> persistent kernel past its dependency wait",
}


def build_debug_library() -> str:
    lib = os.path.join(build.HERE, "libsllm_b200_timeline.so")
    srcs = [s for s in build.sources() if s.endswith(".cu")]
    if not os.path.exists(lib) or any(os.path.getmtime(s) > os.path.getmtime(lib) for s in build.sources()):
        nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
        subprocess.run([nvcc, *build.NVCC_FLAGS, "-DSLLM_TIMELINE", "-o", lib, *srcs], check=True)
    return lib


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=40)
    ap.add_argument("--prompt", type=int, default=256)
    args = ap.parse_args()
    lib = api.load_library(build_debug_library())
    api._LIB = lib
    lib.sllm_debug_timeline.argtypes = [C.POINTER(C.c_ulonglong), C.c_uint, C.POINTER(C.c_uint)]
    from .api import Engine, EngineOptions, ModelConfig, SamplingOptions
    eng = Engine(ModelConfig(), EngineOptions(max_batch=1))
    rng = np.random.default_rng(0)
    for name, shape in eng.param_infos():
        eng.set_param(name, rng.normal(0, 0.02, size=shape).astype(np.float32) if len(shape) == 2 else np.ones(shape, np.float32))
    prompt = rng.integers(0, 32768, size=args.prompt).astype(np.uint32)
    draws = rng.random((args.tokens, 1))
    opt = SamplingOptions(temperature=0.8, top_p=0.95, repetition_penalty=1.15)
    eng.prefill([prompt])

    def grab():
        buf = (C.c_ulonglong * (2 * 32768))()
        n = C.c_uint(0)
        lib.sllm_debug_timeline(buf, 32768, C.byref(n))
        return np.array([(int(buf[2 * i]), int(buf[2 * i + 1])) for i in range(n.value)], dtype=np.int64).reshape(-1, 2)

    eng.decode_loop(args.tokens, opt, draws, eos=1 << 30)         # warm-up: graphs captured, caches warm
    grab()
    eng.truncate(0, args.prompt)
    eng.decode_step()
    grab()
    eng.decode_loop(args.tokens, opt, draws, eos=1 << 30)
    tl = grab()
    tl = tl[tl[:, 0] != 0]
    tl = tl[np.argsort(tl[:, 1], kind="stable")]
    deltas = collections.defaultdict(list)
    for (a, ta), (b, tb) in zip(tl[:-1], tl[1:]):
        deltas[(int(a), int(b))].append(int(tb - ta))
    print(f"{len(tl)} stamps over {args.tokens} tokens at context {args.prompt}..{args.prompt + args.tokens}")
    for key, label in LABELS.items():
        if key in deltas:
            v = np.array(deltas[key])
            print(f"  {label:62s} n={len(v):5d}  median {np.median(v) / 1000:6.2f} us")
    starts = tl[tl[:, 0] == 400, 1]
    if len(starts) > 2:
        print(f"token period: {np.median(np.diff(starts)) / 1000:.1f} us")


if __name__ == "__main__":
    main()
