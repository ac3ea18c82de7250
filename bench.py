#!/usr/bin/env python
"""Benchmark of the token loop on B200: decode tokens/s against the HBM roofline.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5] [--impl reference]

Default workload (N=1): BASELINE config 2 -- the 100.3M model, batch 1, a prompt of 256 uniform
random ids, 512 sampled decode steps (temperature 0.8, top-p 0.95, repetition penalty 1.15,
per-step uniform draws generated on the host from seed 2).  One benchmark "step" is one such
generation of 512 tokens from the prefilled prompt: the slot is rewound to the prompt, the last
prompt position is recomputed (so the sampler has fresh logits) and 512 x (sampler + model pass) run
on the device as CUDA-graph replays.  With N GPUs every rank runs its own sequence(s) (independent
units, sharded by batch, no collective in the loop: weak scaling); finished token streams are
gathered to rank 0 with NCCL after the timed region.

Weights are random-init N(0, 0.02) (numpy seed 0; gains 1) -- there are no trained checkpoints
offline -- and the prompt/draw streams are the std::mt19937 streams the parity tests use.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_PROMPT, N_NEW = 256, 512
SAMPLING = dict(temperature=0.8, top_p=0.95, repetition_penalty=1.15)
EOS_NEVER = 1 << 30            # a sequence must run its full 512 steps to be comparable
METRIC = "decode tok/s at batch 1 (1 B200) vs HBM roofline; p50 per-token ms"
WORKLOAD = ("BASELINE config 2: 100.3M model, batch 1 per GPU, prompt 256, 512 sampled decode steps "
            "(T 0.8, top-p 0.95, penalty 1.15, host draws)")


def mt19937_raw(seed: int, n: int) -> np.ndarray:
    """Raw 32-bit outputs of std::mt19937(seed)."""
    bg = np.random.MT19937()
    bg._legacy_seeding(seed)
    return bg.random_raw(n).astype(np.uint32)


def prompt_ids(seed: int, n: int, vocab: int = 32768) -> np.ndarray:
    return mt19937_raw(seed, n) & np.uint32(vocab - 1)


def uniform_draws(seed: int, n: int) -> np.ndarray:
    return (mt19937_raw(seed, n) >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -24)


def peaks() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.stop = index, [], threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                for line in out.strip().splitlines():
                    self.rows.append([c.strip() for c in line.split(",")])
            except Exception:
                pass
            self.stop.wait(0.2)

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.thread.join(timeout=6)

    def summary(self) -> dict:
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def algorithmic_bytes_per_token(cfg, ctx_mean: float, wbytes: int = 2) -> float:
    """Weights streamed once (tied head included) + norm gains + KV read up to the context + one
    position written."""
    D, F, V, L = cfg.d_model, cfg.ffn_hidden, cfg.vocab_size, cfg.num_layers
    p_mat = L * (4 * D * D + 3 * D * F) + V * D
    p_norm = (2 * L + 1) * D
    kv_per_pos = 2 * L * D * wbytes
    return wbytes * p_mat + 4 * p_norm + kv_per_pos * (ctx_mean + 1)


# ------------------------------------------------------------------------------- our arm ---
def run_ours(args):
    import torch
    import torch.distributed as dist

    from small_llm_b200 import Engine, EngineOptions, ModelConfig, SamplingOptions, build

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            sys.exit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()

    cfg = ModelConfig()
    eng = Engine(cfg, EngineOptions(max_batch=1, device=local))
    rng = np.random.default_rng(0)
    for name, shape in eng.param_infos():
        if len(shape) == 2:
            eng.set_param(name, rng.normal(0.0, 0.02, size=shape).astype(np.float32))
        else:
            eng.set_param(name, np.ones(shape, np.float32))
    prompt = prompt_ids(1 + 1000 * rank, N_PROMPT)           # rank r owns sequence r
    draws = uniform_draws(2 + 1000 * rank, N_NEW).astype(np.float64).reshape(-1, 1)
    opt = SamplingOptions(**SAMPLING)
    stream = torch.cuda.ExternalStream(eng.stream(), device=torch.device("cuda", local))

    def one_generation():
        eng.truncate(0, N_PROMPT)
        eng.decode_step()
        eng.decode_loop(N_NEW, opt, draws, eos=EOS_NEVER)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    eng.prefill([prompt])
    n_warm = args.warmup if args.profile_only else max(args.warmup, 3)
    for _ in range(n_warm):
        one_generation()
    launches0 = eng.stats()["launches"]
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        ev0.record(stream)
        marks = []
        for _ in range(args.steps):
            one_generation()
            marks.append(torch.cuda.Event(enable_timing=True))
            marks[-1].record(stream)                              # one event per generation of N_NEW tokens
        ev1.record(stream)
        ev1.synchronize()
        barrier()
    ms = ev0.elapsed_time(ev1)
    gen_ms = [a.elapsed_time(b) for a, b in zip([ev0] + marks[:-1], marks)]
    p50_token_ms = statistics.median(gen_ms) / N_NEW                  # median over the generations of their mean step time
    launches = eng.stats()["launches"] - launches0
    n_tok = eng.tokens(0).size - N_PROMPT
    assert n_tok == N_NEW, f"sequence produced {n_tok} tokens"

    # end to end through the C ABI with host buffers: H2D prompt + draws, prefill, decode, D2H tokens
    e2e_steps = max(1, min(args.steps, 5))
    eng.generate([prompt], N_NEW, opt, draws, eos=EOS_NEVER)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        out = eng.generate([prompt], N_NEW, opt, draws, eos=EOS_NEVER)[0]
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps

    t_ms = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
        # the path's only exchange: finished token streams to rank 0 (NCCL)
        from small_llm_b200.shard import gather_streams
        streams = gather_streams([out], world, N_PROMPT + N_NEW + 1, device=torch.device("cuda", local))
        assert rank != 0 or (len(streams) == world and all(len(x) == N_PROMPT + N_NEW for x in streams))
    ms, e2e_ms = float(t_ms[0]), float(t_ms[1])

    if rank == 0:
        peak, peak_kind = peaks()
        tokens = world * args.steps * N_NEW
        value = tokens / (ms * 1e-3)
        step_ms = ms / (args.steps * N_NEW)                       # one token step (graph replay)
        ctx_mean = N_PROMPT + (N_NEW - 1) / 2.0
        bytes_tok = algorithmic_bytes_per_token(cfg, ctx_mean)
        achieved = bytes_tok / (step_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC,
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": n_warm,
            "ms_per_step": ms / args.steps, "per_token_ms": step_ms, "per_token_ms_p50": p50_token_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: N(0,0.02) weights (numpy seed 0), std::mt19937 prompt ids and draws",
            "config": {"workload": WORKLOAD,
                       "sequences_per_gpu": 1, "precision": "bf16 weights and KV cache, fp32 residual stream and accumulation",
                       "l2": "inputs larger than L2 (200.6 MB of weights streamed per token)"},
            "e2e": {"value": world * N_NEW / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(N_PROMPT * 4 + N_NEW * 8), "d2h_bytes_per_step": int((N_PROMPT + N_NEW + 1) * 4),
                    "note": "sllm_generate with host buffers: prompt upload, prefill of 256 ids, 512 decode steps, token download"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm",
                         "kernel": "one decode step = one CUDA-graph replay: 3 sampler kernels + 16 x (k_attn_block, k_ffn_block) + final norm + head",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind + " copy bandwidth (burst figure; the step is latency-bound)",
                         "algorithmic_bytes_per_token": bytes_tok,
                         # dram__bytes_read+write summed over the kernels of one step, ncu capture at context 260
                         # (profiles/decode_step_batch1_launch_list.md): the weights; KV pages were served by L2
                         "traffic": 200.3e6},
            "clocks": clocks.summary(),
        }
        if args.profile_only:
            line["profile_only"] = True
        if args.cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(budget_s=20.0)
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------- batch-512 decode (config 4) ---
def run_c4(args):
    """BASELINE config 4: 512 sequences (sharded by batch over the ranks), prompt lengths uniform in
    [256,1536] (seed 4), greedy decode towards 2048 tokens.  One step = 64 decode iterations of the
    whole shard; with the default 3 warm-up + 5 timed steps the longest sequence ends exactly at 2048."""
    import torch
    import torch.distributed as dist

    from small_llm_b200 import Engine, EngineOptions, ModelConfig, SamplingOptions, build

    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    c5, c3 = args.workload == "c5", args.workload == "c3"
    B, ITERS = (args.batch if not (c5 or c3) or args.batch != 512 else (32 * world if c5 else 64)), 64
    per = B // world
    # config 5: the scaled model (24 layers, d 1536, 24 heads of 64, FFN 4096), 32 sequences per GPU, prompts of 1024
    cfg = ModelConfig(num_layers=24, d_model=1536, num_heads=24, ffn_hidden=4096) if c5 else ModelConfig()
    eng = Engine(cfg, EngineOptions(max_batch=per, device=local))
    rng = np.random.default_rng(5 if c5 else 0)
    for name, shape in eng.param_infos():
        eng.set_param(name, rng.normal(0.0, 0.02, size=shape).astype(np.float32) if len(shape) == 2 else np.ones(shape, np.float32))
    lens_all = (np.full(B, 1024, np.int64) if c5 else np.full(B, 512, np.int64) if c3 else
                256 + (mt19937_raw(4, B) % np.uint32(1281)).astype(np.int64))
    lens = lens_all[rank * per:(rank + 1) * per]
    prompts = [prompt_ids(100 + rank * per + i, int(n)) for i, n in enumerate(lens)]
    opt = SamplingOptions(temperature=0.0, repetition_penalty=1.0)
    stream = torch.cuda.ExternalStream(eng.stream(), device=torch.device("cuda", local))
    t0 = time.perf_counter()
    eng.prefill(prompts)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    n_warm = args.warmup
    for _ in range(n_warm):
        eng.decode_loop(ITERS, opt, None, eos=EOS_NEVER)
    ctx0 = lens + n_warm * ITERS
    launches0 = eng.stats()["launches"]
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev0.record(stream)
        for _ in range(args.steps):
            eng.decode_loop(ITERS, opt, None, eos=EOS_NEVER)
        ev1.record(stream)
        ev1.synchronize()
        if world > 1:
            dist.barrier()
    ms = ev0.elapsed_time(ev1)
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    n_iter = args.steps * ITERS
    alive = np.minimum(ctx0 + n_iter, cfg.context_length + 1) - np.minimum(ctx0, cfg.context_length + 1)
    tok_local = torch.tensor([float(alive.sum())], dtype=torch.float64, device="cuda")
    # bytes: weights once per iteration + every live sequence's KV up to its context
    ctx_sum = float(sum(np.minimum(ctx0 + i, cfg.context_length).sum() for i in range(n_iter)))
    kv_per_pos = 2.0 * cfg.num_layers * cfg.d_model * 2
    by = torch.tensor([n_iter * (algorithmic_bytes_per_token(cfg, 0.0) - kv_per_pos) + kv_per_pos * ctx_sum], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(tok_local); dist.all_reduce(by, op=dist.ReduceOp.MAX)
    if rank == 0:
        peak, kind = peaks()
        achieved = float(by[0]) / (ms * 1e-3) / 1e9
        emit(({
            "metric": f"decode tok/s at batch {B} vs HBM roofline", "value": float(tok_local[0]) / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": n_warm, "ms_per_step": ms / args.steps,
            "per_iteration_ms": ms / n_iter, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 weights+KV, f32 accumulate", "data": "synthetic: N(0,0.02) weights, std::mt19937 ids and lengths",
            "config": {"workload": (f"BASELINE config 5: 0.73B model, batch {B} over {world} GPU(s), prompts of 1024, greedy decode, " if c5 else
                                    f"BASELINE config 3: batch {B} over {world} GPU(s), prompts of 512, greedy decode, " if c3 else
                                    f"BASELINE config 4: batch {B} over {world} GPU(s), prompts uniform in [256,1536], greedy decode, ")
                                   + f"{ITERS} iterations per step", "mean_context_at_start": float(lens_all.mean()) + n_warm * ITERS,
                       "l2": "inputs larger than L2 (KV cache of tens of GB)"},
            "prefill_s": prefill_s, "gpu_launches": int(eng.stats()["launches"] - launches0),
            "roofline": {"bound": "hbm", "kernel": "one decode iteration of the shard", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": kind, "traffic": None},
            "clocks": clocks.summary()}))
    if world > 1:
        dist.barrier(); dist.destroy_process_group()


# --------------------------------------------------------------------- reference / CPU arm ---
def _ref_model(fast=True):
    """The reference's own CPU code (oracle/_ref, compiled from its sources) when present, else
    this repository's C restatement of it."""
    from oracle import binding
    cfgo = binding.Config()
    if binding.ref_available():
        import ctypes
        flags = open("/proc/cpuinfo").read()
        use_fast = fast and " avx2" in flags and " fma" in flags and os.path.exists(binding.REF_FAST_SO)
        m = binding.RefModel(cfgo, fast=use_fast)
        m.init_normal(0, 0.02)
        return m, "reference", 1
    m = binding.OracleModel(cfgo)
    m.init_normal(0, 0.02)
    return m, "port", os.cpu_count() or 1


def _ref_token_step(model, kind, window: int) -> float:
    """Seconds for ONE token of the reference's loop at the given window: a full forward over the
    window (the reference keeps no KV cache) plus its host sampler."""
    prompt = prompt_ids(1, N_PROMPT)[:window]
    t0 = time.perf_counter()
    if kind == "reference":
        model.generate_tokens(prompt, 1, SAMPLING["temperature"], SAMPLING["top_p"], SAMPLING["repetition_penalty"], 2)
    else:
        model.generate(prompt, 1, SAMPLING["temperature"], SAMPLING["top_p"], SAMPLING["repetition_penalty"],
                       us=uniform_draws(2, 1), eos=EOS_NEVER & 0x7fffffff)
    return time.perf_counter() - t0


def cpu_baseline(budget_s: float) -> dict:
    model, kind, cores = _ref_model()
    probe = _ref_token_step(model, kind, 8)
    window = int(max(8, min(N_PROMPT, 8 * budget_s / max(probe, 1e-3))))
    dt = _ref_token_step(model, kind, window)
    return {"value": 1.0 / dt, "unit": "tokens/s", "cores": cores, "kind": kind,
            "sample": f"one token of the reference loop (full forward over a {window}-id window + host sampler); "
                      f"the configured window is {N_PROMPT}..{N_PROMPT + N_NEW - 1} and the cost grows linearly with it, "
                      f"so this figure favours the CPU side"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model, kind, cores = _ref_model()
    total = max(args.steps + args.warmup, 1)
    probe = _ref_token_step(model, kind, 8)
    per_step_budget = max(1.0, 150.0 / total)
    window = int(max(8, min(N_PROMPT, 8 * per_step_budget / max(probe, 1e-3))))
    for _ in range(args.warmup):
        _ref_token_step(model, kind, window)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _ref_token_step(model, kind, window)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    value = 1.0 / dt
    sample = (f"each step = one token of the reference's own loop on CPU (full forward over a {window}-id window, no KV "
              f"cache, + host sampler); configured window {N_PROMPT}..{N_PROMPT + N_NEW - 1}, cost linear in the window")
    emit(({
        "impl": "reference", "metric": METRIC,
        "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic: N(0,0.02) weights (reference generator, seed 0), std::mt19937 prompt ids",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


_REAL_STDOUT = None


def emit(line: dict):
    """The one JSON line, on the process's real standard output."""
    text = json.dumps(line) + "\n"
    if _REAL_STDOUT is None:
        sys.stdout.write(text); sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, text.encode())


def main():
    global N_NEW, _REAL_STDOUT
    # Libraries print to standard output on their own (the collective library announces its version there when the
    # process group comes up): everything but the JSON line goes to standard error instead.
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--decode-steps", type=int, default=N_NEW,
                    help="profiling only: shorter generations (the printed value is then not a benchmark figure)")
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5"],
                    help="c2 (default, the headline), c3 = 64 sequences with prompts of 512, c4 = batch-512 decode, "
                         "c5 = the 0.73B model at 32 sequences per GPU")
    ap.add_argument("--batch", type=int, default=512, help="c4 only: total sequences")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    args = ap.parse_args()
    if args.decode_steps != N_NEW:
        N_NEW = args.decode_steps
        args.profile_only = True
        args.cpu_baseline = False
    else:
        args.profile_only = False
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("c3", "c4", "c5"):
        run_c4(args)
    else:
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            args.cpu_baseline = False
        run_ours(args)


if __name__ == "__main__":
    main()
