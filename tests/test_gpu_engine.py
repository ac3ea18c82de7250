"""GPU parity tests: the CUDA engine, called through the C ABI, against the CPU oracle.

Tolerances.  Logits: max|gpu - ref| / max|ref| per position <= 2e-2 (bf16 weights / KV cache, the
bound the task states); in fp32-weights mode the only difference is summation order, so 2e-5 is
demanded.  Greedy streams: identical except after a step whose reference top-2 margin is below
1e-2.  Sampled streams, same draws: identical, a step being exempt only when the draw lies within
1e-7 of a cumulative boundary (the device uses CUDA's expf, glibc's differs in the last bit).
"""
import os

import numpy as np
import pytest

from oracle.binding import OracleSession, greedy, prompt_ids, sample, uniforms
from small_llm_b200 import SamplingOptions, SllmError
from tests.helpers import FULL, MID, ODD, SMALL, SMALL_EOS, WIDE, make_pair, rel_err

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2
TOL_F32 = 2e-5


@pytest.mark.parametrize("cfg,fp32,tol", [(SMALL, True, TOL_F32), (SMALL, False, TOL_BF16), (ODD, True, TOL_F32),
                                          (ODD, False, TOL_BF16), (MID, True, TOL_F32), (MID, False, TOL_BF16)])
def test_forward_logits_match_oracle(cfg, fp32, tol):
    # bf16 cases use a weight scale at which activations stay O(1), as in a trained or N(0,0.02) model;
    # fp32 cases use a harsher scale (peaked logits)
    std = (0.2 if cfg is not MID else 0.1) if fp32 else 0.05
    o, eng = make_pair(cfg, seed=3, stddev=std, fp32=fp32, max_batch=2)
    T = cfg.context
    ids = prompt_ids(1, 3 * T, cfg.vocab)
    ref = o.forward(ids, 3, T)
    got = eng.forward_logits(ids, 3, T)          # 3 rows through 2 slots: two groups
    assert got.shape == ref.shape
    assert rel_err(got, ref) <= tol
    one = eng.forward_logits(ids[:1], 1, 1)      # single token
    assert rel_err(one, o.forward(ids[:1], 1, 1)) <= tol


@pytest.mark.parametrize("cfg,fp32,tol", [(MID, True, TOL_F32), (MID, False, TOL_BF16), (SMALL, True, TOL_F32)])
def test_decode_steps_equal_prefill_rows(cfg, fp32, tol):
    """KV-cache invariant: logits of decode step t == last row of a forward over the prefix, for
    every t up to the context limit (page boundaries and the split-K merge included)."""
    o, eng = make_pair(cfg, seed=5, stddev=0.1 if fp32 else 0.05, fp32=fp32, via_checkpoint=False)
    T = cfg.context
    ids = prompt_ids(2, T, cfg.vocab)
    ref = o.forward(ids, 1, T)[0]
    n0 = 5
    eng.prefill([ids[:n0]])
    assert rel_err(eng.step_logits(0), ref[n0 - 1]) <= tol
    greedy_opt = SamplingOptions(temperature=0.0, repetition_penalty=1.0)
    worst = 0.0
    for t in range(n0, T):
        eng.sample(greedy_opt, eos=cfg.vocab + 5)       # appends some token ...
        eng.force_token(0, int(ids[t]))                 # ... which teacher forcing replaces
        eng.decode_step()
        worst = max(worst, rel_err(eng.step_logits(0), ref[t]))
    assert worst <= tol
    assert np.array_equal(eng.tokens(0), ids)


@pytest.mark.parametrize("fp32,tol", [(True, TOL_F32), (False, TOL_BF16)])
def test_wide_layer_shape_of_config5(fp32, tol):
    """The 0.73B configuration's layer shape (d_model 1536, 24 heads, ffn 4096) through prefill, the fused
    single-token decode path and a small batch."""
    cfg = WIDE
    o, eng = make_pair(cfg, seed=5, stddev=0.02, fp32=fp32, max_batch=3, via_checkpoint=False)
    ids = prompt_ids(21, 3 * 100, cfg.vocab)
    ref = o.forward(ids, 3, 100)
    assert rel_err(eng.forward_logits(ids, 3, 100), ref) <= tol
    # decode steps, teacher-forced: slot 0 alone (fused path), then three slots together
    for n_slots in (1, 3):
        prompts = [ids[s * 100: s * 100 + 70] for s in range(n_slots)]
        eng.prefill(prompts)
        opt = SamplingOptions(temperature=0.0, repetition_penalty=1.0)
        for t in range(70, 100):
            eng.sample(opt, eos=cfg.vocab + 1)
            for s in range(n_slots):
                eng.force_token(s, int(ids[s * 100 + t]))
            eng.decode_step()
            for s in range(n_slots):
                assert rel_err(eng.step_logits(s), ref[s, t]) <= tol, (n_slots, s, t)


def test_batched_ragged_prefill_and_decode():
    cfg = MID
    o, eng = make_pair(cfg, seed=6, stddev=0.1, fp32=True, max_batch=5)
    lens = [1, 7, 64, 65, 130]
    prompts = [prompt_ids(10 + i, n, cfg.vocab) for i, n in enumerate(lens)]
    eng.prefill(prompts)
    sessions = [OracleSession(o) for _ in prompts]
    for s, (sess, p) in enumerate(zip(sessions, prompts)):
        assert rel_err(eng.step_logits(s), sess.feed(p)) <= TOL_F32
    opt = SamplingOptions(temperature=0.0, repetition_penalty=1.0)
    for step in range(3):
        eng.sample(opt, eos=cfg.vocab + 5)
        eng.decode_step()
        for s, sess in enumerate(sessions):
            tok = eng.tokens(s)[-1]
            assert rel_err(eng.step_logits(s), sess.feed([tok])) <= TOL_F32


def _check_sampled_stream(eng, o, cfg, prompt, n_new, opt, us, eos):
    """Free-running engine stream vs the oracle fed the same draws; on a mismatch the oracle's
    margin at that step must be below 1e-7 (and the comparison stops there)."""
    got = eng.generate([prompt], n_new, opt, draws=us.astype(np.float64).reshape(-1, 1), eos=eos)[0]
    ref = o.generate(prompt, n_new, opt.temperature, opt.top_p, opt.repetition_penalty, us=us, eos=eos,
                     stop=opt.stop_token)
    n = min(len(got), len(ref))
    if np.array_equal(got, ref):
        return len(ref) - len(prompt), None
    first = int(np.argmax(got[:n] != ref[:n])) if not np.array_equal(got[:n], ref[:n]) else n
    return first - len(prompt), first


@pytest.mark.parametrize("t,p,pen", [(0.8, 0.95, 1.15), (0.7, 0.8, 1.1), (1.3, 0.5, 1.0), (0.2, 0.999, 2.0), (1.0, 1.0, 1.0)])
def test_sampled_streams_fp32_identical(t, p, pen):
    cfg = SMALL
    o, eng = make_pair(cfg, seed=3, stddev=0.2, fp32=True)
    prompt = prompt_ids(5, 8, cfg.vocab)
    us = uniforms(2, 50)
    opt = SamplingOptions(temperature=t, top_p=p, repetition_penalty=pen)
    n_same, first = _check_sampled_stream(eng, o, cfg, prompt, 50, opt, us, SMALL_EOS)
    assert first is None, f"streams diverge at generated token {n_same}"


def test_sampler_only_on_reference_logits():
    """Identical logits + identical draws -> identical token, including ties and a peaked row."""
    cfg = SMALL
    o, eng = make_pair(cfg, seed=3, stddev=0.2, fp32=True)
    rng = np.random.default_rng(0)
    hist = prompt_ids(8, 12, cfg.vocab)
    eng.prefill([hist])
    rows = [rng.normal(0, s, cfg.vocab).astype(np.float32) for s in (0.5, 2.0, 8.0)]
    tie = np.round(rng.normal(0, 1.0, cfg.vocab) * 4).astype(np.float32) / 4     # many exact ties
    rows.append(tie)
    flat = np.zeros(cfg.vocab, np.float32)                                        # all equal
    rows.append(flat)
    exempt = 0
    for r, row in enumerate(rows):
        for k, (t, p, pen) in enumerate([(0.8, 0.95, 1.15), (1.0, 0.5, 1.0), (0.3, 0.999, 1.3), (2.0, 0.1, 1.0)]):
            for u in (0.0, 0.123456789, 0.5, 0.87654321, 0.999999):
                eng.truncate(0, len(hist))
                eng.set_step_logits(0, row)
                eng.sample(SamplingOptions(temperature=t, top_p=p, repetition_penalty=pen), draws=[u], eos=cfg.vocab + 1)
                got = int(eng.tokens(0)[-1])
                want, margin = sample(row, hist, t, p, pen, u)
                if got != want:
                    assert margin < 1e-7, (r, k, u, got, want, margin)
                    exempt += 1
    assert exempt <= 2
    # greedy: first maximum after the penalty
    for row in rows:
        eng.truncate(0, len(hist))
        eng.set_step_logits(0, row)
        eng.sample(SamplingOptions(temperature=0.0, repetition_penalty=1.3), eos=cfg.vocab + 1)
        assert int(eng.tokens(0)[-1]) == greedy(row, hist, 1.3)[0]


def test_seeded_mode_reproduces_reference_loop(golden_dir):
    """fp32 weights, no draws supplied: the engine consumes std::mt19937_64(seed) the way
    std::discrete_distribution does, so it reproduces the streams that the reference's own
    Inference::generateTokens produced (golden file written by the unmodified reference)."""
    import os
    g = np.load(os.path.join(golden_dir, "small_ref.npz"))
    o, eng = make_pair(SMALL, seed=3, stddev=0.2, fp32=True)
    for seed in (2, 1234, 3):
        t, p, pen, n = g[f"opts_seed{seed}"]
        ref = g[f"stream_seed{seed}"]
        opt = SamplingOptions(temperature=float(t), top_p=float(p), repetition_penalty=float(pen), seed=seed)
        got = eng.generate([g["prompt"]], int(n), opt, draws=None, eos=SMALL_EOS)[0]
        assert np.array_equal(got, ref), seed
    assert len(g["stream_seed2"]) > SMALL.context + 1          # these streams slid the window, as the reference does


def test_sliding_window_and_long_prompt_match_oracle():
    """Beyond context_length the reference re-runs the last context_length tokens for every new token
    (positions restart at 0); prompts longer than the context are windowed the same way."""
    cfg = SMALL
    o, eng = make_pair(cfg, seed=3, stddev=0.2, fp32=True, max_batch=2)
    us = uniforms(7, 30)
    opt = SamplingOptions(temperature=0.9, top_p=0.9, repetition_penalty=1.2)
    long_prompt = prompt_ids(11, cfg.context + 9, cfg.vocab)
    short_prompt = prompt_ids(12, cfg.context - 3, cfg.vocab)
    draws = np.repeat(us.astype(np.float64).reshape(-1, 1), 2, axis=1)
    got = eng.generate([long_prompt, short_prompt], 30, opt, draws=draws, eos=SMALL_EOS)
    for p, gs in zip((long_prompt, short_prompt), got):
        ref = o.generate(p, 30, 0.9, 0.9, 1.2, us=us, eos=SMALL_EOS)
        assert np.array_equal(gs, ref)
    with pytest.raises(ValueError, match="token buffer"):
        eng.generate([prompt_ids(1, 2 * cfg.context + 2, cfg.vocab)], 1, opt, draws=draws[:1], eos=SMALL_EOS)


def test_stop_rules_and_errors():
    cfg = SMALL
    o, eng = make_pair(cfg, seed=3, stddev=0.2, fp32=True, max_batch=2)
    prompt = prompt_ids(5, 8, cfg.vocab)
    opt = SamplingOptions(temperature=0.0, repetition_penalty=1.0)
    ref = o.generate(prompt, 6, 0.0, 1.0, 1.0, eos=SMALL_EOS)
    got = eng.generate([prompt], 6, opt, eos=SMALL_EOS)[0]
    assert np.array_equal(got, ref)
    # EOS is appended, then generation stops (src/inference.cpp:158-160)
    eos = int(ref[len(prompt) + 2])
    want = o.generate(prompt, 6, 0.0, 1.0, 1.0, eos=eos)
    assert len(want) <= len(prompt) + 3 and want[-1] == eos
    got = eng.generate([prompt], 6, opt, eos=eos)[0]
    assert np.array_equal(got, want)
    # an extra stop token behaves the same way
    got = eng.generate([prompt], 6, SamplingOptions(temperature=0.0, repetition_penalty=1.0, stop_token=eos), eos=SMALL_EOS)[0]
    assert np.array_equal(got, want)
    # max_new = 0 returns the prompt
    assert np.array_equal(eng.generate([prompt], 0, opt, eos=SMALL_EOS)[0], prompt)
    with pytest.raises(ValueError, match="zero tokens"):
        eng.generate([np.zeros(0, np.uint32)], 3, opt)
    with pytest.raises(ValueError, match="exceeds context_length"):
        eng.forward_logits(np.zeros(cfg.context + 1, np.uint32), 1, cfg.context + 1)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.prefill([np.array([cfg.vocab], np.uint32)])
    with pytest.raises(SllmError, match="max_batch"):
        eng.prefill([prompt, prompt, prompt])
    with pytest.raises(SllmError, match="cannot open"):
        eng.load_checkpoint("/nonexistent/ck.bin")
    # non-finite logits are reported like the reference's runtime_error
    eng.prefill([prompt])
    eng.set_step_logits(0, np.full(cfg.vocab, -np.inf, np.float32))
    with pytest.raises(SllmError, match="non-finite"):
        eng.sample(SamplingOptions(temperature=0.8), draws=[0.5], eos=SMALL_EOS)


def test_config1_greedy_100m_bf16_and_fp32():
    """BASELINE config 1: 100.3M model, seed-0 N(0,0.02) weights, prompt of 128 seed-1 ids, 128
    greedy steps.  Teacher-forced logits within tolerance at every step; greedy tokens equal the
    oracle's except after a step whose reference top-2 margin is below 1e-2."""
    cfg = FULL
    n_prompt, n_new = 128, 128
    prompt = prompt_ids(1, n_prompt)
    o, eng = make_pair(cfg, seed=0, stddev=0.02, fp32=False)
    ref_stream = o.generate(prompt, n_new, 0.0, 1.0, 1.0, eos=32762)
    assert len(ref_stream) == n_prompt + n_new
    ref_logits = o.forward(ref_stream[:-1], 1, len(ref_stream) - 1, row_from=n_prompt - 1)[0]   # rows for every step
    # (a) prefill path, all positions in one call
    got_all = eng.forward_logits(ref_stream[:-1], 1, len(ref_stream) - 1)[0][n_prompt - 1:]
    err_prefill = rel_err(got_all, ref_logits)
    # (b) decode path, teacher-forced on the reference stream
    eng.prefill([prompt])
    opt = SamplingOptions(temperature=0.0, repetition_penalty=1.0)
    worst, flips = 0.0, []
    for i in range(n_new):
        step_ref = ref_logits[i]
        worst = max(worst, rel_err(eng.step_logits(0), step_ref))
        eng.sample(opt)
        tok = int(eng.tokens(0)[-1])
        want = int(ref_stream[n_prompt + i])
        if tok != want:
            _, margin = greedy(step_ref, prompt, 1.0)
            flips.append((i, margin))
            eng.force_token(0, want)
        if i + 1 < n_new:
            eng.decode_step()
    msg = f"config1 bf16: prefill rel err {err_prefill:.2e}, decode rel err {worst:.2e}, greedy flips (step, ref margin) {flips}"
    print(msg)
    report_dir = os.environ.get("SLLM_REPORT_DIR")
    if report_dir and os.path.isdir(report_dir):
        open(os.path.join(report_dir, "config1_parity.txt"), "w").write(msg + "\n")
    assert err_prefill <= TOL_BF16 and worst <= TOL_BF16
    assert all(m < 1e-2 for _, m in flips), flips
    # fp32 weights: the free-running greedy stream is the oracle's stream
    del eng
    o2, eng32 = make_pair(cfg, seed=0, stddev=0.02, fp32=True)
    got = eng32.generate([prompt], n_new, opt)[0]
    same = np.array_equal(got, ref_stream)
    if not same:
        first = int(np.argmax(got != ref_stream))
        _, margin = greedy(ref_logits[first - n_prompt], prompt, 1.0)
        assert margin < 1e-4, (first, margin)


def test_config3_batch64_subset_against_oracle():
    """BASELINE config 3 shape: 100.3M model, bf16, 64 sequences with 512-id prompts (seed 3), greedy decode.
    The oracle (fp32) is run on a stated subset -- sequences 0, 21 and 63 -- teacher-forced on the engine's own
    streams: every engine token must be the oracle's arg-max at that step unless the oracle's top-2 margin
    there is below 1e-2; logits of the last prompt position within 2e-2."""
    cfg = FULL
    n_seq, n_prompt, n_new = 64, 512, 48
    o, eng = make_pair(cfg, seed=0, stddev=0.02, fp32=False, max_batch=n_seq)
    all_ids = prompt_ids(3, n_seq * n_prompt)
    prompts = [all_ids[i * n_prompt:(i + 1) * n_prompt] for i in range(n_seq)]
    opt = SamplingOptions(temperature=0.0, repetition_penalty=1.0)
    eng.prefill(prompts)
    first_logits = {s: eng.step_logits(s) for s in (0, 21, 63)}
    streams = eng.generate(prompts, n_new, opt)
    assert all(len(x) == n_prompt + n_new for x in streams)
    flips = []
    for s in (0, 21, 63):
        st = streams[s]
        ref = o.forward(st[:-1], 1, len(st) - 1, row_from=n_prompt - 1)[0]
        assert rel_err(first_logits[s], ref[0]) <= TOL_BF16
        for i in range(n_new):
            want, margin = greedy(ref[i], st[:n_prompt + i], 1.0)
            if int(st[n_prompt + i]) != want:
                flips.append((s, i, margin))
    assert all(m < 1e-2 for _, _, m in flips), flips
    assert len(flips) <= 6, flips


@pytest.mark.parametrize("fp32", [True, False])
def test_eval_loss_matches_reference_cross_entropy(fp32, golden_dir):
    """sllm_eval_loss against the reference's own ops::cross_entropy values (tests/golden/ce_ref.npz, produced by
    the unmodified reference for these weights, ids and targets) and against the oracle on a ragged group count."""
    import os
    from oracle.binding import cross_entropy
    g = np.load(os.path.join(golden_dir, "ce_ref.npz"))
    o, eng = make_pair(SMALL, seed=3, stddev=0.2 if fp32 else 0.05, fp32=fp32, max_batch=2, via_checkpoint=False)
    tol = 2e-5 if fp32 else 2e-2
    nv = int((g["masked"] >= 0).sum())
    if fp32:                                                # the golden values belong to the stddev-0.2 weights
        assert abs(eng.eval_loss(g["ids"], g["targets"], 2, 24) - float(g["loss_all"])) <= tol
        assert abs(eng.eval_loss(g["ids"], g["masked"], 2, 24, nv) - float(g["loss_masked"])) <= tol
    # three rows on an engine with two slots: the third goes through in a second group
    ids = prompt_ids(9, 3 * 40, SMALL.vocab)
    targets = np.roll(ids.reshape(3, 40), -1, axis=1).reshape(-1).astype(np.int32)
    targets[5::7] = -1
    n = int((targets >= 0).sum())
    ref = cross_entropy(o.forward(ids, 3, 40).reshape(120, SMALL.vocab), targets, n)
    assert abs(eng.eval_loss(ids, targets, 3, 40, n) - ref) <= tol
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.eval_loss(ids, np.full(120, SMALL.vocab, np.int32), 3, 40)


@pytest.mark.parametrize("split,epilogue", [(2, "transposing"), (4, "transposing"), (2, "thread-per-row"), (4, "thread-per-row")])
def test_split_k_cluster_projections(split, epilogue, monkeypatch):
    """The tensor-core projections with their K blocks dealt over a thread-block cluster (forced here; the engine
    chooses it by itself only when few tiles exist), with either epilogue: same logits as the oracle within the bf16
    tolerance, and the same as the unsplit kernel up to the rounding of intermediate activations."""
    cfg = MID                                               # K = 128 (2 K blocks) and 200 (4, the last one ragged)
    ids = prompt_ids(1, 2 * 100, cfg.vocab)
    if epilogue == "thread-per-row":
        monkeypatch.setenv("SLLM_NO_WIDE_EPI", "1")
    monkeypatch.setenv("SLLM_TC_SPLIT", "1")
    o, eng1 = make_pair(cfg, seed=3, stddev=0.05, fp32=False, max_batch=2, via_checkpoint=False)
    base = eng1.forward_logits(ids, 2, 100)
    monkeypatch.setenv("SLLM_TC_SPLIT", str(split))
    _, eng = make_pair(cfg, seed=3, stddev=0.05, fp32=False, max_batch=2, via_checkpoint=False)
    got = eng.forward_logits(ids, 2, 100)
    ref = o.forward(ids, 2, 100)
    assert rel_err(got, ref) <= TOL_BF16
    assert rel_err(got, base) <= 5e-3
    # decode at 20 sequences goes through the same kernels with one token per sequence
    prompts = [prompt_ids(10 + i, 30 + i, cfg.vocab) for i in range(20)]
    _, engb = make_pair(cfg, seed=3, stddev=0.05, fp32=False, max_batch=20, via_checkpoint=False)
    engb.prefill(prompts)
    engb.decode_loop(3, SamplingOptions(temperature=0.0, repetition_penalty=1.0), None, eos=cfg.vocab + 5)
    for i in (0, 7, 19):
        toks = engb.tokens(i)
        assert toks.size == prompts[i].size + 3
        assert rel_err(engb.step_logits(i), o.forward(toks, 1, toks.size)[0, -1]) <= TOL_BF16


def test_gemv_family_for_small_bf16_passes(monkeypatch):
    """bf16 passes of 2 and more tokens take the tensor-core kernels by default; the weight-streaming GEMV family
    (what runs when the driver offers no tensor-map encoder, and in fp32 mode) is forced here: prefill of ragged
    prompts and decode steps against the oracle."""
    monkeypatch.setenv("SLLM_TC_MIN_TOKENS", "100000")
    cfg = MID
    o, eng = make_pair(cfg, seed=7, stddev=0.05, fp32=False, max_batch=5, via_checkpoint=False)
    prompts = [prompt_ids(30 + i, n, cfg.vocab) for i, n in enumerate([3, 70, 1, 129, 40])]
    eng.prefill(prompts)
    for i, p in enumerate(prompts):
        assert rel_err(eng.step_logits(i), o.forward(p, 1, p.size)[0, -1]) <= TOL_BF16
    eng.decode_loop(4, SamplingOptions(temperature=0.0, repetition_penalty=1.0), None, eos=cfg.vocab + 5)
    for i, p in enumerate(prompts):
        toks = eng.tokens(i)
        assert toks.size == p.size + 4
        assert rel_err(eng.step_logits(i), o.forward(toks, 1, toks.size)[0, -1]) <= TOL_BF16


def test_sampler_with_one_block_per_slot_at_large_batch():
    """At 300 and more slots the sampler's partial kernels get a single block per slot (each thread then walks
    many vocabulary entries) and the attention grid is ordered longest sequence first: sampled streams of a few
    slots against the oracle."""
    cfg = SMALL
    n_seq, n_new = 320, 12
    o, eng = make_pair(cfg, seed=3, stddev=0.2, fp32=True, max_batch=n_seq, via_checkpoint=False)
    prompts = [prompt_ids(200 + i, 3 + (i * 7) % 40, cfg.vocab) for i in range(n_seq)]
    us = np.stack([uniforms(500 + i, n_new) for i in range(n_seq)], axis=1).astype(np.float64)     # [step][slot]
    opt = SamplingOptions(temperature=0.9, top_p=0.9, repetition_penalty=1.1)
    got = eng.generate(prompts, n_new, opt, draws=us, eos=SMALL_EOS)
    for i in (0, 1, 17, 160, 299, 319):
        ref = o.generate(prompts[i], n_new, 0.9, 0.9, 1.1, us=us[:, i].astype(np.float32), eos=SMALL_EOS)
        assert np.array_equal(got[i], ref), i


@pytest.mark.parametrize("cfg,std", [(MID, 0.05), (ODD, 0.05), (SMALL, 0.05), (FULL, 0.02)], ids=["hd32", "hd16", "small", "100m-hd64"])
def test_persistent_decode_kernel_against_oracle_and_layerwise_kernels(cfg, std, monkeypatch):
    """Batch-1 decode in bf16 runs as one resident kernel per token (every layer and the head; vectors handed between
    blocks as tagged words).  Teacher-forced over a context that crosses page boundaries: its logits against the
    oracle (2e-2) and against the two-kernels-per-layer path it replaces (same arithmetic, other summation order),
    which SLLM_NO_PERSIST selects; then a free-running greedy generation must give the same stream on both paths
    unless the oracle's top-2 margin is small."""
    T = min(cfg.context, 200)
    ids = prompt_ids(2, T, cfg.vocab)
    o, eng = make_pair(cfg, seed=5, stddev=std, fp32=False, via_checkpoint=False)
    monkeypatch.setenv("SLLM_NO_PERSIST", "1")
    _, old = make_pair(cfg, seed=5, stddev=std, fp32=False, via_checkpoint=False)
    monkeypatch.delenv("SLLM_NO_PERSIST")
    ref = o.forward(ids, 1, T)[0]
    n0 = 3
    opt = SamplingOptions(temperature=0.0, repetition_penalty=1.0)
    worst_ref, worst_old = 0.0, 0.0
    for e in (eng, old):
        e.prefill([ids[:n0]])
    for t in range(n0, T):
        for e in (eng, old):
            e.sample(opt, eos=cfg.vocab + 5)
            e.force_token(0, int(ids[t]))
            e.decode_step()
        a, b = eng.step_logits(0), old.step_logits(0)
        worst_ref = max(worst_ref, rel_err(a, ref[t]))
        worst_old = max(worst_old, rel_err(a, b))
    assert worst_ref <= TOL_BF16, worst_ref
    assert worst_old <= 5e-3, worst_old
    assert np.array_equal(eng.tokens(0), ids)
    # one-token prompt: the kernel without its head (the prefill path asks for the residual only)
    one = eng.forward_logits(ids[:1], 1, 1)
    assert rel_err(one, o.forward(ids[:1], 1, 1)) <= TOL_BF16
    # the graph-replayed loop
    n_new = 40
    got = eng.generate([ids[:20]], n_new, opt, eos=cfg.vocab + 5)[0]
    want = old.generate([ids[:20]], n_new, opt, eos=cfg.vocab + 5)[0]
    if not np.array_equal(got, want):
        first = int(np.argmax(got != want))
        rl = o.forward(got[:first], 1, first)[0, -1]
        _, margin = greedy(rl, got[:first], 1.0)
        assert margin < 1e-2, (first, margin)


@pytest.mark.parametrize("t,p,pen", [(0.8, 0.95, 1.15), (1.0, 0.5, 1.0), (0.0, 1.0, 1.3)])
def test_sampler_kernels_folded_into_the_persistent_kernel(t, p, pen, monkeypatch):
    """Inside a graph of several decode iterations the persistent batch-1 kernel also does the work of the next
    sampling step's first two kernels (per-block maxima of the penalised scores, weights, level-0 histogram).  Same
    logits, same expf, same fixed-point masses: the generated stream must be identical, token for token, to the one
    produced with the three sampler kernels kept apart (SLLM_NO_FOLD), at the real vocabulary and on a small model."""
    for cfg, std, n_new in ((FULL, 0.02, 70), (MID, 0.05, 100)):
        prompt = prompt_ids(7, 40, cfg.vocab)
        us = uniforms(9, n_new).astype(np.float64).reshape(-1, 1)
        opt = SamplingOptions(temperature=t, top_p=p, repetition_penalty=pen)
        o, eng = make_pair(cfg, seed=0, stddev=std, fp32=False, via_checkpoint=False)
        got = eng.generate([prompt], n_new, opt, draws=us, eos=cfg.vocab + 1)[0]
        monkeypatch.setenv("SLLM_NO_FOLD", "1")
        _, plain = make_pair(cfg, seed=0, stddev=std, fp32=False, via_checkpoint=False)
        monkeypatch.delenv("SLLM_NO_FOLD")
        want = plain.generate([prompt], n_new, opt, draws=us, eos=cfg.vocab + 1)[0]
        assert got.size == prompt.size + n_new
        assert np.array_equal(got, want), (cfg.vocab, int(np.argmax(got != want)))
