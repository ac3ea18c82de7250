"""Error paths and state hygiene of the engine on a GPU.  Every failure here is made on the host or runs out by
itself: nothing faults, traps or spins without bound on the device."""
import numpy as np
import pytest

from oracle.binding import Config, prompt_ids, uniforms
from small_llm_b200 import Engine, EngineOptions, SamplingOptions, SllmError
from small_llm_b200.api import ERR_CAPACITY, ERR_DEVICE_WAIT
from small_llm_b200.batching import ContinuousBatcher, Request
from tests.helpers import MID, SMALL, make_pair, rel_err, to_model_config

pytestmark = pytest.mark.gpu


def test_bounded_device_wait_runs_out_and_engine_stays_usable():
    """A device thread waits on a barrier that nothing arrives at; after its limit (3 ms here) it raises the
    engine's status word and returns; the host reports SLLM_ERR_DEVICE_WAIT, clears the word, and the engine
    computes as before."""
    cfg = SMALL
    o, eng = make_pair(cfg, seed=3, stddev=0.2, fp32=True, via_checkpoint=False)
    ids = prompt_ids(1, 20, cfg.vocab)
    before = eng.forward_logits(ids, 1, 20)
    with pytest.raises(SllmError, match="bounded device-side wait gave up") as ei:
        eng.wait_probe(3000)
    assert ei.value.code == ERR_DEVICE_WAIT
    after = eng.forward_logits(ids, 1, 20)                       # the status word was cleared: no stale error
    assert np.array_equal(before, after)
    assert rel_err(after, o.forward(ids, 1, 20)) <= 2e-5
    with pytest.raises(ValueError, match="limit must be"):
        eng.wait_probe(0)


def test_kv_page_pool_exhaustion_is_reported_and_recoverable():
    cfg = MID                                                    # context 256 = 4 pages per sequence
    o, eng = make_pair(cfg, seed=3, stddev=0.1, fp32=True, max_batch=2, via_checkpoint=False, kv_pages=3)
    a, b = prompt_ids(1, 100, cfg.vocab), prompt_ids(2, 100, cfg.vocab)      # 2 pages each
    with pytest.raises(SllmError, match="KV page pool exhausted") as ei:
        eng.prefill([a, b])
    assert ei.value.code == ERR_CAPACITY
    eng.reset()
    assert eng.stats()["kv_pages_free"] == 3
    eng.prefill([a])
    assert rel_err(eng.step_logits(0), o.forward(a, 1, a.size)[0, -1]) <= 2e-5
    # growth during decode: the third page is the last one; the step that needs a fourth page fails cleanly
    opt = SamplingOptions(temperature=0.0, repetition_penalty=1.0)
    eng.decode_loop(92, opt, None, eos=cfg.vocab + 1)            # 192 positions = 3 pages
    assert eng.tokens(0).size == 192
    with pytest.raises(SllmError, match="KV page pool exhausted"):
        eng.decode_loop(2, opt, None, eos=cfg.vocab + 1)


def test_recycled_device_memory_does_not_reach_the_prefill_attention():
    """The KV pool is cleared when an engine is created.  Here an fp32 engine first fills its pool with NaN rows,
    is destroyed, and a bf16 engine of the same size (which gets the same device memory back) prefills prompts
    that end inside a page: the rows of the last page behind the last position must not poison the tensor-core
    attention, which multiplies whole pages by probabilities that are zero there."""
    cfg = Config(vocab=512, context=256, layers=2, d_model=128, heads=2, ffn=192)      # head_dim 64: tcgen05 prefill attention
    mc = to_model_config(cfg)
    junk = Engine(mc, EngineOptions(max_batch=2, fp32_weights=True))
    junk.prefill([prompt_ids(1, cfg.context, cfg.vocab), prompt_ids(2, cfg.context, cfg.vocab)])
    nan_rows = np.full((cfg.context, cfg.d_model), np.nan, np.float32)
    for layer in range(cfg.layers):
        for slot in range(2):
            junk.kv_write(layer, slot, 0, nan_rows, nan_rows)
    k, _ = junk.kv_read(1, 1, 0, cfg.context)
    assert np.isnan(k).all()
    junk.close()
    o, eng = make_pair(cfg, seed=6, stddev=0.05, fp32=False, max_batch=2, via_checkpoint=False)
    prompts = [prompt_ids(3, 70, cfg.vocab), prompt_ids(4, 131, cfg.vocab)]            # both end mid-page
    eng.prefill(prompts)
    for s, p in enumerate(prompts):
        got = eng.step_logits(s)
        assert np.isfinite(got).all(), s
        assert rel_err(got, o.forward(p, 1, p.size)[0, -1]) <= 2e-2
    rows = eng.forward_logits(prompts[1], 1, prompts[1].size)[0]
    assert np.isfinite(rows).all()


def test_generate_refuses_requests_that_outgrow_the_token_buffer():
    cfg = SMALL
    o, eng = make_pair(cfg, seed=3, stddev=0.2, fp32=True, via_checkpoint=False)
    opt = SamplingOptions(temperature=0.0, repetition_penalty=1.0)
    prompt = prompt_ids(5, 8, cfg.vocab)
    with pytest.raises(SllmError, match="exceed a slot's token buffer") as ei:
        eng.generate([prompt], 2 * cfg.context + 2, opt, eos=cfg.vocab + 1)
    assert ei.value.code == ERR_CAPACITY
    out = eng.generate([prompt], 2 * cfg.context + 2 - 8, opt, eos=cfg.vocab + 1)[0]   # the largest request that fits
    assert out.size == 2 * cfg.context + 2


def test_sampled_batching_when_the_highest_slot_drains_first():
    """Three slots; the request in the highest slot stops first and nothing is waiting, so the engine's live range
    shrinks while lower slots keep sampling: their draws must still be read from the right columns."""
    cfg = MID
    o, eng = make_pair(cfg, seed=4, stddev=0.1, fp32=True, max_batch=3, via_checkpoint=False)
    opt = SamplingOptions(temperature=0.9, top_p=0.9, repetition_penalty=1.1)
    eos = cfg.vocab + 1
    budgets = [40, 33, 5]                                        # slot 2 drains first, then slot 1
    reqs = [Request(prompt_ids(90 + i, 10 + 3 * i, cfg.vocab), n, uniforms(80 + i, n)) for i, n in enumerate(budgets)]
    ContinuousBatcher(eng, opt, eos=eos, burst=4).run(reqs)
    assert eng.num_live() == 0
    for i, r in enumerate(reqs):
        ref = o.generate(r.prompt, r.max_new_tokens, 0.9, 0.9, 1.1, us=uniforms(80 + i, r.max_new_tokens), eos=eos)
        assert np.array_equal(r.tokens, ref), i
