"""Continuous batching: more requests than slots, different prompt lengths and budgets; every request's
tokens must equal what the oracle generates for it alone."""
import numpy as np
import pytest

from oracle.binding import prompt_ids, uniforms
from small_llm_b200 import SamplingOptions
from small_llm_b200.batching import ContinuousBatcher, Request
from tests.helpers import MID, make_pair

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("sampled", [False, True])
def test_continuous_batching_matches_single_sequence_generation(sampled):
    cfg = MID
    o, eng = make_pair(cfg, seed=4, stddev=0.1, fp32=True, max_batch=3, via_checkpoint=False)
    eos = 700                                                    # a token that does come up: some requests stop early
    opt = SamplingOptions(temperature=0.9 if sampled else 0.0, top_p=0.9, repetition_penalty=1.1 if sampled else 1.0)
    rng = np.random.default_rng(1)
    reqs = []
    for i in range(8):
        n_prompt = int(rng.integers(1, 90))
        max_new = int(rng.integers(1, 40))
        reqs.append(Request(prompt_ids(50 + i, n_prompt, cfg.vocab), max_new, uniforms(70 + i, max_new) if sampled else None))
    ContinuousBatcher(eng, opt, eos=eos, burst=7).run(reqs)
    for i, r in enumerate(reqs):
        ref = o.generate(r.prompt, r.max_new_tokens, opt.temperature, opt.top_p, opt.repetition_penalty,
                         us=uniforms(70 + i, r.max_new_tokens) if sampled else None, eos=eos)
        assert np.array_equal(r.tokens, ref), i
