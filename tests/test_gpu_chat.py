"""Multi-turn chat with the KV cache carried across turns: every turn's reply must equal what the oracle
generates from the whole conversation so far (the browser demo's history rules, docs/script.js:288-305)."""
import numpy as np
import pytest

from oracle.binding import prompt_ids, uniforms
from small_llm_b200 import SamplingOptions, SllmError
from small_llm_b200.chat import ChatSession
from tests.helpers import MID, make_pair

pytestmark = pytest.mark.gpu

T, TOP_P, PEN = 0.9, 0.9, 1.1


def _pick_eos(o, user0, n_new, us, ending):
    """An EOS id (the chat ids follow it) with which the oracle's first reply ends the wanted way."""
    for eos in range(520, 1000):
        ctx0 = np.concatenate([[eos + 1], user0, [eos + 3, eos + 2]]).astype(np.uint32)
        gen = o.generate(ctx0, n_new, T, TOP_P, PEN, us=us, eos=eos, stop=eos + 3)[ctx0.size:]
        last = int(gen[-1])
        if ending == "budget" and last not in (eos, eos + 3):
            return eos
        if ending == "end" and last == eos + 3 and gen.size >= 3:
            return eos
        if ending == "eos" and last == eos and gen.size >= 3:
            return eos
    raise AssertionError("no suitable EOS id found")


@pytest.mark.parametrize("ending", ["budget", "end", "eos"])
def test_chat_session_reuses_kv_and_matches_oracle(ending):
    cfg = MID
    o, eng = make_pair(cfg, seed=8, stddev=0.1, fp32=True, max_batch=1, via_checkpoint=False)
    opt = SamplingOptions(temperature=T, top_p=TOP_P, repetition_penalty=PEN)
    n_new = 24
    users = [prompt_ids(300 + t, 10 + 7 * t, 512) for t in range(6)]          # ids below the special tokens
    draws = [uniforms(400 + t, n_new) for t in range(6)]
    eos = _pick_eos(o, users[0], n_new, draws[0], ending)
    user_id, asst_id, end_id = eos + 1, eos + 2, eos + 3

    chat = ChatSession(eng, eos=eos)
    history = np.zeros(0, np.uint32)     # the conversation as the demo stores it
    stops = 0
    for t in range(6):
        prompt = np.concatenate([[user_id], users[t], [end_id, asst_id]]).astype(np.uint32)
        if history.size + prompt.size + n_new > cfg.context:
            history = np.zeros(0, np.uint32)                               # context full: forget
        context = np.concatenate([history, prompt]).astype(np.uint32)
        ref = o.generate(context, n_new, T, TOP_P, PEN, us=draws[t], eos=eos, stop=end_id)
        ref_reply = ref[context.size:]
        if ref_reply.size and ref_reply[-1] in (eos, end_id):
            ref_reply = ref_reply[:-1]
            stops += 1
        before, owed, fresh = eng.stats()["prefill_tokens"], chat.need_end, history.size == 0
        reply = chat.say(users[t], n_new, opt, draws[t])
        assert np.array_equal(reply, ref_reply), (ending, t)
        # only the new ids went through the model (plus the slot's last token, and the <|end|> still owed)
        ran = eng.stats()["prefill_tokens"] - before
        assert ran == (prompt.size if fresh else prompt.size + 1 + (1 if owed else 0)), (ending, t)
        history = np.concatenate([context, ref_reply, [end_id]]).astype(np.uint32)
        # what the slot holds is the stored history, minus a closing <|end|> that is still owed
        held = chat.history()
        want = history[:-1] if chat.need_end else history
        assert np.array_equal(held, want), (ending, t)
    assert chat.dropped_history >= 1                                       # 6 turns do not fit 256 positions
    if ending != "budget":
        assert stops >= 1
    with pytest.raises(ValueError, match="exceed context_length"):
        chat.say(prompt_ids(1, cfg.context, 512), 8, opt, uniforms(1, 8))


def test_slot_append_errors_and_equivalence_with_fresh_prefill():
    cfg = MID
    o, eng = make_pair(cfg, seed=8, stddev=0.1, fp32=True, max_batch=2, via_checkpoint=False)
    a, b = prompt_ids(1, 40, cfg.vocab), prompt_ids(2, 70, cfg.vocab)
    with pytest.raises(SllmError, match="holds no sequence"):
        eng.slot_append(0, b)
    eng.slot_assign(0, a)
    eng.slot_append(0, b)                                   # 110 tokens: crosses a page boundary
    got = eng.step_logits(0)
    eng.slot_assign(1, np.concatenate([a, b]))
    ref = eng.step_logits(1)
    assert np.abs(got - ref).max() <= 2e-5 * np.abs(ref).max()
    assert np.array_equal(eng.tokens(0), np.concatenate([a, b]))
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.slot_append(0, np.array([cfg.vocab], np.uint32))
    with pytest.raises(SllmError, match="exceed context_length"):
        eng.slot_append(0, prompt_ids(3, cfg.context, cfg.vocab))
