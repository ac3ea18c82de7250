"""Multi-turn chat over one engine slot with the KV cache carried across turns.

The reference's chat loop (src/main.cpp:46-62) treats every line as a fresh single-turn prompt.  Its browser
demo keeps a history (docs/script.js:288-305): each turn's context is the earlier turns followed by
`<|user|> text <|end|> <|assistant|>`; a finished turn is stored as prompt + reply + `<|end|>`; when history,
prompt and the reply budget no longer fit the context, the history is dropped.  The demo re-runs the whole
context every turn; this class keeps the slot's KV pages instead and sends only the new ids through the model
(`sllm_slot_append`).  Token-id level, like `Inference.generateTokens`: text goes through the tokenizer outside.
"""
from __future__ import annotations

import dataclasses

import numpy as np

from .api import Engine, SamplingOptions


class ChatSession:
    def __init__(self, engine: Engine, slot: int = 0, eos: int = 32762):
        self.eng, self.slot, self.eos = engine, slot, eos
        self.user, self.assistant, self.end = eos + 1, eos + 2, eos + 3     # include/data/sft.h:18-26
        self.started = False
        self.need_end = False            # the stored history does not end in <|end|> yet
        self.dropped_history = 0         # how many times the context was restarted

    def history(self) -> np.ndarray:
        return self.eng.tokens(self.slot) if self.started else np.zeros(0, np.uint32)

    def say(self, user_ids, max_new_tokens: int, opt: SamplingOptions | None = None, draws=None) -> np.ndarray:
        """One turn: returns the reply's ids (without the token that ended it).  draws: [max_new_tokens]
        uniforms when opt.temperature > 0."""
        opt = dataclasses.replace(opt or SamplingOptions(), stop_token=self.end)
        ctx = self.eng.config.context_length
        prompt = np.concatenate([[self.user], np.asarray(user_ids, dtype=np.uint32), [self.end, self.assistant]]).astype(np.uint32)
        if prompt.size + max_new_tokens > ctx:
            raise ValueError("ChatSession.say: prompt and reply budget exceed context_length")
        held = self.history().size + (1 if self.need_end else 0)
        if not self.started or held + prompt.size + max_new_tokens > ctx:
            if self.started:
                self.dropped_history += 1          # docs/script.js:291-301: start a fresh context
            self.eng.slot_assign(self.slot, prompt)
            self.started = True
        else:
            extra = np.concatenate([[self.end], prompt]).astype(np.uint32) if self.need_end else prompt
            self.eng.slot_append(self.slot, extra)
        n_before = self.eng.tokens(self.slot).size
        d = None
        if opt.temperature > 0.0:
            live = self.eng.num_live()         # other sessions may hold higher slots of the same engine
            d = np.zeros((max_new_tokens, live), dtype=np.float64)
            d[:, self.slot] = np.asarray(draws, dtype=np.float64)[:max_new_tokens]
        self.eng.decode_loop(max_new_tokens, opt, d, eos=self.eos)
        toks = self.eng.tokens(self.slot)
        reply = toks[n_before:]
        if reply.size and reply[-1] == self.eos:   # the demo drops EOS and closes the turn with <|end|>
            self.eng.truncate(self.slot, toks.size - 1)
            reply, self.need_end = reply[:-1], True
        elif reply.size and reply[-1] == self.end:
            reply, self.need_end = reply[:-1], False
        else:
            self.need_end = True                   # budget exhausted
        return reply.copy()
