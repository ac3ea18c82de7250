"""Continuous batching around the batched decode step.

The reference generates one sequence per call; at batch 512 a decode loop that waits for its longest
sequence wastes the slots of those that stopped early (EOS, stop token, budget).  This scheduler keeps the
slots of one engine full: it decodes in short bursts on the device, collects the slots that stopped,
parks them and assigns the next waiting prompt to the freed slot while the other slots keep their KV cache
and sampler state.  Each request's tokens are exactly what a single `generate` call would have produced
(stop rules of src/inference.cpp:158-160; draws are indexed by the request's own step number).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .api import Engine, SamplingOptions


@dataclass
class Request:
    prompt: np.ndarray
    max_new_tokens: int
    draws: np.ndarray | None = None          # [max_new_tokens] uniforms in [0,1); None = greedy options only
    tokens: np.ndarray | None = None         # result: prompt + continuation
    _made: int = field(default=0, repr=False)


class ContinuousBatcher:
    def __init__(self, engine: Engine, opt: SamplingOptions, eos: int = 32762, burst: int = 16):
        self.eng, self.opt, self.eos, self.burst = engine, opt, eos, burst
        self.n_slots = engine.options.max_batch

    def run(self, requests: list[Request]) -> list[Request]:
        eng, ctx = self.eng, self.eng.config.context_length
        waiting = list(range(len(requests)))
        slot_req: list[int | None] = [None] * self.n_slots
        eng.reset()
        sampled = self.opt.temperature > 0.0

        def fill():
            for s in range(self.n_slots):
                if slot_req[s] is None and waiting:
                    r = waiting.pop(0)
                    eng.slot_assign(s, requests[r].prompt)
                    slot_req[s] = r

        fill()
        while any(r is not None for r in slot_req):
            live = eng.num_live()              # the engine reads draws as [steps][its live-slot range]
            steps = self.burst
            draws = None
            if sampled:
                draws = np.zeros((steps, live), dtype=np.float64)
                for s in range(live):
                    r = slot_req[s]
                    if r is None:
                        continue
                    d = np.asarray(requests[r].draws, dtype=np.float64)[requests[r]._made:requests[r]._made + steps]
                    draws[: d.size, s] = d
            eng.decode_loop(steps, self.opt, draws, eos=self.eos)
            flags = eng.finished(live)
            for s in range(live):
                r = slot_req[s]
                if r is None:
                    continue
                req = requests[r]
                toks = eng.tokens(s)
                made = toks.size - req.prompt.size
                req._made = made
                stopped = flags[s] != 0
                if made >= req.max_new_tokens or stopped:
                    keep = req.prompt.size + min(made, req.max_new_tokens)
                    out = toks[:keep]
                    # a stop token inside the budget ends the sequence there (it is kept, as in the reference)
                    gen = out[req.prompt.size:]
                    hits = np.nonzero((gen == self.eos) | (gen == np.uint32(self.opt.stop_token & 0xFFFFFFFF) if self.opt.stop_token >= 0 else False))[0]
                    if hits.size:
                        out = out[: req.prompt.size + hits[0] + 1]
                    req.tokens = out.copy()
                    eng.slot_release(s)
                    slot_req[s] = None
            fill()
        return requests
