"""The allocation-free attention entry point (sllm_k_attn_decode_static).

Some hosts of this library cannot allocate device memory while they decode: a server that gave
the whole GPU to its own memory pool at start-up, or a decode thread that must not stall on the
device-wide synchronisation an allocation may cause.  For them the split-K flash-decode kernel is
offered with its scratch in a fixed device array inside the library.  This file checks, through
the C ABI, that it returns exactly what the ordinary entry point returns (same kernel, same
deterministic merge order, so bit-equal), on two calls in a row -- the second one finds the
array as the first one left it -- and that it refuses requests beyond its fixed size.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It also passes when run alone in a fresh process.
"""
import numpy as np
import pytest

from oracle.binding import prompt_ids
from small_llm_b200 import SllmError
from tests.helpers import MID, make_pair

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_allocated_scratch_twice():
    import torch
    cfg = MID
    o, eng = make_pair(cfg, seed=9, stddev=0.05, fp32=False, via_checkpoint=False)
    prompt = prompt_ids(4, 250, cfg.vocab)
    eng.prefill([prompt])
    gen = torch.Generator(device="cuda").manual_seed(7)
    n_tok = 5
    slot = torch.zeros(n_tok, dtype=torch.int32, device="cuda")
    for call, (positions, splits, layer) in enumerate([([249, 130, 64, 63, 0], 4, 0), ([17, 249, 200, 1, 128], 2, 2)]):
        q = torch.randn(n_tok, cfg.d_model, device="cuda", generator=gen)
        pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
        want = torch.full((n_tok, cfg.d_model), float("nan"), device="cuda")
        got = torch.full((n_tok, cfg.d_model), float("nan"), device="cuda")
        torch.cuda.synchronize()
        eng.k_attn_decode(layer, n_tok, q.data_ptr(), slot.data_ptr(), pos.data_ptr(), splits, want.data_ptr())
        torch.cuda.synchronize()
        eng.k_attn_decode(layer, n_tok, q.data_ptr(), slot.data_ptr(), pos.data_ptr(), splits, got.data_ptr(),
                          static_scratch=True)
        torch.cuda.synchronize()
        assert torch.isfinite(want).all() and torch.isfinite(got).all(), call
        # tolerance of the attention tests is 2e-6 relative; the two paths are in fact bit-equal
        assert np.array_equal(got.cpu().numpy(), want.cpu().numpy()), call


def test_static_scratch_refuses_oversized_requests():
    import torch
    cfg = MID                                                  # 4 heads: 17 tokens * 4 heads > 64 pairs
    o, eng = make_pair(cfg, seed=9, stddev=0.05, fp32=False, via_checkpoint=False)
    eng.prefill([prompt_ids(4, 20, cfg.vocab)])
    n_tok = 17
    q = torch.zeros(n_tok, cfg.d_model, device="cuda")
    slot = torch.zeros(n_tok, dtype=torch.int32, device="cuda")
    pos = torch.zeros(n_tok, dtype=torch.int32, device="cuda")
    out = torch.zeros(n_tok, cfg.d_model, device="cuda")
    with pytest.raises(SllmError, match="exceeds the fixed scratch"):
        eng.k_attn_decode(0, n_tok, q.data_ptr(), slot.data_ptr(), pos.data_ptr(), 2, out.data_ptr(), static_scratch=True)
