"""Single-kernel entry points of the C ABI (device pointers in and out)."""
import numpy as np
import pytest

from oracle.binding import prompt_ids
from small_llm_b200 import SllmError
from tests.helpers import MID, make_pair

pytestmark = pytest.mark.gpu


def _setup(n_tok=3):
    import torch
    cfg = MID
    o, eng = make_pair(cfg, seed=9, stddev=0.05, fp32=False, via_checkpoint=False)
    prompt = prompt_ids(4, 200, cfg.vocab)
    eng.prefill([prompt])                                     # fills slot 0's KV pages of every layer
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(n_tok, cfg.d_model, device="cuda", generator=g)
    slot = torch.zeros(n_tok, dtype=torch.int32, device="cuda")
    pos = torch.tensor([199, 64, 0][:n_tok], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    return torch, cfg, eng, q, slot, pos


def test_attention_kernel_split_invariance_and_checks():
    torch, cfg, eng, q, slot, pos = _setup()
    outs = []
    for splits in (1, 2, 4):
        out = torch.full((q.shape[0], cfg.d_model), float("nan"), device="cuda")
        eng.k_attn_decode(1, q.shape[0], q.data_ptr(), slot.data_ptr(), pos.data_ptr(), splits, out.data_ptr())
        torch.cuda.synchronize()
        assert torch.isfinite(out).all()
        outs.append(out.cpu().numpy())
    assert np.abs(outs[1] - outs[0]).max() <= 2e-6 * np.abs(outs[0]).max() + 1e-7
    assert np.abs(outs[2] - outs[0]).max() <= 2e-6 * np.abs(outs[0]).max() + 1e-7
    # position 0 attends a single key: the output is that key's value row, whatever q is
    q2 = q.clone()
    q2[2] *= -3.0
    out2 = torch.empty_like(q)
    eng.k_attn_decode(1, 3, q2.data_ptr(), slot.data_ptr(), pos.data_ptr(), 1, out2.data_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(out2[2].cpu().numpy(), outs[0][2])
    with pytest.raises(ValueError, match="layer out of range"):
        eng.k_attn_decode(cfg.layers, 3, q.data_ptr(), slot.data_ptr(), pos.data_ptr(), 1, out2.data_ptr())
    with pytest.raises(ValueError, match="n_splits"):
        eng.k_attn_decode(0, 3, q.data_ptr(), slot.data_ptr(), pos.data_ptr(), 33, out2.data_ptr())
    with pytest.raises(ValueError, match="null device pointer"):
        eng.k_attn_decode(0, 3, 0, slot.data_ptr(), pos.data_ptr(), 1, out2.data_ptr())
