"""Single-kernel entry points of the C ABI (device pointers in and out)."""
import numpy as np
import pytest

from oracle.binding import Config, prompt_ids
from small_llm_b200 import SllmError
from tests.helpers import MID, ODD, WIDE, make_pair

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


HD128 = Config(vocab=256, context=192, layers=1, d_model=256, heads=2, ffn=64)


@pytest.mark.parametrize("cfg,fp32", [(MID, False), (MID, True), (ODD, False), (ODD, True), (WIDE, False), (HD128, False),
                                      (HD128, True)],
                         ids=["hd32-bf16", "hd32-f32", "hd16-bf16", "hd16-f32", "hd64-bf16", "hd128-bf16", "hd128-f32"])
def test_streaming_attention_matches_split_kernel(cfg, fp32):
    """More than 64 tokens take the page-streaming kernel (each warp owns a quarter of every page); up to 64
    take the per-lane kernel.  Same queries, every position of a prompt that ends inside a page: the two
    must agree to rounding, whatever quarter of the last page a position falls in."""
    import torch
    o, eng = make_pair(cfg, seed=5, stddev=0.05, fp32=fp32, via_checkpoint=False)
    n_prompt = min(cfg.context - 3, 171)
    eng.prefill([prompt_ids(6, n_prompt, cfg.vocab)])
    n_tok = n_prompt
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(n_tok, cfg.d_model, device="cuda", generator=g)
    slot = torch.zeros(n_tok, dtype=torch.int32, device="cuda")
    pos = torch.arange(n_tok, dtype=torch.int32, device="cuda")
    layer = cfg.layers - 1
    out_stream = torch.full((n_tok, cfg.d_model), float("nan"), device="cuda")
    eng.k_attn_decode(layer, n_tok, q.data_ptr(), slot.data_ptr(), pos.data_ptr(), 1, out_stream.data_ptr())
    out_ref = torch.full((n_tok, cfg.d_model), float("nan"), device="cuda")
    for b in range(0, n_tok, 64):
        n = min(64, n_tok - b)
        eng.k_attn_decode(layer, n, q[b:].data_ptr(), slot[b:].data_ptr(), pos[b:].data_ptr(), 1, out_ref[b:].data_ptr())
    torch.cuda.synchronize()
    a, r = out_stream.cpu().numpy(), out_ref.cpu().numpy()
    assert np.isfinite(a).all()
    assert np.abs(a - r).max() <= 4e-6 * np.abs(r).max() + 1e-7
    assert np.array_equal(a[0], r[0])          # one key: the value row itself


def test_tensor_core_prefill_attention_matches_cuda_core_kernel(monkeypatch):
    """Prefill over several pages and ragged sequence lengths (tiles of 128, 128 and fewer queries; a tile that
    starts inside a page) with head_dim 64: the tcgen05 attention kernel against the oracle, and against the same
    engine with that kernel switched off."""
    import os
    cfg = Config(vocab=512, context=448, layers=2, d_model=128, heads=2, ffn=192)
    lens = [300, 129, 64, 17, 448]
    prompts = [prompt_ids(20 + i, n, cfg.vocab) for i, n in enumerate(lens)]
    o, eng = make_pair(cfg, seed=6, stddev=0.05, fp32=False, max_batch=5, via_checkpoint=False, max_chunk_tokens=512)
    eng.prefill(prompts)
    got = np.stack([eng.step_logits(i) for i in range(5)])
    monkeypatch.setenv("SLLM_NO_ATTN_TC", "1")
    _, eng2 = make_pair(cfg, seed=6, stddev=0.05, fp32=False, max_batch=5, via_checkpoint=False, max_chunk_tokens=512)
    eng2.prefill(prompts)
    old = np.stack([eng2.step_logits(i) for i in range(5)])
    ref = np.stack([o.forward(p, 1, p.size)[0, -1] for p in prompts])
    from tests.helpers import rel_err
    assert rel_err(got, ref) <= 2e-2
    assert rel_err(old, ref) <= 2e-2
    assert rel_err(got, old) <= 1e-2
    # every position of one sequence, chunked so that a chunk boundary falls inside a tile
    ids = prompts[0]
    all_rows = eng.forward_logits(ids, 1, ids.size)[0]
    assert rel_err(all_rows, o.forward(ids, 1, ids.size)[0]) <= 2e-2


def test_tensor_core_prefill_attention_full_context():
    """A prompt that fills a 2048-position context (32 KV pages, 16 query tiles per head, several prefill chunks):
    last-row logits and a few inner rows against the oracle; then three more tokens, which makes the window slide
    (every token re-runs the last 2048 ids from position 0)."""
    cfg = Config(vocab=512, context=2048, layers=1, d_model=128, heads=2, ffn=128)
    o, eng = make_pair(cfg, seed=11, stddev=0.05, fp32=False, max_batch=1, via_checkpoint=False, max_chunk_tokens=768)
    ids = prompt_ids(40, cfg.context, cfg.vocab)
    from tests.helpers import rel_err
    ref = o.forward(ids, 1, cfg.context)[0]
    got = eng.forward_logits(ids, 1, cfg.context)[0]
    for r in (0, 63, 64, 127, 128, 767, 768, 1500, 2047):
        assert rel_err(got[r], ref[r]) <= 2e-2, r
    from small_llm_b200 import SamplingOptions
    out = eng.generate([ids], 3, SamplingOptions(temperature=0.0, repetition_penalty=1.0), None, eos=cfg.vocab + 5)[0]
    assert out.size == cfg.context + 3
    window = out[-cfg.context - 1:-1]                          # what the last step saw, positions restarting at 0
    want = o.forward(window, 1, cfg.context)[0, -1]
    # the last token is the arg-max of the oracle's logits for that window unless the top two are within the tolerance
    top2 = np.sort(want)[-2:]
    assert out[-1] == int(np.argmax(want)) or (top2[1] - top2[0]) <= 2e-2 * np.abs(want).max()


def test_wide_projection_tiles_in_all_their_variants(monkeypatch):
    """A prefill chunk large enough for more projection tiles than SMs (4 x 2048 positions: 192 QKV and 352 gate/up
    tiles of 128 x 256, 128 tiles of 128 x 128 for the two residual projections): the persistent tile loop with the
    transposing epilogue (default), the same loop with the thread-per-row epilogue, and one tile per block, each
    against the oracle on the last position of every sequence and on every position of one, and against each other."""
    from tests.helpers import rel_err
    cfg = Config(vocab=1024, context=2048, layers=2, d_model=256, heads=4, ffn=704)
    prompts = [prompt_ids(60 + i, cfg.context, cfg.vocab) for i in range(4)]
    got = {}
    o = None
    for name, var in (("default", None), ("thread-per-row", "SLLM_NO_WIDE_EPI"), ("one tile per block", "SLLM_NO_PERSISTENT_TC")):
        if var:
            monkeypatch.setenv(var, "1")
        o, eng = make_pair(cfg, seed=12, stddev=0.05, fp32=False, max_batch=4, via_checkpoint=False, max_chunk_tokens=8192)
        if var:
            monkeypatch.delenv(var)
        eng.prefill(prompts)
        last = np.stack([eng.step_logits(i) for i in range(4)])
        rows = eng.forward_logits(prompts[1], 1, cfg.context)[0]
        got[name] = (last, rows)
        del eng
    ref_last = np.stack([o.forward(p, 1, p.size, row_from=p.size - 1)[0, -1] for p in prompts])
    ref_rows = o.forward(prompts[1], 1, cfg.context)[0]
    for name, (last, rows) in got.items():
        assert np.isfinite(last).all() and np.isfinite(rows).all(), name
        assert rel_err(last, ref_last) <= 2e-2, name
        assert rel_err(rows, ref_rows) <= 2e-2, name
    for name in ("thread-per-row", "one tile per block"):
        assert rel_err(got[name][0], got["default"][0]) <= 1e-2, name
        assert rel_err(got[name][1], got["default"][1]) <= 1e-2, name


@pytest.mark.parametrize("fp32", [True, False])
def test_attention_kernels_match_reference_op(fp32, golden_dir):
    """The decode attention kernels against the reference's own ops::attention (src/ops/attention.cpp:143-184): q, k, v
    and the expected output come from tests/golden/attention_op_ref.npz, written by the unmodified reference
    (1 x 2 heads x 200 positions x 32).  K and V go into a slot's cache through sllm_kv_write; query t attends keys
    0..t.  All three launch shapes are checked: the page-streaming kernel (200 tokens in one call), the split-K
    flash-decode kernel (chunks of 50 tokens, 1 and 4 splits) and its allocation-free variant.  fp32 cache: only the
    summation order differs (1e-5); bf16 cache: K and V are rounded to bf16 (2e-2)."""
    import os
    import torch
    g = np.load(os.path.join(golden_dir, "attention_op_ref.npz"))
    q, k, v, want = g["q"][0], g["k"][0], g["v"][0], g["out"][0]              # [H, T, hd]
    H, T, hd = q.shape
    cfg = Config(vocab=256, context=256, layers=1, d_model=H * hd, heads=H, ffn=64)
    o, eng = make_pair(cfg, seed=1, stddev=0.05, fp32=fp32, via_checkpoint=False)
    eng.prefill([prompt_ids(1, T, cfg.vocab)])                                  # the slot now holds pages for T positions
    rows = lambda a: np.ascontiguousarray(a.transpose(1, 0, 2).reshape(T, H * hd))      # [T][H * hd]
    eng.kv_write(0, 0, 0, rows(k), rows(v))
    k_back, v_back = eng.kv_read(0, 0, 0, T)
    if fp32:
        assert np.array_equal(k_back, rows(k)) and np.array_equal(v_back, rows(v))
    else:
        assert np.abs(k_back - rows(k)).max() <= 2 ** -8 * np.abs(k).max()
    qd = torch.from_numpy(rows(q)).cuda()
    slot = torch.zeros(T, dtype=torch.int32, device="cuda")
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    expect = rows(want)
    tol = 1e-5 if fp32 else 2e-2

    def check(out, what):
        torch.cuda.synchronize()
        a = out.cpu().numpy()
        assert np.isfinite(a).all(), what
        assert np.abs(a - expect).max() <= tol * np.abs(expect).max(), (what, float(np.abs(a - expect).max()))

    out = torch.full((T, H * hd), float("nan"), device="cuda")
    eng.k_attn_decode(0, T, qd.data_ptr(), slot.data_ptr(), pos.data_ptr(), 1, out.data_ptr())
    check(out, "streaming kernel")
    for splits, static in ((1, False), (4, False), (4, True)):
        out = torch.full((T, H * hd), float("nan"), device="cuda")
        step = 50 if not static else 25                                          # 25 tokens x 2 heads fit the fixed scratch
        for b in range(0, T, step):
            eng.k_attn_decode(0, step, qd[b:].data_ptr(), slot[b:].data_ptr(), pos[b:].data_ptr(), splits, out[b:].data_ptr(),
                              static_scratch=static)
        check(out, f"flash-decode kernel, {splits} splits, static={static}")
