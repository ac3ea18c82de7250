"""The header-only C++ layer (the reference's class names over the C ABI) on a GPU: a small program loads a
checkpoint, calls Model::forward, Inference::generateTokenIds and ChatSession::sayIds; its results are
compared with the oracle."""
import os
import subprocess

import numpy as np
import pytest

import small_llm_b200 as sl
from oracle.binding import OracleModel
from tests.helpers import MID, rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _read(f, dtype):
    n = int(np.frombuffer(f.read(8), dtype=np.uint64)[0])
    return np.frombuffer(f.read(4 * n), dtype=dtype)


def test_cpp_facade_on_gpu_matches_oracle(tmp_path):
    cfg = MID
    o = OracleModel(cfg)
    o.init_normal(12, 0.1)
    ckpt = str(tmp_path / "w.bin")
    o.save_checkpoint(ckpt, 3, 4)
    libdir = os.path.dirname(sl.lib_path())
    exe, res = str(tmp_path / "facade_gpu"), str(tmp_path / "out.bin")
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "facade_gpu.cpp"),
                    "-o", exe, "-L", libdir, "-lsllm_b200", f"-Wl,-rpath,{libdir}"], check=True)
    eos = 1000
    r = subprocess.run([exe, ckpt, res, str(cfg.vocab), str(cfg.context), str(cfg.layers), str(cfg.d_model), str(cfg.heads),
                        str(cfg.ffn), str(eos - 256)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    ids = np.array([(i * 7919 + 13) % 500 for i in range(2 * 37)], dtype=np.uint32)
    with open(res, "rb") as f:
        logits = _read(f, np.float32).reshape(2, 37, cfg.vocab)
        loss = float(np.frombuffer(f.read(4), dtype=np.float32)[0])
        sampled = _read(f, np.uint32)
        reply1 = _read(f, np.uint32)
        reply2 = _read(f, np.uint32)
    assert rel_err(logits, o.forward(ids, 2, 37)) <= 2e-5                      # fp32 weights
    from oracle.binding import cross_entropy
    targets = np.array([-1 if i % 5 == 0 else int(ids[(i + 1) % ids.size]) for i in range(ids.size)], dtype=np.int32)
    assert abs(loss - cross_entropy(o.forward(ids, 2, 37).reshape(74, cfg.vocab), targets, int((targets >= 0).sum()))) <= 2e-5
    ref = o.generate(ids[:21], 30, 0.8, 0.9, 1.2, seed=77, eos=eos)
    assert np.array_equal(sampled, ref)
    user, asst, end = eos + 1, eos + 2, eos + 3
    ctx1 = np.concatenate([[user], ids[:9], [end, asst]]).astype(np.uint32)
    g1 = o.generate(ctx1, 12, 0.0, 1.0, 1.0, eos=eos, stop=end)
    r1 = g1[ctx1.size:]
    r1 = r1[:-1] if r1[-1] in (eos, end) else r1
    assert np.array_equal(reply1, r1)
    ctx2 = np.concatenate([ctx1, r1, [end], [user], ids[9:20], [end, asst]]).astype(np.uint32)
    g2 = o.generate(ctx2, 12, 0.0, 1.0, 1.0, eos=eos, stop=end)
    r2 = g2[ctx2.size:]
    r2 = r2[:-1] if r2[-1] in (eos, end) else r2
    assert np.array_equal(reply2, r2)


def _tiny_tokenizer(path, n_merges=250):
    """A tokenizer file in the reference's format (src/tokenizer.cpp:443-602: u32 next id, u64 n, n x (u32 id, u64 len,
    bytes), i32 merges, merges x (u32 a, u32 b, u32 new)): the 256 byte tokens plus merges learnt greedily from a sample
    text.  Returns the id -> bytes table."""
    import struct
    sample = ("the cat sat on the mat and the other cat sat there too. what is on the mat? then the dog and the cat "
              "sat together on another mat, there and then. " * 4).encode()
    vocab = {i: bytes([i]) for i in range(256)}
    import re
    words = [list(w) for w in re.findall(rb" ?[a-z]+|[^a-z ]+| ", sample)]          # a word keeps its leading space, as the pre-tokeniser cuts it
    merges = []
    for new in range(256, 256 + n_merges):
        counts = {}
        for w in words:
            for a, b in zip(w, w[1:]):
                counts[(a, b)] = counts.get((a, b), 0) + 1
        if not counts:
            break
        (a, b), _ = max(counts.items(), key=lambda kv: (kv[1], -kv[0][0], -kv[0][1]))
        merges.append((a, b, new))
        vocab[new] = vocab[a] + vocab[b]
        for w in words:
            i = 0
            while i + 1 < len(w):
                if w[i] == a and w[i + 1] == b:
                    w[i:i + 2] = [new]
                else:
                    i += 1
    while len(merges) < n_merges:                                               # pad with merges that never apply
        new = 256 + len(merges)
        merges.append((0, 1, new))
        vocab[new] = b"\x00\x01"
    with open(path, "wb") as f:
        f.write(struct.pack("<IQ", 256 + n_merges, len(vocab)))
        for i, b in vocab.items():
            f.write(struct.pack("<IQ", i, len(b)) + b)
        f.write(struct.pack("<i", n_merges))
        for a, b, new in merges:
            f.write(struct.pack("<III", a, b, new))
    return vocab


def test_string_entry_points_with_a_tokenizer_file(tmp_path):
    """Inference::generate(text) and Inference::generateChat(text) of the C++ layer on the GPU with a tokenizer loaded
    from a file: the ids the prompt encoded to must decode back to the text, and the returned strings must be the
    decoded oracle streams (the reference's own seeded draws; chat: <|user|> text <|end|> <|assistant|>, stops at <|end|>)."""
    from tests.helpers import SMALL
    cfg = SMALL                                                  # vocabulary 512 = 256 bytes + 250 merges + EOS + 5 reserved ids
    o = OracleModel(cfg)
    o.init_normal(3, 0.2)
    ckpt, tokf = str(tmp_path / "w.bin"), str(tmp_path / "tokenizer.bin")
    o.save_checkpoint(ckpt, 0, 0)
    vocab = _tiny_tokenizer(tokf)
    eos = 506
    names = {507: b"<|user|>", 508: b"<|assistant|>", 509: b"<|end|>", 510: b"<|reserved4|>", 511: b"<|reserved5|>"}

    def decode(ids):
        return b"".join(b"\n<EOS>\n" if t == eos else names[t] if t > eos else vocab[int(t)] for t in ids)

    libdir = os.path.dirname(sl.lib_path())
    exe, res = str(tmp_path / "facade_text_gpu"), str(tmp_path / "out.bin")
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "facade_text_gpu.cpp"),
                    "-o", exe, "-L", libdir, "-lsllm_b200", f"-Wl,-rpath,{libdir}"], check=True)
    r = subprocess.run([exe, ckpt, tokf, res, str(cfg.vocab), str(cfg.context), str(cfg.layers), str(cfg.d_model), str(cfg.heads),
                        str(cfg.ffn)], capture_output=True)          # bytes: random weights generate arbitrary byte strings
    assert r.returncode == 0, r.stdout[-500:] + r.stderr[-500:]
    with open(res, "rb") as f:
        ids = _read(f, np.uint32)
        n = int(np.frombuffer(f.read(8), dtype=np.uint64)[0]); text_out = f.read(n)
        chat_ids = _read(f, np.uint32)
        n = int(np.frombuffer(f.read(8), dtype=np.uint64)[0]); chat_out = f.read(n)
    text = b"the cat sat on the mat, and then the other cat sat there too"
    assert decode(ids) == text and ids.size < len(text) // 2          # merges were applied
    ref = o.generate(ids, 20, 0.8, 0.9, 1.2, eos=eos, seed=4321)
    assert text_out == decode(ref)
    question = b"what is on the mat?"
    assert chat_ids[0] == 507 and list(chat_ids[-2:]) == [509, 508] and decode(chat_ids[1:-2]) == question
    ref = o.generate(chat_ids, 24, 0.8, 0.9, 1.2, eos=eos, stop=509, seed=4321)
    assert chat_out == decode(ref)
    assert text_out in r.stdout                                  # generateTokens prints what it returns (src/inference.cpp:167-169)
