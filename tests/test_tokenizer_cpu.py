"""Tokenizer::encode / decode of the C++ layer (include/sllm_tokenizer.hpp, no PCRE2) against the
reference's own tokenizer compiled from its source and linked to the PCRE2 runtime
(oracle/_ref/libsllm_ref_tok.so).  Needs the reference's tokenizer/tokenizer.bin, so it runs only where
the reference tree is present."""
import ctypes as C
import os
import random
import struct
import subprocess

import numpy as np
import pytest

import small_llm_b200 as sl
from oracle import binding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOK_BIN = os.path.join(binding.REF_TREE, "tokenizer", "tokenizer.bin")
REF_TOK_SO = os.path.join(ROOT, "oracle", "_ref", "libsllm_ref_tok.so")

pytestmark = pytest.mark.skipif(not (os.path.exists(TOK_BIN) and os.path.exists(REF_TOK_SO)),
                                reason="reference tokenizer (tokenizer.bin + compiled library) not on this machine")


def _texts():
    fixed = ["Hello world!  It's 2024, isn't it?\n\n  naïve café 你好 \t x", "", " ", "  ", "a", " a", "  a  ",
             "we'll they've I'm he'd she's don't 'quoted' 'll 'RE", "x\n\ny\r\n z w q　", "123 4567 ٣٤ Ⅷ ½ x²",
             "foo_bar-baz@ex.com #tag $5.00 50%", "tab\tsep\t\tend\t", "emoji 🙂🙂 ok", "\n", " \n", "\n a", "end  ",
             "<|user|> hi <|end|>", "The quick brown fox jumps over the lazy dog. " * 20]
    rnd = random.Random(0)
    pool = [chr(c) for c in list(range(32, 127)) + [9, 10, 13, 0xA0, 0x85, 0x1680, 0x180E, 0x2003, 0x2028, 0x3000, 0xE9,
                                                     0x3B1, 0x416, 0x4E2D, 0x661, 0x2167, 0xBD, 0x1F600, 0x200B, 0x301,
                                                     0xB2, 0x5D0, 0xFF10, 0xFEFF]]
    for _ in range(1500):
        k = rnd.randint(1, 40)
        fixed.append("".join(rnd.choice(pool) if rnd.random() < 0.5 else rnd.choice(" a1'\n.,") for _ in range(k)))
    return fixed


def test_encode_decode_match_reference_tokenizer(tmp_path):
    libdir = os.path.dirname(sl.lib_path())
    exe = str(tmp_path / "tokcli")
    subprocess.run(["g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "tokenizer_cli.cpp"),
                    "-o", exe, "-L", libdir, "-lsllm_b200", f"-Wl,-rpath,{libdir}"], check=True)
    ref = C.CDLL(REF_TOK_SO)
    ref.reftok_load.restype = C.c_void_p
    ref.reftok_load.argtypes = [C.c_char_p]
    ref.reftok_encode.restype = C.c_uint64
    ref.reftok_encode.argtypes = [C.c_void_p, C.c_char_p, C.c_uint64, C.POINTER(C.c_uint32), C.c_uint64]
    ref.reftok_decode.restype = C.c_int64
    ref.reftok_decode.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_uint64, C.c_char_p, C.c_uint64]
    ref.reftok_eos.restype = C.c_uint32
    ref.reftok_eos.argtypes = [C.c_void_p]
    t = ref.reftok_load(TOK_BIN.encode())
    assert t and ref.reftok_eos(t) == 32762
    texts = [x.encode() for x in _texts()]
    inp = b"".join(struct.pack("<I", len(x)) + x for x in texts)
    out = subprocess.run([exe, TOK_BIN], input=inp, capture_output=True, check=True).stdout
    pos = 0
    for x in texts:
        (c,) = struct.unpack_from("<I", out, pos); pos += 4
        ids = np.frombuffer(out, dtype="<u4", count=c, offset=pos).copy(); pos += 4 * c
        (m,) = struct.unpack_from("<I", out, pos); pos += 4
        back = out[pos:pos + m]; pos += m
        want = np.zeros(len(x) + 8, np.uint32)
        n = ref.reftok_encode(t, x, len(x), want.ctypes.data_as(C.POINTER(C.c_uint32)), want.size)
        assert ids.tolist() == want[:n].tolist(), x
        buf = C.create_string_buffer(len(x) + 64)
        k = ref.reftok_decode(t, want.ctypes.data_as(C.POINTER(C.c_uint32)), n, buf, len(x) + 64)
        assert back == buf.raw[:k] == x
