// C-ABI shim over the UNMODIFIED reference tokenizer (src/tokenizer.cpp) -- TEST INFRASTRUCTURE ONLY.
// Built by `make -C oracle ref` into oracle/_ref/libsllm_ref_tok.so and linked against the system's
// PCRE2 runtime; every id and byte it returns is produced by the reference's own encode/decode.
#include "tokenizer.h"

#include <cstring>
#include <string>
#include <vector>

extern "C" {
void* reftok_load(const char* path) {
    try { Tokenizer* t = new Tokenizer(); t->load(path); return t; } catch (...) { return nullptr; }
}
void reftok_free(void* t) { delete static_cast<Tokenizer*>(t); }
uint32_t reftok_eos(void* t) { return static_cast<Tokenizer*>(t)->getEosToken(); }
// returns the number of ids (may exceed cap: call again with a larger buffer)
uint64_t reftok_encode(void* t, const char* text, uint64_t n, uint32_t* out, uint64_t cap) {
    std::vector<Token> ids = static_cast<Tokenizer*>(t)->encode(std::string(text, n));
    for (uint64_t i = 0; i < ids.size() && i < cap; ++i) out[i] = ids[i];
    return ids.size();
}
int64_t reftok_decode(void* t, const uint32_t* ids, uint64_t n, char* out, uint64_t cap) {
    try {
        std::string s = static_cast<Tokenizer*>(t)->decode(std::vector<Token>(ids, ids + n));
        if (s.size() <= cap) std::memcpy(out, s.data(), s.size());
        return (int64_t)s.size();
    } catch (...) { return -1; }
}
}
