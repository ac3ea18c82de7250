// Reads length-prefixed texts from stdin (u32 length, bytes), writes for each the ids produced by
// Tokenizer::encode (u32 count, ids) and the bytes of Tokenizer::decode of those ids (u32 length, bytes).
#include "sllm_tokenizer.hpp"
#include "tokenizer.h"

#include <cstdio>

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    Tokenizer tok;
    tok.load(argv[1]);
    uint32_t n;
    while (std::fread(&n, 4, 1, stdin) == 1) {
        std::string text(n, '\0');
        if (n && std::fread(&text[0], 1, n, stdin) != n) return 3;
        const std::vector<uint32_t> ids = tok.encode(text);
        const uint32_t c = (uint32_t)ids.size();
        std::fwrite(&c, 4, 1, stdout);
        std::fwrite(ids.data(), 4, c, stdout);
        const std::string back = tok.decode(ids);
        const uint32_t m = (uint32_t)back.size();
        std::fwrite(&m, 4, 1, stdout);
        std::fwrite(back.data(), 1, m, stdout);
    }
    return 0;
}
