// Writes the initial weights of the C++ layer's Model(config) after Tensor::seed(seed) to a file, parameter by
// parameter in registry order: u32 count, then per parameter u32 name length, name, u64 element count, fp32 data.
// The test compares them with the reference constructor's weights (src/model.cpp:15-29).
#include <cstdio>
#include <cstdlib>
#include "model.h"
int main(int argc, char** argv) {
    if (argc < 3) return 2;
    ModelConfig cfg; cfg.vocab_size = 512; cfg.context_length = 64; cfg.num_layers = 2; cfg.d_model = 64; cfg.num_heads = 2; cfg.ffn_hidden = 96;
    Tensor::seed(static_cast<uint32_t>(std::atoi(argv[2])));
    Model model(cfg);
    FILE* f = std::fopen(argv[1], "wb");
    if (!f) return 3;
    const std::vector<Param> ps = model.parameters();
    const uint32_t n = static_cast<uint32_t>(ps.size());
    std::fwrite(&n, 4, 1, f);
    for (const Param& p : ps) {
        const uint32_t nl = static_cast<uint32_t>(p.name.size());
        const uint64_t ne = p.value->numel();
        std::fwrite(&nl, 4, 1, f); std::fwrite(p.name.data(), 1, nl, f);
        std::fwrite(&ne, 8, 1, f); std::fwrite(p.value->data(), 4, ne, f);
    }
    std::fclose(f);
    return 0;
}
