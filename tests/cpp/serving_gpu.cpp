// Drives include/sllm_serving.hpp on a GPU: a ContinuousBatcher with more sampled requests than slots, and a
// ShardedInference of two engines (two host threads) on the devices given.  Every token stream goes to a binary file
// that the Python test compares with the oracle's single-sequence generation of the same request.
//   argv: checkpoint path, output path, vocab, context, layers, d_model, heads, ffn, eos, device ordinals ("0,0")
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <sstream>
#include "sllm_serving.hpp"
#include "checkpoint.h"

static void put(std::ofstream& f, const std::vector<uint32_t>& v) {
    const uint64_t n = v.size();
    f.write(reinterpret_cast<const char*>(&n), 8);
    f.write(reinterpret_cast<const char*>(v.data()), n * 4);
}
static std::vector<uint32_t> prompt_of(uint32_t r) {
    std::vector<uint32_t> p(5 + 7 * r);
    for (uint32_t i = 0; i < p.size(); ++i) p[i] = (r * 131u + i * 7919u + 13u) % 1000u;
    return p;
}
static std::vector<double> draws_of(uint32_t seed, size_t n) {         // float(mt19937() >> 8) * 2^-24, as the oracle's generator
    std::mt19937 g(seed);
    std::vector<double> d(n);
    for (auto& v : d) v = static_cast<double>(static_cast<float>(g() >> 8) * (1.0f / 16777216.0f));
    return d;
}

int main(int argc, char** argv) {
    if (argc < 11) return 2;
    ModelConfig cfg;
    cfg.vocab_size = std::atoi(argv[3]); cfg.context_length = std::atoi(argv[4]); cfg.num_layers = std::atoi(argv[5]);
    cfg.d_model = std::atoi(argv[6]); cfg.num_heads = std::atoi(argv[7]); cfg.ffn_hidden = std::atoi(argv[8]);
    const uint32_t eos = static_cast<uint32_t>(std::atoi(argv[9]));
    std::vector<int> devices;
    { std::stringstream ss(argv[10]); std::string t; while (std::getline(ss, t, ',')) devices.push_back(std::atoi(t.c_str())); }
    std::ofstream out(argv[2], std::ios::binary);
    const std::string ckpt = argv[1];

    {   // continuous batching: 7 sampled requests through 3 slots, budgets chosen so that the highest slot drains early
        Model model(cfg);
        sllm_engine_options o;
        sllm_default_engine_options(&o);
        o.max_batch = 3; o.device = devices[0];
        model.set_engine_options(o);
        model.to(Device::CUDA);                                // fp32 weights: the streams must equal the oracle's
        load_checkpoint_weights(ckpt, model);
        SamplingOptions opt; opt.temperature = 0.9f; opt.top_p = 0.9f; opt.repetition_penalty = 1.1f;
        const size_t budgets[7] = {30, 22, 4, 17, 9, 25, 12};
        std::vector<BatchRequest> reqs(7);
        for (uint32_t r = 0; r < 7; ++r) { reqs[r].prompt = prompt_of(r); reqs[r].max_new_tokens = budgets[r]; reqs[r].draws = draws_of(70 + r, budgets[r]); }
        ContinuousBatcher(model, eos, opt, 5).run(reqs);
        for (const auto& r : reqs) put(out, r.tokens);
    }
    {   // sharding: 5 greedy prompts over the given devices, one engine and one host thread each
        ShardedInference sharded(cfg, devices, 2, false, [&](Model& m) { load_checkpoint_weights(ckpt, m); });
        std::vector<std::vector<uint32_t>> prompts;
        for (uint32_t r = 0; r < 5; ++r) prompts.push_back(prompt_of(10 + r));
        SamplingOptions greedy; greedy.temperature = 0.0f; greedy.repetition_penalty = 1.0f;
        for (const auto& t : sharded.generateTokenIds(prompts, 12, eos, greedy)) put(out, t);
        // and sampled, with supplied draws
        SamplingOptions opt; opt.temperature = 0.8f; opt.top_p = 0.95f; opt.repetition_penalty = 1.15f;
        std::vector<std::vector<double>> draws;
        for (uint32_t r = 0; r < 5; ++r) draws.push_back(draws_of(90 + r, 12));
        for (const auto& t : sharded.generateTokenIds(prompts, 12, eos, opt, draws)) put(out, t);
    }
    std::cout << "ok\n";
    return 0;
}
