// Drives the header-only C++ layer on a GPU: checkpoint load, Model::forward, Inference::generateTokenIds (seeded),
// ChatSession (two greedy turns).  Results go to a binary file the Python test compares with the oracle.
//   argv: checkpoint path, output path, vocab, context, layers, d_model, heads, ffn, n_merges
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include "config.h"
#include "model.h"
#include "inference.h"
#include "checkpoint.h"

static void put(std::ofstream& f, const std::vector<uint32_t>& v) {
    const uint64_t n = v.size();
    f.write(reinterpret_cast<const char*>(&n), 8);
    f.write(reinterpret_cast<const char*>(v.data()), n * 4);
}

int main(int argc, char** argv) {
    if (argc < 10) return 2;
    ModelConfig cfg;
    cfg.vocab_size = std::atoi(argv[3]); cfg.context_length = std::atoi(argv[4]); cfg.num_layers = std::atoi(argv[5]);
    cfg.d_model = std::atoi(argv[6]); cfg.num_heads = std::atoi(argv[7]); cfg.ffn_hidden = std::atoi(argv[8]);
    Model model(cfg);
    model.to(Device::CUDA);                                    // fp32 weights: enable_bf16 is not called
    const TrainState st = load_checkpoint_weights(argv[1], model);
    if (st.step != 3 || st.data_position != 4) return 3;
    Tokenizer tok; tok.setMerges(std::atoi(argv[9]));          // EOS = 256 + merges
    std::ofstream out(argv[2], std::ios::binary);

    std::vector<uint32_t> ids;
    for (uint32_t i = 0; i < 2 * 37; ++i) ids.push_back((i * 7919u + 13u) % 500u);
    Tensor logits = model.forward(ids, 2, 37);
    if (logits.ndim() != 3 || logits.dim(0) != 2 || logits.dim(1) != 37 || logits.dim(2) != cfg.vocab_size) return 4;
    const uint64_t n = logits.numel();
    out.write(reinterpret_cast<const char*>(&n), 8);
    out.write(reinterpret_cast<const char*>(logits.data()), n * 4);

    std::vector<int32_t> targets(ids.size());
    for (size_t i = 0; i < ids.size(); ++i) targets[i] = (i % 5 == 0) ? -1 : (int32_t)ids[(i + 1) % ids.size()];
    size_t n_valid = 0;
    for (int32_t v : targets) n_valid += v >= 0;
    const float loss = model.evalLoss(ids, targets, 2, 37, n_valid);       // two rows on an engine with one slot: two groups
    out.write(reinterpret_cast<const char*>(&loss), 4);

    Inference inf(model, tok);
    SamplingOptions opt; opt.temperature = 0.8f; opt.top_p = 0.9f; opt.repetition_penalty = 1.2f; opt.seed = 77;
    std::vector<uint32_t> prompt(ids.begin(), ids.begin() + 21);
    put(out, inf.generateTokenIds(prompt, 30, opt));

    ChatSession chat(model, tok);
    SamplingOptions greedy; greedy.temperature = 0.0f; greedy.repetition_penalty = 1.0f;
    put(out, chat.sayIds(std::vector<uint32_t>(ids.begin(), ids.begin() + 9), 12, greedy));
    put(out, chat.sayIds(std::vector<uint32_t>(ids.begin() + 9, ids.begin() + 20), 12, greedy));
    if (chat.droppedHistory() != 0) return 5;
    try { inf.generateTokenIds({}, 3); return 6; } catch (const std::invalid_argument&) {}
    try { model.forward(ids, 1, 37); return 7; } catch (const std::invalid_argument&) {}
    std::cout << "ok\n";
    return 0;
}
