// The string entry points of the C++ layer on a GPU: Tokenizer::load of a tokenizer file, Inference::generate(text)
// and Inference::generateChat(text) (src/inference.cpp:175-183, chat template of include/data/sft.h:18-35).
// Writes, for the Python test: the ids each prompt encoded to and the strings the two calls returned.
//   argv: checkpoint, tokenizer file, output file, vocab, context, layers, d_model, heads, ffn
#include <cstdlib>
#include <fstream>
#include <iostream>
#include "sllm_tokenizer.hpp"
#include "model.h"
#include "inference.h"
#include "checkpoint.h"

static void put_ids(std::ofstream& f, const std::vector<uint32_t>& v) {
    const uint64_t n = v.size();
    f.write(reinterpret_cast<const char*>(&n), 8);
    f.write(reinterpret_cast<const char*>(v.data()), n * 4);
}
static void put_str(std::ofstream& f, const std::string& s) {
    const uint64_t n = s.size();
    f.write(reinterpret_cast<const char*>(&n), 8);
    f.write(s.data(), n);
}

int main(int argc, char** argv) {
    if (argc < 10) return 2;
    ModelConfig cfg;
    cfg.vocab_size = std::atoi(argv[4]); cfg.context_length = std::atoi(argv[5]); cfg.num_layers = std::atoi(argv[6]);
    cfg.d_model = std::atoi(argv[7]); cfg.num_heads = std::atoi(argv[8]); cfg.ffn_hidden = std::atoi(argv[9]);
    Tokenizer tok;
    tok.load(argv[2]);
    if (tok.getEosToken() + 6 != cfg.vocab_size) return 3;           // EOS + the five reserved ids fill the vocabulary
    Model model(cfg);
    model.to(Device::CUDA);                                           // fp32 weights: the seeded streams equal the reference's
    load_checkpoint_weights(argv[1], model);
    Inference inf(model, tok);
    std::ofstream out(argv[3], std::ios::binary);
    const std::string text = "the cat sat on the mat, and then the other cat sat there too";
    SamplingOptions opt; opt.temperature = 0.8f; opt.top_p = 0.9f; opt.repetition_penalty = 1.2f; opt.seed = 4321;
    put_ids(out, tok.encode(text));
    put_str(out, inf.generate(text, 20, opt));
    const std::string question = "what is on the mat?";
    put_ids(out, encodeChatPrompt(tok, question));
    put_str(out, inf.generateChat(question, 24, opt));
    try { inf.generate("", 3, opt); return 4; } catch (const std::invalid_argument&) {}
    return 0;
}
