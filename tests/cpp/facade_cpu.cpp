// CPU-side check of the C++ layer (include/small_llm.hpp): it compiles from the reference's own
// include names, keeps the reference's error types, and refuses to compute without a GPU.
#include "model.h"
#include "inference.h"
#include "checkpoint.h"
int main() {
    ModelConfig cfg; cfg.vocab_size = 512; cfg.context_length = 64; cfg.num_layers = 2; cfg.d_model = 64; cfg.num_heads = 2; cfg.ffn_hidden = 96;
    Model model(cfg);
    try { model.enable_bf16(true); return 1; } catch (const std::logic_error&) {}
    try { model.forward({1,2,3}, 1, 3); return 2; } catch (const std::logic_error&) {}
    try { model.forward({1,2,3}, 1, 4); return 3; } catch (const std::invalid_argument&) {}
    if (model.parameters().size() != 20) return 4;
    Tokenizer tok; Inference inf(model, tok);
    try { inf.generateTokens({}, 3); return 5; } catch (const std::invalid_argument&) {}
    ChatSession chat(model, tok);
    try { chat.sayIds(std::vector<uint32_t>(80, 1u), 8); return 7; } catch (const std::invalid_argument&) {}   // does not fit 64 positions
    model.to(Device::CUDA);
    try { model.forward({1,2,3}, 1, 3); return 6; } catch (const std::runtime_error& e) { std::cout << e.what() << "\n"; }
    return 0;
}
