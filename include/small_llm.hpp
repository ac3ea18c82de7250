// small_llm.hpp -- the reference's C++ inference API over the C ABI of sllm.h (header only).
//
// A program written against small-llm's inference classes compiles against this header with
// the same names, fields, defaults and call sequence
//     Model model(cfg); model.to(Device::CUDA); model.enable_bf16(true);
//     load_checkpoint_weights(path, model); model.refresh_bf16_weights();
//     Inference inference(model, tokenizer); inference.generateTokens(ids, n, opt);
// (the sequence of src/main.cpp:37-63) and links with libsllm_b200.so.  What each class stands in
// for, by path inside the small-llm tree:
//     ModelConfig             include/config.h:6-47
//     Device, DType, Tensor   include/tensor.h:13-147   (host container only: logits and parameters)
//     Param, Model            include/model.h:12-50     (forward, parameters, config, to, bf16 switches)
//     TrainState, load_checkpoint_weights   include/checkpoint.h:9-17, src/checkpoint.cpp:57-102
//     SamplingOptions, Inference            include/inference.h:9-27, src/inference.cpp:21-183
//     Tokenizer               include/tokenizer.h:54-72 (interface; see the note at the class)
// Error behaviour follows the reference: std::invalid_argument for bad shapes and empty prompts,
// std::runtime_error for I/O, CUDA and non-finite logits, std::logic_error for calls in the wrong
// state.  There is no CPU execution path: forward and generate* throw std::logic_error until the
// model has been moved to Device::CUDA.
#pragma once

#include <cstdint>
#include <cstring>
#include <fstream>
#include <iostream>
#include <memory>
#include <random>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "sllm.h"

enum class Device { CPU, CUDA };
enum class DType { F32, BF16 };

struct ModelConfig {
    size_t vocab_size = 32768;
    size_t context_length = 2048;
    size_t num_layers = 16;
    size_t d_model = 640;
    size_t num_heads = 10;
    size_t head_dim() const { return d_model / num_heads; }
    size_t ffn_hidden = 1728;
    float rope_theta = 10000.0f;
    size_t totalParams() const {
        const size_t per_layer = 4 * d_model * d_model + 3 * d_model * ffn_hidden + 2 * d_model;
        return vocab_size * d_model + num_layers * per_layer + d_model;
    }
    uint32_t seed = 1234;
    float kRmsNormEps = 1e-5f;
};

// Host-side fp32 container with the accessors the inference path uses.
class Tensor {
public:
    Tensor() = default;
    explicit Tensor(const std::vector<size_t>& shape) : shape_(shape) { alloc(0.0f); }
    Tensor(const std::vector<size_t>& shape, float value) : shape_(shape) { alloc(value); }

    const std::vector<size_t>& shape() const { return shape_; }
    size_t ndim() const { return shape_.size(); }
    size_t numel() const { return data_ ? data_->size() : 0; }
    size_t size() const { return numel(); }
    size_t dim(size_t axis) const {
        if (axis >= shape_.size()) throw std::out_of_range("Tensor::dim: axis out of range");
        return shape_[axis];
    }
    Device device() const { return Device::CPU; }
    bool is_cuda() const { return false; }
    Tensor to(Device) const { return *this; }                 // results already live on the host
    DType dtype() const { return DType::F32; }
    float* data() { return data_ ? data_->data() : nullptr; }
    const float* data() const { return data_ ? data_->data() : nullptr; }
    float& operator[](size_t i) { return (*data_)[i]; }
    const float& operator[](size_t i) const { return (*data_)[i]; }
    void fill(float v) { if (data_) std::fill(data_->begin(), data_->end(), v); }
    Tensor reshaped(const std::vector<size_t>& s) const {
        size_t n = 1;
        for (size_t d : s) n *= d;
        if (n != numel()) throw std::invalid_argument("Tensor::reshaped: element count differs");
        Tensor t = *this;                                     // shares storage, like the reference's view
        t.shape_ = s;
        return t;
    }
    // global generator of include/tensor.h:82-85 (default seed 0)
    static std::mt19937& rng() { static std::mt19937 gen(0); return gen; }
    static void seed(uint32_t s) { rng().seed(s); }
    void randomNormal(float mean, float stddev) {
        std::normal_distribution<float> dist(mean, stddev);
        for (float& v : *data_) v = dist(rng());
    }

private:
    void alloc(float v) {
        size_t n = 1;
        for (size_t d : shape_) n *= d;
        data_ = std::make_shared<std::vector<float>>(n, v);
    }
    std::vector<size_t> shape_;
    std::shared_ptr<std::vector<float>> data_;
};

struct Param {
    std::string name;
    Tensor* value;
    Tensor* grad;            // always null here: training is outside this library
    bool decay;              // true for matrices, false for norm gains
    Tensor* shadow = nullptr;
};

namespace sllm_detail {
[[noreturn]] inline void raise(int code, const std::string& msg) {
    switch (code) {
        case SLLM_ERR_INVALID: throw std::invalid_argument(msg);
        case SLLM_ERR_STATE: throw std::logic_error(msg);
        default: throw std::runtime_error(msg);
    }
}
inline void check(int code, const sllm_engine* e) {
    if (code != SLLM_OK) raise(code, sllm_last_error(e));
}
}  // namespace sllm_detail

// ------------------------------------------------------------------------------- Model ---
class Model {
public:
    explicit Model(const ModelConfig& config) : config_(config) {
        if (config.num_heads == 0 || config.d_model != config.num_heads * config.head_dim())
            throw std::invalid_argument("Attention: d_model must equal num_heads * head_dim");
        const size_t D = config.d_model, F = config.ffn_hidden, L = config.num_layers;
        const float std_in = 0.02f;
        const float std_out = 0.02f / std::sqrt(2.0f * static_cast<float>(L));
        // registry and initialisation order of src/model.cpp:15-29,106-131, src/nn/attention.cpp:39-45,
        // src/nn/swiglu.cpp:17-22: embedding, then per block q k v out gate up down; gains 1
        add("embedding", {config.vocab_size, D}, true).randomNormal(0.0f, std_in);
        for (size_t i = 0; i < L; ++i) {
            const std::string p = "blocks." + std::to_string(i) + ".";
            add(p + "attn_norm", {D}, false).fill(1.0f);
            add(p + "attn.q", {D, D}, true).randomNormal(0.0f, std_in);
            add(p + "attn.k", {D, D}, true).randomNormal(0.0f, std_in);
            add(p + "attn.v", {D, D}, true).randomNormal(0.0f, std_in);
            add(p + "attn.out", {D, D}, true).randomNormal(0.0f, std_out);
            add(p + "ffn_norm", {D}, false).fill(1.0f);
            add(p + "ffn.gate", {D, F}, true).randomNormal(0.0f, std_in);
            add(p + "ffn.up", {D, F}, true).randomNormal(0.0f, std_in);
            add(p + "ffn.down", {F, D}, true).randomNormal(0.0f, std_out);
        }
        add("final_norm", {D}, false).fill(1.0f);
        sllm_default_engine_options(&options_);
        options_.weight_dtype = SLLM_WEIGHTS_F32;            // until enable_bf16(true), as in the reference
    }
    ~Model() { drop_engine(); }
    Model(const Model&) = delete;
    Model& operator=(const Model&) = delete;

    // token_ids [B, T] -> logits [B, T, vocab_size] fp32 (src/model.cpp:31-62)
    Tensor forward(const std::vector<uint32_t>& token_ids, size_t batch_size, size_t seq_len) {
        if (token_ids.size() != batch_size * seq_len)
            throw std::invalid_argument("Model::forward: token_ids.size() must equal batch_size * seq_len");
        if (seq_len > config_.context_length)
            throw std::invalid_argument("Model::forward: seq_len exceeds context_length");
        Tensor logits({batch_size, seq_len, config_.vocab_size});
        sllm_engine* e = engine();
        // rows are independent: more rows than the engine has sequence slots go through in groups
        const size_t group = options_.max_batch ? options_.max_batch : 1;
        for (size_t b0 = 0; b0 < batch_size; b0 += group) {
            const size_t nb = std::min(group, batch_size - b0);
            sllm_detail::check(sllm_forward_logits(e, token_ids.data() + b0 * seq_len, nb, seq_len,
                                                   logits.data() + b0 * seq_len * config_.vocab_size), e);
        }
        return logits;
    }

    // ops::cross_entropy(forward(token_ids), targets, num_valid) (src/ops/cross_entropy.cpp:14-54) without moving the
    // logits off the device; targets are ids, negative = position ignored, num_valid 0 = mean over all positions.
    // An extension: what a perplexity check of a checkpoint needs (exp of the returned loss).
    float evalLoss(const std::vector<uint32_t>& token_ids, const std::vector<int32_t>& targets, size_t batch_size, size_t seq_len,
                   size_t num_valid = 0) {
        if (token_ids.size() != batch_size * seq_len || targets.size() != token_ids.size())
            throw std::invalid_argument("Model::evalLoss: token_ids and targets must hold batch_size * seq_len entries");
        if (seq_len > config_.context_length)
            throw std::invalid_argument("Model::forward: seq_len exceeds context_length");
        sllm_engine* e = engine();
        const size_t group = options_.max_batch ? options_.max_batch : 1;
        if (batch_size <= group) {
            float loss = 0.f;
            sllm_detail::check(sllm_eval_loss(e, token_ids.data(), targets.data(), batch_size, seq_len, num_valid, &loss), e);
            return loss;
        }
        // more rows than sequence slots: per-group sums of the counted positions, recombined in double
        double total = 0.0;
        size_t counted = 0;
        for (size_t b0 = 0; b0 < batch_size; b0 += group) {
            const size_t nb = std::min(group, batch_size - b0);
            size_t n = 0;
            for (size_t i = b0 * seq_len; i < (b0 + nb) * seq_len; ++i) n += targets[i] >= 0;
            if (n == 0) continue;
            float loss = 0.f;
            sllm_detail::check(sllm_eval_loss(e, token_ids.data() + b0 * seq_len, targets.data() + b0 * seq_len, nb, seq_len, n, &loss), e);
            total += (double)loss * (double)n;
            counted += n;
        }
        return static_cast<float>(total / static_cast<double>(num_valid ? num_valid : batch_size * seq_len));
    }

    // every tensor in registry order; writing through Param::value takes effect at the next
    // forward / generate (or at refresh_bf16_weights())
    std::vector<Param> parameters() {
        dirty_ = true;
        std::vector<Param> out;
        for (size_t i = 0; i < names_.size(); ++i) out.push_back({names_[i], &values_[i], nullptr, decay_[i], nullptr});
        return out;
    }
    const ModelConfig& config() const { return config_; }

    void to(Device device) {
        on_cuda_ = device == Device::CUDA;
        if (!on_cuda_) drop_engine();
    }
    void enable_bf16(bool on) {
        if (on && !on_cuda_) throw std::logic_error("Model::enable_bf16: move the model to CUDA first");
        const uint32_t want = on ? SLLM_WEIGHTS_BF16 : SLLM_WEIGHTS_F32;
        if (want != options_.weight_dtype) drop_engine();
        options_.weight_dtype = want;
    }
    bool bf16() const { return options_.weight_dtype == SLLM_WEIGHTS_BF16; }
    void refresh_bf16_weights() { if (on_cuda_) { dirty_ = true; engine(); } }

    // ---- extensions -------------------------------------------------------------------------
    // engine shape (batch slots, KV pages, device); takes effect when the engine is next built
    void set_engine_options(const sllm_engine_options& o) {
        const uint32_t dt = options_.weight_dtype;
        drop_engine();
        options_ = o;
        options_.weight_dtype = dt;
    }
    const sllm_engine_options& engine_options() const { return options_; }
    // the C-ABI handle behind this model (built and loaded on first use)
    sllm_engine* engine() {
        if (!on_cuda_) throw std::logic_error("Model: this build has no CPU path; call to(Device::CUDA) first");
        if (!engine_) {
            sllm_model_config c;
            c.vocab_size = config_.vocab_size; c.context_length = config_.context_length;
            c.num_layers = config_.num_layers; c.d_model = config_.d_model; c.num_heads = config_.num_heads;
            c.ffn_hidden = config_.ffn_hidden; c.rope_theta = config_.rope_theta; c.rms_eps = config_.kRmsNormEps;
            sllm_detail::check(sllm_engine_create(&c, &options_, &engine_), nullptr);
            dirty_ = true;
        }
        if (dirty_) {
            for (size_t i = 0; i < names_.size(); ++i) {
                const std::vector<size_t>& s = values_[i].shape();
                const uint64_t dims[2] = {s[0], s.size() > 1 ? s[1] : 0};
                sllm_detail::check(sllm_set_param(engine_, names_[i].c_str(), values_[i].data(), dims,
                                                  static_cast<uint32_t>(s.size())), engine_);
            }
            dirty_ = false;
        }
        return engine_;
    }

private:
    Tensor& add(const std::string& name, const std::vector<size_t>& shape, bool decay) {
        names_.push_back(name);
        values_.emplace_back(shape);
        decay_.push_back(decay);
        return values_.back();
    }
    void drop_engine() {
        if (engine_) sllm_engine_destroy(engine_);
        engine_ = nullptr;
    }
    ModelConfig config_;
    std::vector<std::string> names_;
    std::vector<Tensor> values_;
    std::vector<bool> decay_;
    sllm_engine_options options_{};
    sllm_engine* engine_ = nullptr;
    bool on_cuda_ = false, dirty_ = true;
};

// --------------------------------------------------------------------------- checkpoint ---
struct TrainState {
    uint64_t step = 0;
    uint64_t data_position = 0;
};

// Weights-only load of the reference's checkpoint file (src/checkpoint.cpp:57-102): u64 step,
// u64 data position, u32 parameter count, then per parameter u32 name length, name, u32 ndim,
// ndim x u64 dims, fp32 data.  An optimizer tail, if present, is not read.
inline TrainState load_checkpoint_weights(const std::string& path, Model& model) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("load_checkpoint: cannot open " + path);
    auto pod = [&in](auto& v) { in.read(reinterpret_cast<char*>(&v), sizeof v); };
    TrainState state;
    pod(state.step);
    pod(state.data_position);
    uint32_t count = 0;
    pod(count);
    const std::vector<Param> params = model.parameters();
    if (count != params.size())
        throw std::runtime_error("load_checkpoint: parameter count differs (different model config?)");
    for (const Param& p : params) {
        uint32_t len = 0;
        pod(len);
        std::string name(in ? len : 0, '\0');
        in.read(name.data(), static_cast<std::streamsize>(name.size()));
        if (name != p.name)
            throw std::runtime_error("load_checkpoint: expected parameter '" + p.name + "', file has '" + name + "'");
        uint32_t ndim = 0;
        pod(ndim);
        std::vector<size_t> shape(in ? ndim : 0);
        for (size_t& d : shape) { uint64_t v = 0; pod(v); d = v; }
        if (shape != p.value->shape()) throw std::runtime_error("load_checkpoint: shape mismatch for '" + p.name + "'");
        in.read(reinterpret_cast<char*>(p.value->data()), static_cast<std::streamsize>(p.value->numel() * sizeof(float)));
    }
    if (!in) throw std::runtime_error("load_checkpoint: file truncated or corrupt");
    return state;
}

// ---------------------------------------------------------------------------- Tokenizer ---
// Interface of include/tokenizer.h:54-72 as far as the token loop needs it: the EOS id, the
// file loader (src/tokenizer.cpp:506-602: u32 next id, u64 n, n x (u32 id, u64 len, bytes),
// i32 merges, merges x (u32 a, u32 b, u32 new)) and decode (src/tokenizer.cpp:237-268).
// encode() needs the reference's Unicode-aware pre-tokenising regular expression (it uses
// PCRE2 for it); it is supplied by sllm_tokenizer.hpp when that header is included first,
// otherwise it throws std::logic_error.
using Token = uint32_t;

class Tokenizer {
public:
    Tokenizer() = default;
    void setMerges(int n) { num_merges_ = n; }
    Token getEosToken() const { return 256 + num_merges_; }
    size_t vocabSize() const { return getEosToken() + 1; }

    void load(const std::string& path) {
        std::ifstream in(path, std::ios::binary);
        if (!in) throw std::runtime_error("Failed to open tokenizer file");
        uint32_t next_id = 0;
        uint64_t n = 0;
        in.read(reinterpret_cast<char*>(&next_id), 4);
        in.read(reinterpret_cast<char*>(&n), 8);
        token_bytes_.clear();
        for (uint64_t i = 0; i < n && in; ++i) {
            uint32_t id = 0;
            uint64_t len = 0;
            in.read(reinterpret_cast<char*>(&id), 4);
            in.read(reinterpret_cast<char*>(&len), 8);
            if (len > (1u << 20)) throw std::runtime_error("tokenizer file corrupt");
            std::string bytes(len, '\0');
            in.read(bytes.data(), static_cast<std::streamsize>(len));
            token_bytes_[id] = std::move(bytes);
        }
        int32_t merges = 0;
        in.read(reinterpret_cast<char*>(&merges), 4);
        merges_.clear();
        for (int32_t i = 0; i < merges && in; ++i) {
            uint32_t abn[3];
            in.read(reinterpret_cast<char*>(abn), 12);
            merges_.push_back({abn[0], abn[1], abn[2]});
        }
        if (!in) throw std::runtime_error("tokenizer file truncated");
        num_merges_ = merges;
    }

    std::string decode(const std::vector<Token>& tokens) const {
        std::string out;
        for (Token t : tokens) {
            if (t == getEosToken()) { out += "\n<EOS>\n"; continue; }
            if (t > getEosToken()) {
                static const char* names[] = {"<|user|>", "<|assistant|>", "<|end|>", "<|reserved4|>", "<|reserved5|>"};
                const size_t k = t - getEosToken() - 1;
                out += k < 5 ? names[k] : "<|?|>";
                continue;
            }
            auto it = token_bytes_.find(t);
            if (it == token_bytes_.end())
                throw std::runtime_error("Unknown token ID during decode: " + std::to_string(t) +
                                         ", expected EOS: " + std::to_string(getEosToken()));
            out += it->second;
        }
        return out;
    }

    std::vector<Token> encode(const std::string& text) const {
#ifdef SLLM_TOKENIZER_ENCODE
        return sllm_tokenizer_encode(*this, text);
#else
        (void)text;
        throw std::logic_error("Tokenizer::encode: include sllm_tokenizer.hpp before small_llm.hpp");
#endif
    }

    struct Merge { Token a, b, merged; };
    const std::vector<Merge>& mergeList() const { return merges_; }

private:
    int num_merges_ = 32506;
    std::unordered_map<Token, std::string> token_bytes_;
    std::vector<Merge> merges_;
};

// chat template ids, include/data/sft.h:18-35
struct ChatTokens { uint32_t user, assistant, end, eos; };
inline ChatTokens chatTokens(const Tokenizer& tokenizer) {
    const uint32_t eos = tokenizer.getEosToken();
    return {eos + 1, eos + 2, eos + 3, eos};
}
inline std::vector<uint32_t> encodeChatPrompt(const Tokenizer& tokenizer, const std::string& user_text) {
    const ChatTokens ids = chatTokens(tokenizer);
    std::vector<uint32_t> tokens{ids.user};
    for (uint32_t id : tokenizer.encode(user_text)) tokens.push_back(id);
    tokens.push_back(ids.end);
    tokens.push_back(ids.assistant);
    return tokens;
}

// ---------------------------------------------------------------------------- Inference ---
struct SamplingOptions {
    float temperature = 0.7f;          // <= 0 means greedy
    float top_p = 0.8f;
    float repetition_penalty = 1.1f;   // 1.0 = off
    uint64_t seed = 1234;
    int64_t stop_token = -1;           // extra stop token; EOS always stops
};

class Inference {
public:
    Inference(Model& model, Tokenizer& tokenizer) : model_(model), tokenizer_(tokenizer) {}

    // Token ids in, token ids out (prompt + continuation): the token loop of
    // src/inference.cpp:21-165 on the GPU.  With a positive temperature and fp32 weights the ids
    // are the ones the reference draws from the same seed (std::mt19937_64 +
    // std::discrete_distribution consumption is reproduced).  With temperature <= 0 the reference
    // computes the arg-max but never appends it (its push_back sits inside the sampling branch,
    // src/inference.cpp:95-162); the arg-max IS appended here, unless SLLM_REFERENCE_GREEDY_QUIRK
    // is defined, in which case the prompt comes back unchanged as it does there.
    std::vector<uint32_t> generateTokenIds(std::vector<uint32_t> tokens, size_t max_new_tokens, SamplingOptions opt = {}) {
        if (tokens.empty()) throw std::invalid_argument("Inference::generate: prompt encoded to zero tokens");
        if (model_.config().context_length == 0)
            throw std::runtime_error("Inference::generate: context length must be greater than zero");
#ifdef SLLM_REFERENCE_GREEDY_QUIRK
        if (opt.temperature <= 0.0f) return tokens;
#endif
        sllm_engine* e = model_.engine();
        sllm_sampling s;
        s.temperature = opt.temperature; s.top_p = opt.top_p; s.repetition_penalty = opt.repetition_penalty;
        s.eos_token = tokenizer_.getEosToken(); s.stop_token = opt.stop_token; s.seed = opt.seed;
        const uint32_t len = static_cast<uint32_t>(tokens.size());
        std::vector<uint32_t> out(tokens.size() + max_new_tokens + 1);
        uint64_t n = 0;
        sllm_detail::check(sllm_generate(e, tokens.data(), &len, 1, max_new_tokens, &s, nullptr, out.data(), out.size(), &n), e);
        out.resize(n);
        return out;
    }

    // src/inference.cpp:21-173: decodes prompt + continuation, prints it and a rule, returns it
    std::string generateTokens(std::vector<uint32_t> tokens, size_t max_new_tokens, SamplingOptions opt = {}) {
        const std::string result = tokenizer_.decode(generateTokenIds(std::move(tokens), max_new_tokens, opt));
        std::cout << result << '\n';
        std::cout << "------------------------------------------------------------ \n";
        return result;
    }
    std::string generate(const std::string& prompt, size_t max_new_tokens, SamplingOptions opt = {}) {
        return generateTokens(tokenizer_.encode(prompt), max_new_tokens, opt);
    }
    // wraps the text in the chat template and stops at <|end|> (src/inference.cpp:180-183)
    std::string generateChat(const std::string& user_text, size_t max_new_tokens, SamplingOptions opt = {}) {
        opt.stop_token = chatTokens(tokenizer_).end;
        return generateTokens(encodeChatPrompt(tokenizer_, user_text), max_new_tokens, opt);
    }

private:
    Model& model_;
    Tokenizer& tokenizer_;
};

// Multi-turn chat on one engine slot with the KV cache carried across turns.  An extension: the reference's
// chat loop (src/main.cpp:46-62) sends every line as a fresh single-turn prompt.  The history rules are those
// of its browser demo (docs/script.js:288-305): a turn's context is the stored turns followed by
// <|user|> text <|end|> <|assistant|>; a finished turn is stored as prompt + reply + <|end|>; when history,
// prompt and reply budget no longer fit context_length, the history is dropped.  Only the new ids run
// through the model (sllm_slot_append); draws come from std::mt19937_64(opt.seed), one per step.
class ChatSession {
public:
    ChatSession(Model& model, Tokenizer& tokenizer, uint32_t slot = 0) : model_(model), tokenizer_(tokenizer), slot_(slot) {}

    // reply ids without the token that ended the turn
    std::vector<uint32_t> sayIds(const std::vector<uint32_t>& user_ids, size_t max_new_tokens, SamplingOptions opt = {}) {
        const ChatTokens ids = chatTokens(tokenizer_);
        const size_t ctx = model_.config().context_length;
        std::vector<uint32_t> prompt;
        prompt.push_back(ids.user);
        prompt.insert(prompt.end(), user_ids.begin(), user_ids.end());
        prompt.push_back(ids.end);
        prompt.push_back(ids.assistant);
        if (prompt.size() + max_new_tokens > ctx)
            throw std::invalid_argument("ChatSession::say: prompt and reply budget exceed context_length");
        sllm_engine* e = model_.engine();
        const size_t held = started_ ? tokens(e).size() + (need_end_ ? 1 : 0) : 0;
        if (!started_ || held + prompt.size() + max_new_tokens > ctx) {
            if (started_) ++dropped_history_;
            sllm_detail::check(sllm_slot_assign(e, slot_, prompt.data(), static_cast<uint32_t>(prompt.size())), e);
            started_ = true;
        } else {
            std::vector<uint32_t> extra;
            if (need_end_) extra.push_back(ids.end);
            extra.insert(extra.end(), prompt.begin(), prompt.end());
            sllm_detail::check(sllm_slot_append(e, slot_, extra.data(), static_cast<uint32_t>(extra.size())), e);
        }
        const size_t n_before = tokens(e).size();
        sllm_sampling s;
        s.temperature = opt.temperature; s.top_p = opt.top_p; s.repetition_penalty = opt.repetition_penalty;
        s.eos_token = ids.eos; s.stop_token = ids.end; s.seed = opt.seed;
        std::vector<double> draws;
        if (opt.temperature > 0.0f) {                      // [step][slot], this slot's column filled
            std::mt19937_64 rng(opt.seed + turns_);
            const size_t live = sllm_num_live(e);       // other sessions may hold higher slots of the same engine
            draws.assign(max_new_tokens * live, 0.0);
            for (size_t i = 0; i < max_new_tokens; ++i) draws[i * live + slot_] = std::generate_canonical<double, 53>(rng);
        }
        sllm_detail::check(sllm_decode_loop(e, max_new_tokens, &s, draws.empty() ? nullptr : draws.data()), e);
        ++turns_;
        std::vector<uint32_t> all = tokens(e);
        std::vector<uint32_t> reply(all.begin() + n_before, all.end());
        if (!reply.empty() && reply.back() == ids.eos) {   // the demo drops EOS and closes the turn with <|end|>
            sllm_detail::check(sllm_truncate(e, slot_, all.size() - 1), e);
            reply.pop_back(); need_end_ = true;
        } else if (!reply.empty() && reply.back() == ids.end) {
            reply.pop_back(); need_end_ = false;
        } else {
            need_end_ = true;                              // budget exhausted
        }
        return reply;
    }
    std::string say(const std::string& user_text, size_t max_new_tokens, SamplingOptions opt = {}) {
        return tokenizer_.decode(sayIds(tokenizer_.encode(user_text), max_new_tokens, opt));
    }
    size_t droppedHistory() const { return dropped_history_; }

private:
    std::vector<uint32_t> tokens(sllm_engine* e) {
        std::vector<uint32_t> out(2 * model_.config().context_length + 2);
        uint64_t n = 0;
        sllm_detail::check(sllm_get_tokens(e, slot_, out.data(), out.size(), &n), e);
        out.resize(n);
        return out;
    }
    Model& model_;
    Tokenizer& tokenizer_;
    uint32_t slot_;
    bool started_ = false, need_end_ = false;
    size_t dropped_history_ = 0;
    uint64_t turns_ = 0;
};
