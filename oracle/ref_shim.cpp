// C-ABI shim over the UNMODIFIED small-llm reference sources (CPU path, USE_CUDA undefined).
//
// TEST INFRASTRUCTURE ONLY.  This file is compiled together with the reference's own
// translation units (see oracle/Makefile) into oracle/_ref/libsllm_ref*.so.  It contains
// no model arithmetic of its own: every number it returns is produced by the reference's
// Model::forward / ops::* / Inference::generateTokens.  Only tests, the smoke check and
// the CPU-baseline legs of the benchmark may load the resulting library.
//
// The one thing the reference cannot link here is its tokenizer (it needs the PCRE2
// development header).  The token loop only uses Tokenizer::getEosToken() (inline) and
// Tokenizer::decode() for the final printout, so this file supplies stand-in definitions
// of encode/decode that spell token ids as decimal text; that is how the ids drawn by the
// reference's sampler are recovered from the std::string that generateTokens returns.
#include "checkpoint.h"
#include "inference.h"
#include "model.h"
#include "ops/attention.h"
#include "ops/cross_entropy.h"
#include "ops/elementwise.h"
#include "ops/embedding.h"
#include "ops/matmul.h"
#include "ops/rmsnorm.h"
#include "ops/rope.h"
#include "ops/softmax.h"
#include "tokenizer.h"

#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

// ---- stand-in tokenizer text codec (ids <-> "12 345 6") -------------------------------
std::vector<Token> Tokenizer::encode(const std::string& text) const {
    std::vector<Token> ids;
    std::istringstream in(text);
    unsigned long v;
    while (in >> v) ids.push_back(static_cast<Token>(v));
    return ids;
}
std::string Tokenizer::decode(const std::vector<Token>& tokens) const {
    std::string s;
    for (Token t : tokens) { s += std::to_string(t); s += ' '; }
    return s;
}

namespace {
thread_local std::string g_err;
int fail(const std::exception& e, int code) { g_err = e.what(); return code; }

ModelConfig make_cfg(const uint64_t* c, float theta, float eps) {
    ModelConfig cfg;
    cfg.vocab_size = c[0]; cfg.context_length = c[1]; cfg.num_layers = c[2];
    cfg.d_model = c[3];    cfg.num_heads = c[4];      cfg.ffn_hidden = c[5];
    cfg.rope_theta = theta; cfg.kRmsNormEps = eps;
    return cfg;
}
Tensor wrap(const float* p, std::vector<size_t> shape) {
    Tensor t(shape);
    std::memcpy(t.data(), p, t.numel() * sizeof(float));
    return t;
}
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

// cfg = {vocab, context, layers, d_model, heads, ffn_hidden}
void* ref_model_create(const uint64_t* cfg, float theta, float eps) {
    try { return new Model(make_cfg(cfg, theta, eps)); }
    catch (const std::exception& e) { fail(e, 1); return nullptr; }
}
// The reference's own initialisation: Tensor::seed(seed), then Model::Model (src/model.cpp:15-29) draws every
// matrix from the global generator in construction order.
void* ref_model_create_seeded(const uint64_t* cfg, float theta, float eps, uint32_t seed) {
    try { Tensor::seed(seed); return new Model(make_cfg(cfg, theta, eps)); }
    catch (const std::exception& e) { fail(e, 1); return nullptr; }
}
void ref_model_destroy(void* m) { delete static_cast<Model*>(m); }

// Benchmark initialisation: reseed the reference's global generator, then every matrix
// N(0, std) in registry order through the reference's own Tensor::randomNormal; gains 1.
int ref_model_init_normal(void* m, uint32_t seed, float stddev) {
    try {
        Tensor::seed(seed);
        for (const Param& p : static_cast<Model*>(m)->parameters()) {
            if (p.decay) p.value->randomNormal(0.0f, stddev);
            else p.value->fill(1.0f);
        }
        return 0;
    } catch (const std::exception& e) { return fail(e, 1); }
}

uint32_t ref_model_num_params(void* m) {
    return static_cast<uint32_t>(static_cast<Model*>(m)->parameters().size());
}
// name_buf >= 64 bytes; dims[4]; returns data pointer (owned by the model)
float* ref_model_param(void* m, uint32_t i, char* name_buf, uint64_t* dims, uint32_t* ndim) {
    std::vector<Param> ps = static_cast<Model*>(m)->parameters();
    if (i >= ps.size()) return nullptr;
    std::snprintf(name_buf, 64, "%s", ps[i].name.c_str());
    *ndim = static_cast<uint32_t>(ps[i].value->ndim());
    for (uint32_t d = 0; d < *ndim && d < 4; ++d) dims[d] = ps[i].value->dim(d);
    return ps[i].value->data();
}

int ref_model_load_weights(void* m, const char* path, uint64_t* step, uint64_t* pos) {
    try {
        TrainState s = load_checkpoint_weights(path, *static_cast<Model*>(m));
        if (step) *step = s.step;
        if (pos) *pos = s.data_position;
        return 0;
    } catch (const std::exception& e) { return fail(e, 2); }
}

// logits: [B*T*V] fp32, written by the reference's Model::forward
int ref_model_forward(void* m, const uint32_t* ids, uint64_t B, uint64_t T, float* logits) {
    try {
        std::vector<uint32_t> v(ids, ids + B * T);
        Tensor out = static_cast<Model*>(m)->forward(v, B, T);
        std::memcpy(logits, out.data(), out.numel() * sizeof(float));
        return 0;
    } catch (const std::exception& e) { return fail(e, 3); }
}

// The reference's own token loop, unmodified.  out must hold n + max_new ids.
int ref_generate_tokens(void* m, const uint32_t* ids, uint64_t n, uint64_t max_new,
                        float temperature, float top_p, float penalty, uint64_t seed,
                        int64_t stop_token, int eos_merges, uint32_t* out, uint64_t* out_n) {
    try {
        Tokenizer tok;
        tok.setMerges(eos_merges);
        Inference inf(*static_cast<Model*>(m), tok);
        SamplingOptions opt;
        opt.temperature = temperature; opt.top_p = top_p; opt.repetition_penalty = penalty;
        opt.seed = seed; opt.stop_token = stop_token;
        std::ostringstream sink;                       // generateTokens prints its result
        std::streambuf* old = std::cout.rdbuf(sink.rdbuf());
        std::string text;
        try { text = inf.generateTokens(std::vector<uint32_t>(ids, ids + n), max_new, opt); }
        catch (...) { std::cout.rdbuf(old); throw; }
        std::cout.rdbuf(old);
        std::vector<Token> all = tok.encode(text);
        *out_n = all.size();
        for (size_t i = 0; i < all.size(); ++i) out[i] = all[i];
        return 0;
    } catch (const std::invalid_argument& e) { return fail(e, 4); }
      catch (const std::exception& e) { return fail(e, 5); }
}

// ---- single ops (CPU loops of the reference) ------------------------------------------
int ref_op_rmsnorm(const float* x, const float* w, uint64_t rows, uint64_t D, float eps, float* y) {
    try { Tensor r = ops::rmsnorm(wrap(x, {rows, D}), wrap(w, {D}), eps, DType::F32);
          std::memcpy(y, r.data(), rows * D * 4); return 0; }
    catch (const std::exception& e) { return fail(e, 6); }
}
int ref_op_matmul(const float* a, const float* b, uint64_t M, uint64_t K, uint64_t N, float* c) {
    try { Tensor r = ops::matmul(wrap(a, {M, K}), wrap(b, {K, N}));
          std::memcpy(c, r.data(), M * N * 4); return 0; }
    catch (const std::exception& e) { return fail(e, 6); }
}
int ref_op_matmul_bt(const float* a, const float* b, uint64_t M, uint64_t K, uint64_t N, float* c) {
    try { Tensor r = ops::matmul_bt(wrap(a, {M, K}), wrap(b, {N, K}));
          std::memcpy(c, r.data(), M * N * 4); return 0; }
    catch (const std::exception& e) { return fail(e, 6); }
}
int ref_op_rope(const float* x, uint64_t G, uint64_t T, uint64_t hd, float theta, float* y) {
    try { Tensor r = ops::rope(wrap(x, {G, T, hd}), theta);
          std::memcpy(y, r.data(), G * T * hd * 4); return 0; }
    catch (const std::exception& e) { return fail(e, 6); }
}
// q,k,v,out: [B,H,T,hd], causal
int ref_op_attention(const float* q, const float* k, const float* v,
                     uint64_t B, uint64_t H, uint64_t T, uint64_t hd, float* out) {
    try { ops::AttentionOutput r = ops::attention(wrap(q, {B, H, T, hd}), wrap(k, {B, H, T, hd}),
                                                  wrap(v, {B, H, T, hd}), true);
          std::memcpy(out, r.out.data(), B * H * T * hd * 4); return 0; }
    catch (const std::exception& e) { return fail(e, 6); }
}
int ref_op_silu_mul(const float* g, const float* u, uint64_t n, float* y) {
    try { Tensor r = ops::multiply(ops::silu(wrap(g, {n})), wrap(u, {n}));
          std::memcpy(y, r.data(), n * 4); return 0; }
    catch (const std::exception& e) { return fail(e, 6); }
}
// ops::cross_entropy on host logits; targets are ids stored as floats, negative = ignored position
int ref_op_cross_entropy(const float* logits, const float* targets, uint64_t n, uint64_t V, uint64_t num_valid, float* loss) {
    try { *loss = ops::cross_entropy(wrap(logits, {n, V}), wrap(targets, {n}), num_valid); return 0; }
    catch (const std::exception& e) { return fail(e, 6); }
}

}  // extern "C"
