// sllm_serving.hpp -- host-side serving components over the C ABI, in C++ like the rest of the host layer:
//
//   ContinuousBatcher   keeps the sequence slots of one engine full: decodes in short bursts on the device, collects
//                       the slots that stopped (EOS, stop token, budget), parks them and assigns the next waiting
//                       prompt to the freed slot while the other slots keep their KV cache and sampler state.
//   ShardedInference    one engine per GPU, each driven by its own host thread: independent sequences are dealt to
//                       the GPUs (balanced by prompt length), weights are replicated, nothing is exchanged inside
//                       the token loop; the finished token streams come back to the caller in request order.
//
// Neither has a counterpart in the reference, which generates one sequence per call on one device
// (src/main.cpp:46-62); both keep its stop rules (src/inference.cpp:158-160: the stop token is appended, then the
// sequence ends) and produce, for every request, exactly the tokens a single Inference::generateTokenIds call
// would: a request's draws are indexed by its own step number.
#pragma once
#include <algorithm>
#include <exception>
#include <functional>
#include <memory>
#include <numeric>
#include <thread>

#include "small_llm.hpp"

struct BatchRequest {
    std::vector<uint32_t> prompt;
    size_t max_new_tokens = 0;
    std::vector<double> draws;          // [max_new_tokens] uniforms in [0,1) when sampling with supplied draws
    std::vector<uint32_t> tokens;       // result: prompt + continuation
    size_t made = 0;                    // tokens generated so far (scheduler state)
};

class ContinuousBatcher {
public:
    // The model's engine must have been given its slots (Model::set_engine_options, max_batch) before first use.
    ContinuousBatcher(Model& model, uint32_t eos_token, SamplingOptions opt = {}, size_t burst = 16)
        : model_(model), eos_(eos_token), opt_(opt), burst_(burst ? burst : 1) {}

    void run(std::vector<BatchRequest>& requests) {
        sllm_engine* e = model_.engine();
        const size_t n_slots = model_.engine_options().max_batch;
        std::vector<long> slot_req(n_slots, -1);
        size_t next = 0, active = 0;
        sllm_detail::check(sllm_reset(e), e);
        sllm_sampling s;
        s.temperature = opt_.temperature; s.top_p = opt_.top_p; s.repetition_penalty = opt_.repetition_penalty;
        s.eos_token = eos_; s.stop_token = opt_.stop_token; s.seed = opt_.seed;
        const bool sampled = opt_.temperature > 0.0f;
        auto fill = [&]() {
            for (size_t slot = 0; slot < n_slots && next < requests.size(); ++slot) {
                if (slot_req[slot] >= 0) continue;
                BatchRequest& r = requests[next];
                if (sampled && r.draws.size() < r.max_new_tokens)
                    throw std::invalid_argument("ContinuousBatcher: a sampled request needs max_new_tokens draws");
                sllm_detail::check(sllm_slot_assign(e, static_cast<uint32_t>(slot), r.prompt.data(), static_cast<uint32_t>(r.prompt.size())), e);
                r.made = 0;
                slot_req[slot] = static_cast<long>(next++);
                ++active;
            }
        };
        fill();
        std::vector<double> draws;
        std::vector<int32_t> flags(n_slots);
        std::vector<uint32_t> buf(2 * model_.config().context_length + 2);
        while (active > 0) {
            const size_t live = sllm_num_live(e);         // the engine reads draws as [steps][its live-slot range]
            const double* dp = nullptr;
            if (sampled) {
                draws.assign(burst_ * live, 0.0);
                for (size_t slot = 0; slot < live; ++slot) {
                    if (slot_req[slot] < 0) continue;
                    const BatchRequest& r = requests[slot_req[slot]];
                    for (size_t k = 0; k < burst_ && r.made + k < r.draws.size(); ++k) draws[k * live + slot] = r.draws[r.made + k];
                }
                dp = draws.data();
            }
            sllm_detail::check(sllm_decode_loop(e, burst_, &s, dp), e);
            sllm_detail::check(sllm_get_finished(e, flags.data(), static_cast<uint32_t>(live)), e);
            for (size_t slot = 0; slot < live; ++slot) {
                if (slot_req[slot] < 0) continue;
                BatchRequest& r = requests[slot_req[slot]];
                uint64_t n = 0;
                sllm_detail::check(sllm_get_tokens(e, static_cast<uint32_t>(slot), buf.data(), buf.size(), &n), e);
                r.made = n - r.prompt.size();
                if (r.made < r.max_new_tokens && flags[slot] == 0) continue;
                size_t keep = r.prompt.size() + std::min(r.made, r.max_new_tokens);
                for (size_t i = r.prompt.size(); i < keep; ++i)       // a stop token inside the budget ends the sequence there (it is kept)
                    if (buf[i] == eos_ || (opt_.stop_token >= 0 && buf[i] == static_cast<uint32_t>(opt_.stop_token))) { keep = i + 1; break; }
                r.tokens.assign(buf.begin(), buf.begin() + keep);
                sllm_detail::check(sllm_slot_release(e, static_cast<uint32_t>(slot)), e);
                slot_req[slot] = -1;
                --active;
            }
            fill();
        }
    }

private:
    Model& model_;
    uint32_t eos_;
    SamplingOptions opt_;
    size_t burst_;
};

// Sequences dealt to `world` shards so that every shard gets the same count (within one) and nearly the same total
// length: sorted by length, longest first, dealt in a snake (0..world-1, world-1..0, ...).  At large batch a decode
// iteration's time follows the KV bytes a GPU streams, i.e. the sum of its sequences' lengths, and the job ends with
// its slowest GPU.  Returns, per shard, the indices it owns in ascending order.
inline std::vector<std::vector<size_t>> balancedAssignment(const std::vector<size_t>& lengths, size_t world) {
    if (world == 0) throw std::invalid_argument("balancedAssignment: world must be at least 1");
    std::vector<size_t> order(lengths.size());
    std::iota(order.begin(), order.end(), size_t{0});
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return lengths[a] > lengths[b]; });
    std::vector<std::vector<size_t>> owners(world);
    for (size_t k = 0; k < order.size(); ++k) {
        const size_t round = k / world, col = k % world;
        owners[round % 2 == 0 ? col : world - 1 - col].push_back(order[k]);
    }
    for (auto& o : owners) std::sort(o.begin(), o.end());
    return owners;
}

class ShardedInference {
public:
    // devices: CUDA ordinals, one engine (and one host thread) each; an ordinal may appear more than once.
    // load: called once per engine, on that engine's thread, to put the weights in (load_checkpoint_weights, or
    // writes through Model::parameters()).
    ShardedInference(const ModelConfig& config, std::vector<int> devices, uint32_t max_batch_per_device, bool bf16,
                     std::function<void(Model&)> load)
        : config_(config), devices_(std::move(devices)), max_batch_(max_batch_per_device), bf16_(bf16), load_(std::move(load)) {
        if (devices_.empty()) throw std::invalid_argument("ShardedInference: no devices");
        models_.resize(devices_.size());
    }

    size_t shards() const { return devices_.size(); }

    // Every prompt's generation (prompt + continuation), in the order of `prompts`.  draws (optional): per prompt,
    // max_new_tokens uniforms, draw k feeding step k; empty = draw k of prompt g is the k-th
    // generate_canonical<double, 53> of std::mt19937_64(opt.seed + g), so a result does not depend on how the prompts
    // were dealt to the GPUs.
    std::vector<std::vector<uint32_t>> generateTokenIds(const std::vector<std::vector<uint32_t>>& prompts, size_t max_new_tokens,
                                                        uint32_t eos_token, SamplingOptions opt = {},
                                                        const std::vector<std::vector<double>>& draws = {}) {
        std::vector<size_t> lens(prompts.size());
        for (size_t i = 0; i < prompts.size(); ++i) lens[i] = prompts[i].size();
        const auto parts = balancedAssignment(lens, devices_.size());
        std::vector<std::vector<uint32_t>> out(prompts.size());
        std::vector<std::exception_ptr> errors(devices_.size());
        std::vector<std::thread> threads;
        for (size_t r = 0; r < devices_.size(); ++r)
            threads.emplace_back([&, r]() {
                try { run_shard(r, parts[r], prompts, max_new_tokens, eos_token, opt, draws, out); }
                catch (...) { errors[r] = std::current_exception(); }
            });
        for (auto& t : threads) t.join();
        for (auto& err : errors) if (err) std::rethrow_exception(err);
        return out;
    }

private:
    void run_shard(size_t r, const std::vector<size_t>& mine, const std::vector<std::vector<uint32_t>>& prompts, size_t max_new_tokens,
                   uint32_t eos_token, const SamplingOptions& opt, const std::vector<std::vector<double>>& draws,
                   std::vector<std::vector<uint32_t>>& out) {
        if (mine.empty()) return;
        if (!models_[r]) {                                     // first use: build this shard's engine and load it, on this thread
            models_[r] = std::make_unique<Model>(config_);
            sllm_engine_options o;
            sllm_default_engine_options(&o);
            o.max_batch = max_batch_; o.device = devices_[r];
            models_[r]->set_engine_options(o);
            models_[r]->to(Device::CUDA);
            models_[r]->enable_bf16(bf16_);
            load_(*models_[r]);
        }
        sllm_engine* e = models_[r]->engine();
        sllm_detail::check(sllm_engine_make_current(e), e);   // this thread is new: its current device is not yet the engine's
        sllm_sampling s;
        s.temperature = opt.temperature; s.top_p = opt.top_p; s.repetition_penalty = opt.repetition_penalty;
        s.eos_token = eos_token; s.stop_token = opt.stop_token; s.seed = opt.seed;
        const size_t stride = 2 * config_.context_length + 2;
        for (size_t b0 = 0; b0 < mine.size(); b0 += max_batch_) {       // more sequences than slots: groups of max_batch
            const size_t nb = std::min<size_t>(max_batch_, mine.size() - b0);
            std::vector<uint32_t> ids, lens(nb), toks(nb * stride);
            std::vector<uint64_t> out_lens(nb);
            for (size_t i = 0; i < nb; ++i) {
                const auto& p = prompts[mine[b0 + i]];
                ids.insert(ids.end(), p.begin(), p.end());
                lens[i] = static_cast<uint32_t>(p.size());
            }
            std::vector<double> d;                              // [step][slot]
            const bool sampled = opt.temperature > 0.0f;
            if (sampled) {
                d.assign(max_new_tokens * nb, 0.0);
                for (size_t i = 0; i < nb; ++i) {
                    const size_t g = mine[b0 + i];
                    if (!draws.empty()) {
                        if (draws[g].size() < max_new_tokens) throw std::invalid_argument("ShardedInference: a prompt needs max_new_tokens draws");
                        for (size_t k = 0; k < max_new_tokens; ++k) d[k * nb + i] = draws[g][k];
                    } else {                                    // this prompt's own generator, whichever shard runs it
                        std::mt19937_64 rng(opt.seed + g);
                        for (size_t k = 0; k < max_new_tokens; ++k) d[k * nb + i] = std::generate_canonical<double, 53>(rng);
                    }
                }
            }
            sllm_detail::check(sllm_generate(e, ids.data(), lens.data(), static_cast<uint32_t>(nb), max_new_tokens, &s,
                                             sampled ? d.data() : nullptr, toks.data(), stride, out_lens.data()), e);
            for (size_t i = 0; i < nb; ++i)                     // disjoint entries of `out`: no lock needed
                out[mine[b0 + i]].assign(toks.begin() + i * stride, toks.begin() + i * stride + out_lens[i]);
        }
    }

    ModelConfig config_;
    std::vector<int> devices_;
    uint32_t max_batch_;
    bool bf16_;
    std::function<void(Model&)> load_;
    std::vector<std::unique_ptr<Model>> models_;
};
