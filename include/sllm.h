/* sllm.h -- C ABI of the B200 token-loop engine (libsllm_b200.so).
 *
 * This is the drop-in boundary for small-llm's generate/sample path: plain pointers and
 * sizes, opaque handles, int status codes, no C++ or CUDA types.  Each entry point names the
 * small-llm interface it stands in for (paths inside the small-llm tree).  The C++ classes
 * with the reference's own names (ModelConfig, Model, Inference, SamplingOptions,
 * load_checkpoint_weights) are a header-only layer over these calls: include/small_llm.hpp.
 *
 * Threading: an engine belongs to one host thread and one GPU: calls on one engine must be
 * serialised by the caller (none of them locks).  Several engines (one per GPU, or several on one
 * GPU) may live in one process, each driven by its own thread.  There is no CPU fallback: every call
 * that computes needs a CUDA device of compute capability 10.x and fails with
 * SLLM_ERR_CUDA otherwise.
 */
#ifndef SLLM_H
#define SLLM_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* status codes; the C++ layer maps them back to the reference's exception types */
enum {
    SLLM_OK = 0,
    SLLM_ERR_INVALID = 1,    /* std::invalid_argument: shapes, empty prompt, bad config      */
    SLLM_ERR_IO = 2,         /* std::runtime_error: checkpoint cannot be opened / is corrupt  */
    SLLM_ERR_CUDA = 3,       /* std::runtime_error: a CUDA call failed, or no usable device   */
    SLLM_ERR_CAPACITY = 4,   /* std::runtime_error: batch slots or KV pages exhausted         */
    SLLM_ERR_DEVICE_WAIT = 5,/* a bounded device-side wait gave up (status word set)          */
    SLLM_ERR_NONFINITE = 6,  /* std::runtime_error: "all logits are non-finite"               */
    SLLM_ERR_STATE = 7       /* std::logic_error: call made in the wrong state                */
};

/* ModelConfig, include/config.h:6-47 (same fields, same defaults when zero-initialised by
 * sllm_default_model_config). */
typedef struct {
    uint64_t vocab_size, context_length, num_layers, d_model, num_heads, ffn_hidden;
    float rope_theta;
    float rms_eps;           /* ModelConfig::kRmsNormEps */
} sllm_model_config;

enum { SLLM_WEIGHTS_BF16 = 0, SLLM_WEIGHTS_F32 = 1 };

typedef struct {
    uint32_t max_batch;        /* sequences that can be live at once                          */
    uint32_t weight_dtype;     /* SLLM_WEIGHTS_BF16: bf16 weights and KV cache, fp32 residual
                                  stream and accumulation.  SLLM_WEIGHTS_F32: fp32 weights and
                                  KV cache (parity runs that need the reference's streams)    */
    uint64_t kv_pages;         /* pages of 64 positions in the pool; 0 = max_batch * ceil(ctx/64) */
    uint32_t max_chunk_tokens; /* tokens one prefill pass may carry; 0 = the engine chooses     */
                               /* (at most 8192; bf16: where the projections' tiles fill the SMs) */
    int32_t device;            /* CUDA device ordinal; -1 = current                           */
    uint32_t use_graph;        /* replay the decode step as a CUDA graph (1) or launch (0)    */
    uint32_t reserved;
} sllm_engine_options;

/* SamplingOptions, include/inference.h:9-15, plus the EOS id that the reference takes from
 * Tokenizer::getEosToken() (include/tokenizer.h:69). */
typedef struct {
    float temperature;         /* <= 0: greedy */
    float top_p;
    float repetition_penalty;  /* 1.0 = off */
    uint32_t eos_token;
    int64_t stop_token;        /* -1 = none */
    uint64_t seed;             /* used only when no draws are supplied */
} sllm_sampling;

typedef struct sllm_engine sllm_engine;

typedef struct {
    uint64_t weight_bytes, kv_bytes, scratch_bytes;   /* device memory held               */
    uint64_t kv_pages_total, kv_pages_free;
    uint64_t launches;           /* kernels launched by this engine since creation (graph nodes counted per replay) */
    uint64_t decode_steps;
    float last_step_ms;          /* device time of the most recent sllm_decode_step         */
    uint32_t reserved;
    uint64_t prefill_tokens;     /* positions run through prefill passes (prompts, appended turns) */
} sllm_stats;

void sllm_default_model_config(sllm_model_config* cfg);      /* include/config.h:15-46 defaults */
void sllm_default_engine_options(sllm_engine_options* opt);
void sllm_default_sampling(sllm_sampling* s);                /* include/inference.h:10-14, eos 32762 */

/* Error text of the last failing call on this engine (engine may be NULL for create errors). */
const char* sllm_last_error(const sllm_engine* e);

/* Model::Model + Model::to(CUDA) + Model::enable_bf16, src/model.cpp:15-29,133-149: allocates
 * every device buffer the engine will ever use (weights, KV page pool, scratch). Weights are
 * zero (gains 1) until set. */
int sllm_engine_create(const sllm_model_config* cfg, const sllm_engine_options* opt, sllm_engine** out);
void sllm_engine_destroy(sllm_engine* e);
int sllm_engine_stats(sllm_engine* e, sllm_stats* out);
/* Makes the engine's GPU the calling thread's current CUDA device.  Every call on an engine must come from a thread
 * whose current device is the engine's (sllm_engine_create leaves it so on the creating thread); a thread that takes
 * an engine over, or drives engines of several GPUs, calls this first. */
int sllm_engine_make_current(sllm_engine* e);
/* cudaStream_t of the engine (as void*), for callers that time with events. */
void* sllm_engine_stream(sllm_engine* e);

/* Model::parameters(), src/model.cpp:106-131: registry order and names. */
uint32_t sllm_num_params(const sllm_engine* e);
int sllm_param_info(const sllm_engine* e, uint32_t index, char name[64], uint64_t dims[2], uint32_t* ndim);
/* Assigning *p.value followed by Model::refresh_bf16_weights(), src/model.cpp:151-158:
 * host fp32 row-major data in the reference's shape; converted and re-laid-out on the device. */
int sllm_set_param(sllm_engine* e, const char* name, const float* host_data, const uint64_t* dims, uint32_t ndim);
/* load_checkpoint_weights, src/checkpoint.cpp:57-102: same file layout, same checks. */
int sllm_load_checkpoint(sllm_engine* e, const char* path, uint64_t* step, uint64_t* data_position);

/* Model::forward, src/model.cpp:31-62: B rows of T ids -> host logits [B,T,vocab] fp32.
 * Uses sequence slots 0..B-1 (their previous contents are dropped). */
int sllm_forward_logits(sllm_engine* e, const uint32_t* ids, uint64_t B, uint64_t T, float* host_logits);

/* ---- the token loop, step by step (src/inference.cpp:39-160) ------------------------- */
/* Drop every sequence and return all KV pages to the pool. */
int sllm_reset(sllm_engine* e);
/* Load prompts into slots 0..n_seq-1 (ids concatenated, lens[i] each >= 1), run them through
 * the model, leave each slot's last-position logits in the step-logits buffer. */
int sllm_prefill(sllm_engine* e, const uint32_t* ids, const uint32_t* lens, uint32_t n_seq);
/* Sampler body, src/inference.cpp:101-160, for every live slot on the device: penalty over the
 * slot's whole history, temperature softmax, top-p, draw, append, stop on EOS / stop token.
 * draws: n_seq doubles in [0,1) in HOST memory, one per slot (NULL allowed when greedy). */
int sllm_sample(sllm_engine* e, const sllm_sampling* opt, const double* draws);
/* Model::forward for the one new token of every live slot (KV-cached): appends K/V, leaves
 * new step logits. */
int sllm_decode_step(sllm_engine* e);
/* Copy a slot's step logits [vocab] to the host (what the reference reads at
 * src/inference.cpp:57,73). */
int sllm_get_step_logits(sllm_engine* e, uint32_t slot, float* host_logits);
/* Replace a slot's step logits with caller-supplied ones (HOST memory, [vocab]); the next
 * sllm_sample then works on them, as the reference's host sampler works on any logits row. */
int sllm_set_step_logits(sllm_engine* e, uint32_t slot, const float* host_logits);
/* Tokens of a slot so far (prompt + continuation); returns the count in *n. */
int sllm_get_tokens(sllm_engine* e, uint32_t slot, uint32_t* host_out, uint64_t capacity, uint64_t* n);
/* Overwrite the token that the next sllm_decode_step will feed to a slot (teacher forcing). */
int sllm_force_token(sllm_engine* e, uint32_t slot, uint32_t token);
/* Rewind a slot to its first n tokens (n >= 1, n <= current length): later positions are
 * forgotten, step logits become stale until the next decode step. */
int sllm_truncate(sllm_engine* e, uint32_t slot, uint64_t n_tokens);

/* ---- the token loop in one call: Inference::generateTokens, src/inference.cpp:21-173 --- */
/* All buffers are HOST memory.  prompts concatenated; out_tokens is [n_seq][out_stride] and
 * receives prompt + continuation per slot, out_lens the counts.
 * draws: [max_new][n_seq] doubles, draw[step][slot] feeds step `step` of that slot (indexed by
 * step, not consumed sequentially); NULL = seeded mode, reproducing the reference's
 * std::mt19937_64(seed) + std::discrete_distribution consumption (a draw is used only when at
 * least two candidates are kept) with slot s using seed + s.
 * A slot stops after EOS or stop_token is appended or after max_new tokens.  When a slot holds more
 * than context_length tokens the window slides as in the reference (src/inference.cpp:40-48): each
 * further token re-runs the last context_length tokens with positions restarting at 0.  Prompts may be
 * longer than context_length for the same reason; a slot can hold 2 * context_length + 2 tokens, and a call
 * whose prompt length + max_new_tokens exceeds that is refused with SLLM_ERR_CAPACITY. */
int sllm_generate(sllm_engine* e, const uint32_t* prompt_ids, const uint32_t* prompt_lens, uint32_t n_seq,
                  uint64_t max_new_tokens, const sllm_sampling* opt, const double* draws,
                  uint32_t* out_tokens, uint64_t out_stride, uint64_t* out_lens);

/* The decode loop only, for slots already prefilled or assigned: runs n_steps x (sample, decode step)
 * without host round trips and returns after the stream is idle.  draws (HOST memory, NULL when greedy):
 * [n_steps][sllm_num_live(e)] doubles, draw[step][slot] feeds step `step` of that slot; the column count
 * is the engine's live-slot range, parked slots included (their column is ignored).  At most
 * 2 * context_length + 2 steps per call (the engine's draw buffer is sized once, at creation). */
int sllm_decode_loop(sllm_engine* e, uint64_t n_steps, const sllm_sampling* opt, const double* draws);
/* The same loop with one CUDA event between consecutive iterations: step_ms[i] (HOST memory, [n_steps]) receives
 * the device time of iteration i in milliseconds -- the per-token latency samples a p50 / p95 is taken from.
 * Each iteration is replayed as its own graph here (the untimed loop replays eight per graph), which adds a few
 * microseconds per iteration.  At most 65536 steps per call. */
int sllm_decode_loop_timed(sllm_engine* e, uint64_t n_steps, const sllm_sampling* opt, const double* draws, float* step_ms);
/* Slots 0..sllm_num_live(e)-1 form the live range: the highest slot that holds a sequence, plus one. */
uint32_t sllm_num_live(const sllm_engine* e);

/* ops::cross_entropy(Model::forward(ids), targets, num_valid), src/ops/cross_entropy.cpp:14-54, without moving
 * the logits off the device: the mean over the counted positions of -logit[target] + log-sum-exp, per-row terms in
 * fp32, summed in double in row order.  targets[i] < 0 = position ignored (the reference's SFT mask); num_valid 0 =
 * divide by B*T.  What a perplexity check of a trained checkpoint needs (exp(loss)).  Uses slots 0..B-1. */
int sllm_eval_loss(sllm_engine* e, const uint32_t* ids, const int32_t* targets, uint64_t B, uint64_t T, uint64_t num_valid,
                   float* loss);

/* ---- single slots: continuous batching ------------------------------------------------------
 * No counterpart in the reference (it generates one sequence at a time); these keep a batched decode
 * loop full: when a slot stops (EOS, stop token, budget), the caller collects its tokens, releases it
 * and assigns the next prompt to it while the other slots keep their state. */
/* Put a prompt (1..context_length ids) into one slot and run it through the model; other slots are untouched.
 * Slots below `slot` that were never assigned are parked (idle). */
int sllm_slot_assign(sllm_engine* e, uint32_t slot, const uint32_t* ids, uint32_t len);
/* Append ids behind a live slot's tokens (a further turn of a conversation) and run only them through the model:
 * the positions before them are served from the slot's KV pages.  The slot's stop state is cleared and its step
 * logits are those of the last appended id.  No counterpart in the reference, whose chat loop re-encodes and
 * re-runs each turn from position 0 (src/main.cpp:46-62); the history handling this serves is that of the
 * browser demo (docs/script.js:288-305).  SLLM_ERR_CAPACITY when history + ids exceed context_length. */
int sllm_slot_append(sllm_engine* e, uint32_t slot, const uint32_t* ids, uint32_t len);
/* Park a slot: its KV pages return to the pool, the sampler skips it. */
int sllm_slot_release(sllm_engine* e, uint32_t slot);
/* Finished flags of slots 0..n-1 to HOST memory: 0 live, 1 EOS / stop token / parked, 2 context full, 3 non-finite logits. */
int sllm_get_finished(sllm_engine* e, int32_t* flags, uint32_t n);

/* ---- single kernels, device pointers in and out --------------------------------------- */
/* The flash-decode attention kernel on its own (the fused form of ops::attention for one cached
 * query position per token, src/ops/attention.cpp:143-184): d_q [n_tok][d_model] fp32 rotated
 * queries, d_tok_slot / d_tok_pos [n_tok] int32 (slot and position of each query; keys
 * 0..position of that slot's KV cache are attended), d_out [n_tok][d_model] fp32.  All four are
 * DEVICE pointers.  n_splits (1..32) blocks share each (token, head); with more than one, partial
 * results go through scratch memory that the engine allocated at creation.  More than 64 tokens need
 * n_splits = 1 and take the page-streaming kernel that the engine uses at large batch (same arithmetic, K/V pages
 * staged through shared memory).  The launch is asynchronous on `stream` (a cudaStream_t as void*; NULL = the
 * engine's stream). */
int sllm_k_attn_decode(sllm_engine* e, uint32_t layer, uint32_t n_tok, const float* d_q, const int32_t* d_tok_slot,
                       const int32_t* d_tok_pos, uint32_t n_splits, float* d_out, void* stream);

/* No counterpart in the reference.  Same kernel, same arguments and same results as
 * sllm_k_attn_decode, for callers that must not allocate device memory or cannot rely on memory
 * obtained from cudaMalloc: a serving process that has handed the whole device to its own pool
 * allocator (so a later cudaMalloc may fail), or a latency-critical decode thread that cannot
 * afford the device-wide synchronisation cudaMalloc / cudaFree may imply.  The split-K scratch
 * lives in a fixed array inside the library's device image (about 1.1 MB, resident on every GPU
 * that loads the library until the process exits) instead of in allocated memory, and the call
 * performs no cudaMalloc, cudaFree or other allocating routine.
 * Limits: n_tok * num_heads <= 64, n_splits <= 32, head_dim <= 128; larger requests are refused
 * with SLLM_ERR_CAPACITY.  The engine's device must be the current device.
 * The first call on a device looks up the array's device address (once per device); make that
 * first call outside any stream capture.  All calls share the one array: it keeps the previous
 * call's contents (the entry point clears the part that must start at zero), and two calls whose
 * kernels overlap on the GPU -- different streams, or different engines on one GPU -- race. */
int sllm_k_attn_decode_static(sllm_engine* e, uint32_t layer, uint32_t n_tok, const float* d_q,
                              const int32_t* d_tok_slot, const int32_t* d_tok_pos, uint32_t n_splits, float* d_out,
                              void* stream);

/* ---- the KV cache of one slot, from and to the host --------------------------------------------
 * No counterpart in the reference (it keeps no KV cache; these rows are what its Attention::forward holds in k and
 * v after split_heads and rope, src/nn/attention.cpp:68-77, for the slot's positions).  Rows are HOST memory,
 * [n_pos][num_heads * head_dim] fp32 with head h in columns h * head_dim .., positions pos0 .. pos0 + n_pos - 1 of
 * `layer`; the positions must lie inside the pages the slot already holds (it was prefilled or assigned at least
 * that far).  Writing converts to the cache's element type (bf16 or fp32); reading converts back.  Uses: moving a
 * prefix between engines, and checking the attention kernels against ops::attention on the same K and V. */
int sllm_kv_write(sllm_engine* e, uint32_t layer, uint32_t slot, uint32_t pos0, uint32_t n_pos, const float* k_rows, const float* v_rows);
int sllm_kv_read(sllm_engine* e, uint32_t layer, uint32_t slot, uint32_t pos0, uint32_t n_pos, float* k_rows, float* v_rows);

/* ---- diagnostics ------------------------------------------------------------------------------ */
/* No counterpart in the reference.  Every device-side wait of this library (mbarrier waits of the TMA / tcgen05
 * pipelines) polls for a bounded time, then raises the engine's status word and lets its kernel return; the host
 * reports SLLM_ERR_DEVICE_WAIT at its next synchronisation and the engine stays usable.  This entry point
 * exercises exactly that path: it launches one thread that waits, for limit_us microseconds at most
 * (1..100000), on a barrier that nothing arrives at, and returns what the host then sees --
 * SLLM_ERR_DEVICE_WAIT.  Nothing faults, traps or spins without bound. */
int sllm_k_wait_probe(sllm_engine* e, uint32_t limit_us);

#ifdef __cplusplus
}
#endif
#endif /* SLLM_H */
