/* CPU oracle for the small-llm token loop -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the reference's CPU algorithm for the generate/sample path.
 * It exists so that the CUDA engine can be checked on machines where the reference tree
 * is not present.  Nothing in the shipped library may include, link or call this file;
 * only tests, the smoke check and the benchmark's cpu_baseline leg do.
 *
 * Parity status: PINNED against the reference itself.  The reference ships no tests or
 * golden vectors for this path, so the pin is the reference's own CPU code compiled from
 * its sources (oracle/Makefile `ref` target): tests/test_oracle_vs_ref.py demands bit-equal
 * logits, weights, checkpoints and token streams whenever that library is present, and
 * tests/golden/ holds vectors produced by it (tests/golden/make_golden.py).
 *
 * Every function names the reference file:line it follows (paths inside the small-llm tree).
 */
#ifndef SLLM_ORACLE_H
#define SLLM_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    uint64_t vocab, context, layers, d_model, heads, ffn; /* include/config.h:15-26 */
    float theta, eps;                                      /* include/config.h:28,46 */
} orc_config;

typedef struct orc_model orc_model;

const char* orc_last_error(void);

orc_model* orc_model_create(const orc_config* cfg);
void orc_model_destroy(orc_model* m);

/* Parameter registry in the reference's order (src/model.cpp:106-131). */
uint32_t orc_num_params(const orc_model* m);
float* orc_param(orc_model* m, uint32_t i, char name[64], uint64_t dims[2], uint32_t* ndim);

/* Reseed a std::mt19937 restatement with `seed`; every matrix N(0,stddev) with a fresh
 * std::normal_distribution<float> per tensor (src/tensor.cpp:136-143), gains = 1. */
void orc_init_normal(orc_model* m, uint32_t seed, float stddev);

/* Checkpoint in the reference layout, weights only (src/checkpoint.cpp:25-55,57-102). */
int orc_save_checkpoint(orc_model* m, const char* path, uint64_t step, uint64_t data_pos);
int orc_load_checkpoint(orc_model* m, const char* path, uint64_t* step, uint64_t* data_pos);

/* Model::forward (src/model.cpp:31-62) for B independent rows of T tokens.
 * logits receives rows [row_from, T) of every sequence: [B, T-row_from, vocab]. */
int orc_forward(orc_model* m, const uint32_t* ids, uint64_t B, uint64_t T, uint64_t row_from,
                float* logits);

/* Incremental form of the same computation: a session keeps K/V of the positions already
 * seen, so feeding tokens one at a time gives the same bits as a full forward. */
typedef struct orc_session orc_session;
orc_session* orc_session_create(orc_model* m);
void orc_session_destroy(orc_session* s);
void orc_session_reset(orc_session* s);
uint64_t orc_session_len(const orc_session* s);
/* append n tokens; logits_last (may be NULL) receives the last position's logits [vocab];
 * logits_all (may be NULL) receives all n rows. */
int orc_session_feed(orc_session* s, const uint32_t* ids, uint64_t n, float* logits_last,
                     float* logits_all);

/* Sampler body (src/inference.cpp:101-154) with the std::discrete_distribution draw replaced
 * by the caller's uniform u in [0,1).  Returns the token, or -1 when every logit is
 * non-finite.  margin (may be NULL) receives how far u was from the nearest cumulative
 * boundary that would have changed the result (for exempting knife-edge draws). */
int64_t orc_sample(const float* logits, uint64_t vocab, const uint32_t* history, uint64_t n_hist,
                   float temperature, float top_p, float penalty, double u, double* margin);
/* Greedy rule the reference intends (src/inference.cpp:104-119): penalty, then first max.
 * top2_margin (may be NULL) receives best - second best after the penalty. */
int64_t orc_greedy(const float* logits, uint64_t vocab, const uint32_t* history, uint64_t n_hist,
                   float penalty, float* top2_margin);

/* Token loop (src/inference.cpp:21-173) on a session: window sliding, EOS / stop token
 * appended before stopping.  uniforms[step] feeds step `step`; temperature <= 0 selects the
 * greedy rule above.  out receives prompt + continuation. */
typedef struct {
    float temperature, top_p, repetition_penalty;
    int64_t stop_token;
    uint32_t eos_token;
} orc_sampling;
int orc_generate(orc_model* m, const uint32_t* prompt, uint64_t n_prompt, uint64_t max_new,
                 const orc_sampling* opt, const float* uniforms, uint32_t* out, uint64_t* out_n);

/* Same loop, drawing as the reference does: std::mt19937_64(seed) feeding
 * std::discrete_distribution, one canonical double per step that keeps >= 2 candidates
 * (src/inference.cpp:37,151-154).  Used to pin the restated sampler to the reference's loop. */
int orc_generate_seeded(orc_model* m, const uint32_t* prompt, uint64_t n_prompt, uint64_t max_new,
                        const orc_sampling* opt, uint64_t seed, uint32_t* out, uint64_t* out_n);

/* Deterministic inputs: ids = mt19937(seed)() & mask; uniforms = (mt19937(seed)() >> 8) * 2^-24. */
void orc_prompt_ids(uint32_t seed, uint64_t n, uint32_t mask, uint32_t* out);
void orc_uniforms(uint32_t seed, uint64_t n, float* out);
/* generate_canonical<double,53>(mt19937_64(seed)) stream: what discrete_distribution consumes. */
void orc_canonical64(uint64_t seed, uint64_t n, double* out);

/* ops::cross_entropy (src/ops/cross_entropy.cpp:14-54): mean over the counted positions of
 * -logit[target] + max + log(sum exp(logit - max)); target < 0 = ignored; num_valid 0 = all n positions. */
float orc_cross_entropy(const float* logits, const int32_t* targets, uint64_t n, uint64_t V, uint64_t num_valid);

#ifdef __cplusplus
}
#endif
#endif
