/* CPU oracle for the small-llm token loop -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * See sllm_oracle.h for the rules on who may use it and how its parity is pinned.
 *
 * The arithmetic below keeps, for every output element, the reference's exact sequence of
 * fp32 operations (sequential sums, no fused multiply-add: build with -ffp-contract=off).
 * Work is only re-ordered ACROSS independent output elements (threads, SIMD lanes), which
 * cannot change any bit.
 */
#include "sllm_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static _Thread_local char g_err[256];
const char* orc_last_error(void) { return g_err; }
static int fail(int code, const char* msg) { snprintf(g_err, sizeof g_err, "%s", msg); return code; }

/* ------------------------------------------------------------------ generators ------- */
/* std::mt19937 (32-bit Mersenne twister, standard parameters). */
typedef struct { uint32_t s[624]; int i; } mt32;
static void mt32_seed(mt32* g, uint32_t seed) {
    g->s[0] = seed;
    for (int i = 1; i < 624; ++i) g->s[i] = 1812433253u * (g->s[i - 1] ^ (g->s[i - 1] >> 30)) + (uint32_t)i;
    g->i = 624;
}
static uint32_t mt32_next(mt32* g) {
    if (g->i >= 624) {
        for (int k = 0; k < 624; ++k) {
            uint32_t y = (g->s[k] & 0x80000000u) | (g->s[(k + 1) % 624] & 0x7fffffffu);
            g->s[k] = g->s[(k + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
        }
        g->i = 0;
    }
    uint32_t y = g->s[g->i++];
    y ^= y >> 11; y ^= (y << 7) & 0x9d2c5680u; y ^= (y << 15) & 0xefc60000u; y ^= y >> 18;
    return y;
}
/* std::mt19937_64 */
typedef struct { uint64_t s[312]; int i; } mt64;
static void mt64_seed(mt64* g, uint64_t seed) {
    g->s[0] = seed;
    for (int i = 1; i < 312; ++i)
        g->s[i] = 6364136223846793005ull * (g->s[i - 1] ^ (g->s[i - 1] >> 62)) + (uint64_t)i;
    g->i = 312;
}
static uint64_t mt64_next(mt64* g) {
    if (g->i >= 312) {
        for (int k = 0; k < 312; ++k) {
            uint64_t y = (g->s[k] & 0xffffffff80000000ull) | (g->s[(k + 1) % 312] & 0x7fffffffull);
            g->s[k] = g->s[(k + 156) % 312] ^ (y >> 1) ^ ((y & 1ull) ? 0xb5026f5aa96619e9ull : 0ull);
        }
        g->i = 0;
    }
    uint64_t y = g->s[g->i++];
    y ^= (y >> 29) & 0x5555555555555555ull; y ^= (y << 17) & 0x71d67fffeda60000ull;
    y ^= (y << 37) & 0xfff7eee000000000ull; y ^= y >> 43;
    return y;
}

void orc_prompt_ids(uint32_t seed, uint64_t n, uint32_t mask, uint32_t* out) {
    mt32 g; mt32_seed(&g, seed);
    for (uint64_t i = 0; i < n; ++i) out[i] = mt32_next(&g) & mask;
}
void orc_uniforms(uint32_t seed, uint64_t n, float* out) {
    mt32 g; mt32_seed(&g, seed);
    for (uint64_t i = 0; i < n; ++i) out[i] = (float)(mt32_next(&g) >> 8) * (1.0f / 16777216.0f);
}
void orc_canonical64(uint64_t seed, uint64_t n, double* out) {
    /* libstdc++ generate_canonical<double,53> over a 64-bit engine: one draw / 2^64 */
    mt64 g; mt64_seed(&g, seed);
    for (uint64_t i = 0; i < n; ++i) {
        double r = (double)mt64_next(&g) / 18446744073709551616.0;
        if (r >= 1.0) r = nextafter(1.0, 0.0);
        out[i] = r;
    }
}

/* libstdc++ std::normal_distribution<float> over std::mt19937 (Marsaglia polar method,
 * generate_canonical<float,24> = one 32-bit draw / 2^32), state reset per tensor as in
 * src/tensor.cpp:139-143. */
static float canon_f32(mt32* g) {
    float r = (float)mt32_next(g) / 4294967296.0f;
    if (r >= 1.0f) r = nextafterf(1.0f, 0.0f);
    return r;
}
static void fill_normal(mt32* g, float* p, uint64_t n, float mean, float stddev) {
    int have = 0; float saved = 0.0f;
    for (uint64_t i = 0; i < n; ++i) {
        float ret;
        if (have) { have = 0; ret = saved; }
        else {
            float x, y, r2;
            do {
                x = 2.0f * canon_f32(g) - 1.0f;
                y = 2.0f * canon_f32(g) - 1.0f;
                r2 = x * x + y * y;
            } while (r2 > 1.0f || r2 == 0.0f);
            float mult = sqrtf(-2.0f * logf(r2) / r2);
            saved = x * mult; have = 1;
            ret = y * mult;
        }
        p[i] = ret * stddev + mean;
    }
}

/* ------------------------------------------------------------------ model ------------ */
typedef struct { char name[64]; uint32_t ndim; uint64_t dims[2]; float* data; int decay; } orc_par;

struct orc_model {
    orc_config c;
    uint32_t np;
    orc_par* p;
    float* embT;         /* [D][V] copy of the embedding for the tied head (same k order) */
};

static uint64_t par_numel(const orc_par* p) { return p->ndim == 2 ? p->dims[0] * p->dims[1] : p->dims[0]; }

static void add_par(orc_model* m, const char* name, uint64_t d0, uint64_t d1, int decay) {
    orc_par* q = &m->p[m->np++];
    snprintf(q->name, sizeof q->name, "%s", name);
    q->ndim = d1 ? 2 : 1; q->dims[0] = d0; q->dims[1] = d1; q->decay = decay;
    q->data = (float*)calloc(par_numel(q), sizeof(float));
    if (!decay) for (uint64_t i = 0; i < d0; ++i) q->data[i] = 1.0f;
}

/* registry order: src/model.cpp:106-131 */
orc_model* orc_model_create(const orc_config* cfg) {
    if (!cfg || !cfg->heads || cfg->d_model % cfg->heads || ((cfg->d_model / cfg->heads) & 1)) {
        fail(1, "orc_model_create: bad config"); return NULL;
    }
    orc_model* m = (orc_model*)calloc(1, sizeof *m);
    m->c = *cfg;
    m->p = (orc_par*)calloc(2 + 9 * cfg->layers, sizeof(orc_par));
    const uint64_t D = cfg->d_model, F = cfg->ffn;
    add_par(m, "embedding", cfg->vocab, D, 1);
    for (uint64_t l = 0; l < cfg->layers; ++l) {
        char n[64];
#define NM(suffix) (snprintf(n, sizeof n, "blocks.%llu." suffix, (unsigned long long)l), n)
        add_par(m, NM("attn_norm"), D, 0, 0);
        add_par(m, NM("attn.q"), D, D, 1);
        add_par(m, NM("attn.k"), D, D, 1);
        add_par(m, NM("attn.v"), D, D, 1);
        add_par(m, NM("attn.out"), D, D, 1);
        add_par(m, NM("ffn_norm"), D, 0, 0);
        add_par(m, NM("ffn.gate"), D, F, 1);
        add_par(m, NM("ffn.up"), D, F, 1);
        add_par(m, NM("ffn.down"), F, D, 1);
#undef NM
    }
    add_par(m, "final_norm", D, 0, 0);
    return m;
}
void orc_model_destroy(orc_model* m) {
    if (!m) return;
    for (uint32_t i = 0; i < m->np; ++i) free(m->p[i].data);
    free(m->p); free(m->embT); free(m);
}
uint32_t orc_num_params(const orc_model* m) { return m->np; }
float* orc_param(orc_model* m, uint32_t i, char name[64], uint64_t dims[2], uint32_t* ndim) {
    if (i >= m->np) return NULL;
    if (name) memcpy(name, m->p[i].name, 64);
    if (dims) { dims[0] = m->p[i].dims[0]; dims[1] = m->p[i].dims[1]; }
    if (ndim) *ndim = m->p[i].ndim;
    return m->p[i].data;
}
void orc_init_normal(orc_model* m, uint32_t seed, float stddev) {
    mt32 g; mt32_seed(&g, seed);
    for (uint32_t i = 0; i < m->np; ++i) {
        orc_par* q = &m->p[i];
        if (q->decay) fill_normal(&g, q->data, par_numel(q), 0.0f, stddev);
        else for (uint64_t k = 0; k < q->dims[0]; ++k) q->data[k] = 1.0f;
    }
}

/* src/checkpoint.cpp:25-55 (writer, without the optimizer tail) */
int orc_save_checkpoint(orc_model* m, const char* path, uint64_t step, uint64_t data_pos) {
    FILE* f = fopen(path, "wb");
    if (!f) return fail(2, "orc_save_checkpoint: cannot open");
    fwrite(&step, 8, 1, f); fwrite(&data_pos, 8, 1, f);
    uint32_t np = m->np; fwrite(&np, 4, 1, f);
    for (uint32_t i = 0; i < m->np; ++i) {
        orc_par* q = &m->p[i];
        uint32_t nl = (uint32_t)strlen(q->name);
        fwrite(&nl, 4, 1, f); fwrite(q->name, 1, nl, f);
        fwrite(&q->ndim, 4, 1, f);
        for (uint32_t d = 0; d < q->ndim; ++d) fwrite(&q->dims[d], 8, 1, f);
        fwrite(q->data, sizeof(float), par_numel(q), f);
    }
    int bad = ferror(f);
    fclose(f);
    return bad ? fail(2, "orc_save_checkpoint: write failed") : 0;
}
/* src/checkpoint.cpp:57-102 */
int orc_load_checkpoint(orc_model* m, const char* path, uint64_t* step, uint64_t* data_pos) {
    FILE* f = fopen(path, "rb");
    if (!f) return fail(2, "load_checkpoint: cannot open");
    uint64_t st = 0, dp = 0; uint32_t np = 0;
    int ok = fread(&st, 8, 1, f) == 1 && fread(&dp, 8, 1, f) == 1 && fread(&np, 4, 1, f) == 1;
    if (ok && np != m->np) { fclose(f); return fail(3, "load_checkpoint: parameter count differs"); }
    for (uint32_t i = 0; ok && i < m->np; ++i) {
        orc_par* q = &m->p[i];
        uint32_t nl = 0, nd = 0; char nm[256] = {0};
        ok = fread(&nl, 4, 1, f) == 1 && nl < sizeof nm && fread(nm, 1, nl, f) == nl;
        if (!ok) break;
        if (strcmp(nm, q->name)) { fclose(f); return fail(4, "load_checkpoint: expected parameter name differs"); }
        ok = fread(&nd, 4, 1, f) == 1;
        if (!ok) break;
        uint64_t dims[4] = {0, 0, 0, 0};
        for (uint32_t d = 0; ok && d < nd && d < 4; ++d) ok = fread(&dims[d], 8, 1, f) == 1;
        if (!ok) break;
        if (nd != q->ndim || dims[0] != q->dims[0] || (nd == 2 && dims[1] != q->dims[1])) {
            fclose(f); return fail(5, "load_checkpoint: shape mismatch");
        }
        ok = fread(q->data, sizeof(float), par_numel(q), f) == par_numel(q);
    }
    fclose(f);
    if (!ok) return fail(6, "load_checkpoint: file truncated or corrupt");
    if (step) *step = st;
    if (data_pos) *data_pos = dp;
    return 0;
}

/* ------------------------------------------------------------------ ops -------------- */
/* ops::matmul CPU loop, src/ops/matmul.cpp:66-75: c[i,j] = sum_k a[i,k]*b[k,j], k ascending,
 * one fp32 multiply and one fp32 add per term.  Four rows and a strip of columns share the
 * loads of b; each c[i,j] still sees exactly that sequence. */
#define JB 64
static void mm(const float* a, const float* b, float* c, uint64_t M, uint64_t K, uint64_t N) {
    const uint64_t nrb = (M + 3) / 4, ncb = (N + JB - 1) / JB;
#pragma omp parallel for collapse(2) schedule(static)
    for (uint64_t rb = 0; rb < nrb; ++rb)
        for (uint64_t cb = 0; cb < ncb; ++cb) {
            const uint64_t i0 = rb * 4, j0 = cb * JB;
            const uint64_t nr = M - i0 < 4 ? M - i0 : 4, nc = N - j0 < JB ? N - j0 : JB;
            float acc[4][JB];
            for (uint64_t r = 0; r < 4; ++r) for (uint64_t j = 0; j < JB; ++j) acc[r][j] = 0.0f;
            if (nr == 4 && nc == JB) {
                for (uint64_t k = 0; k < K; ++k) {
                    const float* br = b + k * N + j0;
                    const float a0 = a[(i0 + 0) * K + k], a1 = a[(i0 + 1) * K + k];
                    const float a2 = a[(i0 + 2) * K + k], a3 = a[(i0 + 3) * K + k];
                    for (uint64_t j = 0; j < JB; ++j) {
                        acc[0][j] += a0 * br[j]; acc[1][j] += a1 * br[j];
                        acc[2][j] += a2 * br[j]; acc[3][j] += a3 * br[j];
                    }
                }
            } else {
                for (uint64_t k = 0; k < K; ++k) {
                    const float* br = b + k * N + j0;
                    for (uint64_t r = 0; r < nr; ++r) {
                        const float av = a[(i0 + r) * K + k];
                        for (uint64_t j = 0; j < nc; ++j) acc[r][j] += av * br[j];
                    }
                }
            }
            for (uint64_t r = 0; r < nr; ++r)
                memcpy(c + (i0 + r) * N + j0, acc[r], nc * sizeof(float));
        }
}

/* ops::rmsnorm CPU loop, src/ops/rmsnorm.cpp:38-60 */
static void rmsnorm(const float* x, const float* w, float* y, uint64_t rows, uint64_t D, float eps) {
#pragma omp parallel for schedule(static)
    for (uint64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * D; float* yr = y + r * D;
        float ms = 0.0f;
        for (uint64_t i = 0; i < D; ++i) { float v = xr[i]; ms += v * v; }
        ms /= (float)D;
        const float inv = 1.0f / sqrtf(ms + eps);
        for (uint64_t i = 0; i < D; ++i) yr[i] = xr[i] * inv * w[i];
    }
}

/* ------------------------------------------------------------------ session ---------- */
struct orc_session {
    orc_model* m;
    uint64_t len;        /* positions already cached */
    float* k;            /* [L][H][ctx][hd] after RoPE */
    float* v;            /* [L][H][ctx][hd] */
    float* cs;           /* rope cos [ctx][hd/2] */
    float* sn;           /* rope sin */
};

static void build_embT(orc_model* m) {
    const uint64_t V = m->c.vocab, D = m->c.d_model;
    if (!m->embT) m->embT = (float*)malloc(V * D * sizeof(float));
    const float* e = m->p[0].data;
#pragma omp parallel for schedule(static)
    for (uint64_t v = 0; v < V; ++v)
        for (uint64_t d = 0; d < D; ++d) m->embT[d * V + v] = e[v * D + d];
}

orc_session* orc_session_create(orc_model* m) {
    orc_session* s = (orc_session*)calloc(1, sizeof *s);
    const orc_config* c = &m->c;
    const uint64_t hd = c->d_model / c->heads, pairs = hd / 2;
    s->m = m;
    s->k = (float*)malloc(c->layers * c->d_model * c->context * sizeof(float));
    s->v = (float*)malloc(c->layers * c->d_model * c->context * sizeof(float));
    s->cs = (float*)malloc(c->context * pairs * sizeof(float));
    s->sn = (float*)malloc(c->context * pairs * sizeof(float));
    /* src/ops/rope.cpp:48-56 */
    for (uint64_t pos = 0; pos < c->context; ++pos)
        for (uint64_t i = 0; i < pairs; ++i) {
            const float freq = 1.0f / powf(c->theta, (float)(2 * i) / (float)hd);
            const float angle = (float)pos * freq;
            s->cs[pos * pairs + i] = cosf(angle);
            s->sn[pos * pairs + i] = 1.0f * sinf(angle);
        }
    build_embT(m);   /* weights may have been rewritten since the last session */
    return s;
}
void orc_session_destroy(orc_session* s) {
    if (!s) return;
    free(s->k); free(s->v); free(s->cs); free(s->sn); free(s);
}
void orc_session_reset(orc_session* s) { s->len = 0; }
uint64_t orc_session_len(const orc_session* s) { return s->len; }

/* One TransformerBlock::forward (src/nn/transformer_ block.cpp:19-31) over n new positions. */
static void block_forward(orc_session* s, uint64_t layer, float* x, uint64_t n, float* ws) {
    orc_model* m = s->m; const orc_config* c = &m->c;
    const uint64_t D = c->d_model, H = c->heads, hd = D / H, F = c->ffn, ctx = c->context;
    const uint64_t pairs = hd / 2, t0 = s->len;
    const orc_par* P = &m->p[1 + 9 * layer];
    float* xn = ws;            /* [n,D] */
    float* q = xn + n * D;     /* [n,D] */
    float* kk = q + n * D;     /* [n,D] */
    float* vv = kk + n * D;    /* [n,D] */
    float* att = vv + n * D;   /* [n,D] merged heads */
    float* o = att + n * D;    /* [n,D] */
    float* g = o + n * D;      /* [n,F] */
    float* u = g + n * F;      /* [n,F] */
    float* sc = u + n * F;     /* per-thread score rows, allocated by caller: [n][ctx] */

    rmsnorm(x, P[0].data, xn, n, D, c->eps);
    /* Attention::forward, src/nn/attention.cpp:61-90 */
    mm(xn, P[1].data, q, n, D, D);
    mm(xn, P[2].data, kk, n, D, D);
    mm(xn, P[3].data, vv, n, D, D);
    float* Kc = s->k + layer * D * ctx;
    float* Vc = s->v + layer * D * ctx;
    /* split_heads + rope (src/ops/rope.cpp:60-76): interleaved pairs */
#pragma omp parallel for collapse(2) schedule(static)
    for (uint64_t i = 0; i < n; ++i)
        for (uint64_t h = 0; h < H; ++h) {
            const uint64_t pos = t0 + i;
            float* qh = q + i * D + h * hd;
            const float* kh = kk + i * D + h * hd;
            float* kd = Kc + (h * ctx + pos) * hd;
            float* vd = Vc + (h * ctx + pos) * hd;
            for (uint64_t p = 0; p < pairs; ++p) {
                const float cc = s->cs[pos * pairs + p], ss = s->sn[pos * pairs + p];
                const float q1 = qh[2 * p], q2 = qh[2 * p + 1];
                qh[2 * p] = q1 * cc - q2 * ss; qh[2 * p + 1] = q1 * ss + q2 * cc;
                const float k1 = kh[2 * p], k2 = kh[2 * p + 1];
                kd[2 * p] = k1 * cc - k2 * ss; kd[2 * p + 1] = k1 * ss + k2 * cc;
            }
            memcpy(vd, vv + i * D + h * hd, hd * sizeof(float));
        }
    /* ops::attention CPU path, src/ops/attention.cpp:45-50,179-183; causal softmax
     * src/ops/softmax.cpp:24-40.  Masked probabilities are exactly 0 there, so the sum over
     * all keys equals the sum over keys <= query. */
    const float scale = 1.0f / sqrtf((float)hd);
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (uint64_t i = 0; i < n; ++i)
        for (uint64_t h = 0; h < H; ++h) {
            const uint64_t valid = t0 + i + 1;
            const float* qh = q + i * D + h * hd;
            const float* Kh = Kc + h * ctx * hd;
            const float* Vh = Vc + h * ctx * hd;
            float* row = sc + (i * H + h) * ctx;
            for (uint64_t j = 0; j < valid; ++j) {
                float sum = 0.0f;
                for (uint64_t d = 0; d < hd; ++d) sum += qh[d] * Kh[j * hd + d];
                row[j] = sum * scale;
            }
            float mx = row[0];
            for (uint64_t j = 1; j < valid; ++j) mx = row[j] > mx ? row[j] : mx;
            float sum = 0.0f;
            for (uint64_t j = 0; j < valid; ++j) { row[j] = expf(row[j] - mx); sum += row[j]; }
            for (uint64_t j = 0; j < valid; ++j) row[j] /= sum;
            float* out = att + i * D + h * hd;
            for (uint64_t d = 0; d < hd; ++d) out[d] = 0.0f;
            for (uint64_t j = 0; j < valid; ++j) {
                const float p = row[j];
                for (uint64_t d = 0; d < hd; ++d) out[d] += p * Vh[j * hd + d];
            }
        }
    mm(att, P[4].data, o, n, D, D);
    for (uint64_t i = 0; i < n * D; ++i) x[i] = x[i] + o[i];            /* residual, elementwise.cpp:19-55 */
    /* SwiGLU::forward, src/nn/swiglu.cpp:37-57; silu src/ops/elementwise.cpp:106-132 */
    rmsnorm(x, P[5].data, xn, n, D, c->eps);
    mm(xn, P[6].data, g, n, D, F);
    mm(xn, P[7].data, u, n, D, F);
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n * F; ++i) {
        const float val = g[i];
        const float sig = 1.0f / (1.0f + expf(-val));
        const float act = val * sig;
        g[i] = act * u[i];
    }
    mm(g, P[8].data, o, n, F, D);
    for (uint64_t i = 0; i < n * D; ++i) x[i] = x[i] + o[i];
}

int orc_session_feed(orc_session* s, const uint32_t* ids, uint64_t n, float* logits_last,
                     float* logits_all) {
    orc_model* m = s->m; const orc_config* c = &m->c;
    const uint64_t D = c->d_model, F = c->ffn, V = c->vocab, H = c->heads;
    if (n == 0) return 0;
    if (s->len + n > c->context) return fail(7, "Model::forward: seq_len exceeds context_length");
    for (uint64_t i = 0; i < n; ++i) if (ids[i] >= V) return fail(8, "token id out of range");
    float* x = (float*)malloc(n * D * sizeof(float));
    float* ws = (float*)malloc((n * (6 * D + 2 * F) + n * H * c->context) * sizeof(float));
    /* ops::embedding, src/ops/embedding.cpp:33-41 */
    for (uint64_t i = 0; i < n; ++i) memcpy(x + i * D, m->p[0].data + (uint64_t)ids[i] * D, D * sizeof(float));
    for (uint64_t l = 0; l < c->layers; ++l) block_forward(s, l, x, n, ws);
    s->len += n;
    /* final norm + tied head, src/model.cpp:55-60; matmul_bt src/ops/matmul.cpp:190-197 has
     * the same k-ascending sum as matmul on the transposed copy */
    const float* gf = m->p[m->np - 1].data;
    if (logits_all) {
        rmsnorm(x, gf, ws, n, D, c->eps);
        mm(ws, m->embT, logits_all, n, D, V);
        if (logits_last) memcpy(logits_last, logits_all + (n - 1) * V, V * sizeof(float));
    } else if (logits_last) {
        rmsnorm(x + (n - 1) * D, gf, ws, 1, D, c->eps);
        mm(ws, m->embT, logits_last, 1, D, V);
    }
    free(ws); free(x);
    return 0;
}

int orc_forward(orc_model* m, const uint32_t* ids, uint64_t B, uint64_t T, uint64_t row_from,
                float* logits) {
    if (T > m->c.context) return fail(7, "Model::forward: seq_len exceeds context_length");
    if (row_from > T) return fail(7, "orc_forward: row_from > T");
    orc_session* s = orc_session_create(m);
    const uint64_t V = m->c.vocab, keep = T - row_from;
    int rc = 0;
    for (uint64_t b = 0; b < B && !rc; ++b) {
        orc_session_reset(s);
        if (row_from > 0) rc = orc_session_feed(s, ids + b * T, row_from, NULL, NULL);
        if (!rc && keep) rc = orc_session_feed(s, ids + b * T + row_from, keep, NULL, logits + b * keep * V);
    }
    orc_session_destroy(s);
    return rc;
}

/* ------------------------------------------------------------------ sampler ---------- */
/* repetition penalty, src/inference.cpp:104-112: once per distinct id of the whole history */
static void apply_penalty(float* sc, uint64_t V, const uint32_t* hist, uint64_t nh, float pen) {
    if (pen == 1.0f) return;
    unsigned char* seen = (unsigned char*)calloc(V, 1);
    for (uint64_t i = 0; i < nh; ++i) {
        const uint32_t id = hist[i];
        if (id >= V || seen[id]) continue;
        seen[id] = 1;
        sc[id] = sc[id] > 0 ? sc[id] / pen : sc[id] * pen;
    }
    free(seen);
}

int64_t orc_greedy(const float* logits, uint64_t V, const uint32_t* hist, uint64_t nh, float pen,
                   float* top2_margin) {
    float* sc = (float*)malloc(V * sizeof(float));
    memcpy(sc, logits, V * sizeof(float));
    apply_penalty(sc, V, hist, nh, pen);
    uint64_t best = 0;                                       /* std::max_element: first max */
    for (uint64_t i = 1; i < V; ++i) if (sc[best] < sc[i]) best = i;
    if (top2_margin) {
        float second = -INFINITY;
        for (uint64_t i = 0; i < V; ++i) if (i != best && sc[i] > second) second = sc[i];
        *top2_margin = sc[best] - second;
    }
    free(sc);
    return (int64_t)best;
}

typedef struct { double p; uint32_t id; } cand;
static int cand_desc(const void* a, const void* b) {
    const cand* x = (const cand*)a; const cand* y = (const cand*)b;
    if (x->p > y->p) return -1;
    if (x->p < y->p) return 1;
    return x->id < y->id ? -1 : (x->id > y->id ? 1 : 0);     /* defined tie-break: lower id first */
}

static int64_t sample_impl(const float* logits, uint64_t V, const uint32_t* hist, uint64_t nh,
                           float temperature, float top_p, float pen, double u, double* margin,
                           uint64_t* kept_out) {
    float* sc = (float*)malloc(V * sizeof(float));
    memcpy(sc, logits, V * sizeof(float));
    apply_penalty(sc, V, hist, nh, pen);
    float mx = sc[0];
    for (uint64_t i = 1; i < V; ++i) if (mx < sc[i]) mx = sc[i];
    if (!isfinite(mx)) { free(sc); fail(9, "all logits are non-finite"); return -1; }
    /* src/inference.cpp:126-135: expf of a float argument, summed in double in id order */
    cand* cs = (cand*)malloc(V * sizeof(cand));
    double total = 0.0;
    for (uint64_t i = 0; i < V; ++i) {
        const double w = (double)expf((sc[i] - mx) / temperature);
        cs[i].p = w; cs[i].id = (uint32_t)i; total += w;
    }
    for (uint64_t i = 0; i < V; ++i) cs[i].p /= total;
    qsort(cs, V, sizeof(cand), cand_desc);                    /* :138 */
    /* top-p, :141-148 */
    double cum = 0.0, cum_prev = 0.0; uint64_t kept = 0;
    while (kept < V && cum < (double)top_p) { cum_prev = cum; cum += cs[kept].p; ++kept; }
    double mg = 1.0;
    if (kept < V || cum >= (double)top_p) {
        const double a = (double)top_p - cum_prev, b = cum - (double)top_p;
        if (a < mg) mg = a;
        if (kept < V && b < mg) mg = b;
    }
    /* std::discrete_distribution (libstdc++ random.tcc): <2 weights -> index 0, no draw;
     * else normalise by the sequential sum, running sum, last entry forced to 1, and
     * lower_bound(cp, u) = first index with cp[i] >= u */
    uint64_t pick = 0;
    if (kept >= 2) {
        double sum = 0.0;
        for (uint64_t i = 0; i < kept; ++i) sum += cs[i].p;
        double run = 0.0, prev = 0.0;
        pick = kept - 1;
        for (uint64_t i = 0; i < kept; ++i) {
            prev = run;
            run += cs[i].p / sum;
            const double cp = (i + 1 == kept) ? 1.0 : run;
            if (cp >= u) {
                pick = i;
                if (u - prev < mg && i > 0) mg = u - prev;
                if (i + 1 < kept && cp - u < mg) mg = cp - u;
                break;
            }
        }
    }
    const int64_t tok = cs[pick].id;
    if (margin) *margin = mg;
    if (kept_out) *kept_out = kept;
    free(cs); free(sc);
    return tok;
}
int64_t orc_sample(const float* logits, uint64_t V, const uint32_t* hist, uint64_t nh,
                   float temperature, float top_p, float pen, double u, double* margin) {
    return sample_impl(logits, V, hist, nh, temperature, top_p, pen, u, margin, NULL);
}

/* src/inference.cpp:21-173 */
static int generate_impl(orc_model* m, const uint32_t* prompt, uint64_t np, uint64_t max_new,
                         const orc_sampling* opt, const float* uniforms, const double* draws,
                         uint32_t* out, uint64_t* out_n) {
    if (np == 0) return fail(10, "Inference::generate: prompt encoded to zero tokens");
    const uint64_t ctx = m->c.context, V = m->c.vocab;
    if (ctx == 0) return fail(11, "Inference::generate: context length must be greater than zero");
    orc_session* s = orc_session_create(m);
    float* lg = (float*)malloc(V * sizeof(float));
    uint64_t n = np, fed = 0, used = 0; int rc = 0;
    memcpy(out, prompt, np * sizeof(uint32_t));
    for (uint64_t step = 0; step < max_new; ++step) {
        if (n > ctx) {                       /* window slides: positions restart at 0 (:40-48) */
            orc_session_reset(s);
            rc = orc_session_feed(s, out + (n - ctx), ctx, lg, NULL);
            fed = n;
        } else {
            rc = orc_session_feed(s, out + fed, n - fed, lg, NULL);
            fed = n;
        }
        if (rc) break;
        int64_t tok;
        if (opt->temperature <= 0.0f) tok = orc_greedy(lg, V, out, n, opt->repetition_penalty, NULL);
        else if (uniforms) tok = sample_impl(lg, V, out, n, opt->temperature, opt->top_p,
                                             opt->repetition_penalty, (double)uniforms[step], NULL, NULL);
        else {   /* the engine's own consumption rule: a draw is taken only when >= 2 are kept */
            uint64_t kept = 0;
            tok = sample_impl(lg, V, out, n, opt->temperature, opt->top_p, opt->repetition_penalty,
                              draws[used], NULL, &kept);
            if (kept >= 2) ++used;
        }
        if (tok < 0) { rc = 9; break; }
        out[n++] = (uint32_t)tok;
        if ((uint32_t)tok == opt->eos_token || tok == opt->stop_token) break;   /* :158-160 */
    }
    *out_n = n;
    free(lg); orc_session_destroy(s);
    return rc;
}
int orc_generate(orc_model* m, const uint32_t* prompt, uint64_t np, uint64_t max_new,
                 const orc_sampling* opt, const float* uniforms, uint32_t* out, uint64_t* out_n) {
    if (!uniforms && opt->temperature > 0.0f) return fail(12, "orc_generate: uniforms required");
    return generate_impl(m, prompt, np, max_new, opt, uniforms, NULL, out, out_n);
}
int orc_generate_seeded(orc_model* m, const uint32_t* prompt, uint64_t np, uint64_t max_new,
                        const orc_sampling* opt, uint64_t seed, uint32_t* out, uint64_t* out_n) {
    double* d = (double*)malloc((max_new + 1) * sizeof(double));
    orc_canonical64(seed, max_new + 1, d);
    const int rc = generate_impl(m, prompt, np, max_new, opt, NULL, d, out, out_n);
    free(d);
    return rc;
}

/* src/ops/cross_entropy.cpp:27-53: per counted row the fp32 maximum, the fp32 sequential sum of expf(l - max),
 * loss = -l[target] + (max + logf(sum)); rows are added in double and divided in double. */
float orc_cross_entropy(const float* logits, const int32_t* targets, uint64_t n, uint64_t V, uint64_t num_valid) {
    double total = 0.0;
    for (uint64_t i = 0; i < n; ++i) {
        if (targets[i] < 0) continue;
        const float* l = logits + i * V;
        float mx = l[0];
        for (uint64_t j = 0; j < V; ++j) mx = l[j] > mx ? l[j] : mx;
        float sum = 0.0f;
        for (uint64_t j = 0; j < V; ++j) sum += expf(l[j] - mx);
        const float lse = mx + logf(sum);
        const float loss = -l[targets[i]] + lse;
        total += loss;
    }
    return (float)(total / (double)(num_valid ? num_valid : n));
}
