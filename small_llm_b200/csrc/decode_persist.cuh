// Decode step for ONE new token as ONE persistent kernel: every layer, the final norm and the tied head.
//
// At batch 1 the model's weights stream in about 30 us, but the step is a chain of dependent products
// (norm -> QKV -> attention -> out-projection -> norm -> gate/up -> down, 16 times); what bounds it is the
// latency of handing a small vector from the blocks that produced it to the blocks that consume it.  This
// kernel keeps one block per SM resident for the whole token and makes that hand-off as short as a memory
// system allows:
//
//   * Every product is split by OUTPUT ROWS over all blocks (each block owns a contiguous range of QKV row
//     pairs, of residual rows for the out- and down-projection, of FFN hidden units, of vocabulary rows), so
//     each output element is computed by exactly one block: no partial sums, no atomics, results independent of
//     timing.
//   * A block's slice of a layer's weights (about 70 KB for the 100M model) is fetched into shared memory by bulk
//     asynchronous copies (cp.async.bulk, one per matrix slice since the rows are contiguous) a layer ahead:
//     weights do not depend on activations, so by the time a vector arrives only shared-memory arithmetic is left.
//     The same holds for the K/V pages of earlier positions, which an attention block fetches a layer ahead.
//   * Vectors travel through global memory (L2) as 64-bit words {value, tag}: the tag names the token step, the
//     layer and the hand-off, so a consumer polls the DATA itself until every word carries the expected tag - one
//     round trip, no separate flag, no fence (a 64-bit access is single-copy atomic).  Five hand-offs per layer:
//     x (all rows) -> QKV rows -> attention partials per (head, key range) -> x -> hidden units -> x.
//   * Every poll is bounded: a block that waits longer than the engine's wait limit raises the status word,
//     waits (bounded) for its own copies in flight and returns; the others run into the same limit.
//
// Buffers are reused by every layer.  That is safe because the hand-offs of x and of the hidden units are
// all-to-all: a block writes hand-off k+1 only after it has read all of hand-off k, i.e. after every block wrote k,
// i.e. after every block finished reading everything before k.
//
// Arithmetic follows the reference as the other decode kernels do (src/ops/rmsnorm.cpp:38-60, src/ops/rope.cpp:60-76,
// src/ops/attention.cpp:45-50,179-183, src/ops/softmax.cpp:24-40, src/nn/swiglu.cpp:37-57); fp32 residual stream
// and accumulation, bf16 weights and KV cache.
#pragma once
#include "common.cuh"

namespace sllm {

constexpr int kPsThreads = 512;
constexpr int kPsWarps = kPsThreads / 32;
constexpr int kPsHeadRows = 16;          // vocabulary rows per head stage (one per warp)
constexpr int kPsMaxHeadStages = 8;

struct PersistArgs {
    ModelDims m;
    KvView kv;
    const uint32_t* tok_id;              // the pass holds one token: index 0
    const int* tok_slot;
    const int* tok_pos;
    const LayerW* layers;                // device array [L]
    const float* emb_f32;                // [V][D] fp32 (gather)
    const __nv_bfloat16* emb_w;          // [V][D] bf16 (tied head)
    const float* g_final;
    const float2* rope;
    unsigned long long* xa;              // [D]   x entering a layer (and the final x)
    unsigned long long* xb;              // [D]   x after the attention half
    unsigned long long* qkv;             // [3D]  rotated q, rotated+rounded k, rounded v
    unsigned long long* ap;              // [H][S][hd + 2] attention partials (out, max, sum)
    unsigned long long* hb;              // [F]   hidden units
    unsigned int* epoch;                 // token-step counter (>= 1), advanced by block 0 at the end
    unsigned int* status;
    float* logits;                       // [V], or null: then the final residual goes to x_out
    float* x_out;                        // [D]
    int na;                              // blocks of the grid (every one owns rows of every product)
    int s_max;                           // key ranges per head at most (na / H)
    int pps_max;                         // KV pages per key range at most
};

// ---- shared-memory layout, the same arithmetic on host and device ---------------------------------------------
struct PsLayout {
    int rq, rx, ru;                      // most QKV rows, residual rows, hidden units of any block
    uint32_t o_wqkv, o_wo, o_wgu, o_wd, o_kv, o_region_end;      // [o_wqkv, o_region_end) is reused by the head stages
    uint32_t o_gattn, o_gffn, o_gfinal, o_xraw, o_xn, o_att, o_hid, o_ap, o_sc, o_qh, o_redo, o_rope, o_pages, o_red, o_bars;
    uint32_t total;
    int head_stages;
};
__host__ __device__ inline uint32_t ps_align(uint32_t v) { return (v + 127u) & ~127u; }
__host__ __device__ inline int ps_ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline PsLayout ps_layout(const ModelDims& m, int na, int s_max, int pps_max, int pages_per_seq) {
    PsLayout L;
    L.rq = 2 * ps_ceil_div(3 * m.D / 2, na);
    L.rx = ps_ceil_div(m.D, na);
    L.ru = ps_ceil_div(m.F, na);
    uint32_t o = 0;
    L.o_wqkv = o; o = ps_align(o + (uint32_t)L.rq * m.D * 2);
    L.o_wo = o;   o = ps_align(o + (uint32_t)L.rx * m.D * 2);
    L.o_wgu = o;  o = ps_align(o + (uint32_t)2 * L.ru * m.D * 2);
    L.o_wd = o;   o = ps_align(o + (uint32_t)L.rx * m.F * 2);
    L.o_kv = o;   o = ps_align(o + (uint32_t)pps_max * 2 * kPage * m.hd * 2);
    L.o_region_end = o;
    L.o_gattn = o;  o = ps_align(o + (uint32_t)m.D * 4);
    L.o_gffn = o;   o = ps_align(o + (uint32_t)m.D * 4);
    L.o_gfinal = o; o = ps_align(o + (uint32_t)m.D * 4);
    L.o_xraw = o;   o = ps_align(o + (uint32_t)m.D * 4);
    L.o_xn = o;     o = ps_align(o + (uint32_t)m.D * 4);
    L.o_att = o;    o = ps_align(o + (uint32_t)m.D * 4);
    L.o_hid = o;    o = ps_align(o + (uint32_t)m.F * 4);
    L.o_ap = o;     o = ps_align(o + (uint32_t)m.H * s_max * (m.hd + 2) * 4);
    L.o_sc = o;     o = ps_align(o + (uint32_t)pps_max * kPage * 4);
    L.o_qh = o;     o = ps_align(o + (uint32_t)3 * m.hd * 4);
    L.o_redo = o;   o = ps_align(o + (uint32_t)(kPsThreads / (m.hd / 2)) * (m.hd + 1) * 4);
    L.o_rope = o;   o = ps_align(o + (uint32_t)(m.hd / 2) * 8);
    L.o_pages = o;  o = ps_align(o + (uint32_t)pages_per_seq * 4);
    L.o_red = o;    o = ps_align(o + 64 * 4);
    L.o_bars = o;   o = ps_align(o + (5 + kPsMaxHeadStages) * 8);
    L.total = o;
    const uint32_t stage = (uint32_t)kPsHeadRows * m.D * 2;
    int hs = (int)((L.o_region_end - L.o_wqkv) / stage);
    L.head_stages = hs > kPsMaxHeadStages ? kPsMaxHeadStages : hs;
    return L;
}

// ---- tagged words through L2 -------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long ll_ld(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ll_st(unsigned long long* p, float val, uint32_t tag) {
    const unsigned long long v = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(val);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ps_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Copies n tagged words into dst as floats, polling each until it carries `tag`.  No barrier inside: the caller
// synchronises.  A wait that runs out raises *s_abort (shared memory) and the status word.
__device__ __forceinline__ void ll_gather(const unsigned long long* buf, int n, uint32_t tag, float* dst, volatile int* s_abort,
                                          unsigned int* status, unsigned int code) {
    constexpr int IF = 4;                    // words in flight per thread
    for (int base = threadIdx.x; base < n; base += kPsThreads * IF) {
        unsigned long long v[IF];
#pragma unroll
        for (int j = 0; j < IF; ++j) {
            const int idx = base + j * kPsThreads;
            v[j] = idx < n ? ll_ld(buf + idx) : ((unsigned long long)tag << 32);
        }
#pragma unroll
        for (int j = 0; j < IF; ++j) {
            const int idx = base + j * kPsThreads;
            if (idx >= n) continue;
            unsigned long long t0 = 0;
            uint32_t spins = 0;
            while ((uint32_t)(v[j] >> 32) != tag) {
                if ((++spins & 255u) == 0u) {
                    if (*s_abort) break;
                    const unsigned long long now = ps_now();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > c_wait_limit_ns) { *s_abort = 1; atomicExch(status, code); break; }
                }
                v[j] = ll_ld(buf + idx);
            }
            dst[idx] = __uint_as_float((uint32_t)v[j]);
        }
    }
}

// ---- shared-memory arithmetic -------------------------------------------------------------------------------------
// dot products of one / two bf16 rows in shared memory with an fp32 vector in shared memory; every lane gets the sums
__device__ __forceinline__ float ps_dot(const __nv_bfloat16* w, const float* x, int K) {
    const int lane = threadIdx.x & 31;
    float acc = 0.f;
    for (int c = lane; c < K / 8; c += 32) {
        float f[8];
        unpack16<__nv_bfloat16>(*reinterpret_cast<const uint4*>(w + c * 8), f);
        const float4 x0 = *reinterpret_cast<const float4*>(x + c * 8), x1 = *reinterpret_cast<const float4*>(x + c * 8 + 4);
        acc += f[0] * x0.x + f[1] * x0.y + f[2] * x0.z + f[3] * x0.w + f[4] * x1.x + f[5] * x1.y + f[6] * x1.z + f[7] * x1.w;
    }
    return warp_sum(acc);
}
__device__ __forceinline__ void ps_dot2(const __nv_bfloat16* w0, const __nv_bfloat16* w1, const float* x, int K, float& r0, float& r1) {
    const int lane = threadIdx.x & 31;
    float a0 = 0.f, a1 = 0.f;
    for (int c = lane; c < K / 8; c += 32) {
        float f[8], g[8];
        unpack16<__nv_bfloat16>(*reinterpret_cast<const uint4*>(w0 + c * 8), f);
        unpack16<__nv_bfloat16>(*reinterpret_cast<const uint4*>(w1 + c * 8), g);
        const float4 x0 = *reinterpret_cast<const float4*>(x + c * 8), x1 = *reinterpret_cast<const float4*>(x + c * 8 + 4);
        a0 += f[0] * x0.x + f[1] * x0.y + f[2] * x0.z + f[3] * x0.w + f[4] * x1.x + f[5] * x1.y + f[6] * x1.z + f[7] * x1.w;
        a1 += g[0] * x0.x + g[1] * x0.y + g[2] * x0.z + g[3] * x0.w + g[4] * x1.x + g[5] * x1.y + g[6] * x1.z + g[7] * x1.w;
    }
    r0 = warp_sum(a0);
    r1 = warp_sum(a1);
}

__device__ __forceinline__ uint32_t ps_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ps_bar_init(uint32_t bar) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar)); }
__device__ __forceinline__ void ps_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ps_bulk(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// generic-proxy reads of a buffer are done (block barrier before this); the bulk copy that refills it may start
__device__ __forceinline__ void ps_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void ps_part(int n, int parts, int i, int& b, int& e) {
    b = (int)((long long)n * i / parts);
    e = (int)((long long)n * (i + 1) / parts);
}

// RMSNorm of xraw into xn with `gain` (shared memory): y = (x * r) * g, r = 1 / sqrt(mean(x^2) + eps)
__device__ __forceinline__ void ps_norm(const float* xraw, const float* gain, float* xn, float* red, int D, float eps) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float ss = 0.f;
    for (int k = tid; k < D; k += kPsThreads) { const float v = xraw[k]; ss += v * v; }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kPsWarps; ++w) s += red[w];
    const float inv = 1.0f / sqrtf(s / (float)D + eps);
    for (int k = tid; k < D; k += kPsThreads) xn[k] = xraw[k] * inv * gain[k];
    __syncthreads();
}

enum { PS_B_QKV = 0, PS_B_O = 1, PS_B_GU = 2, PS_B_D = 3, PS_B_KV = 4, PS_B_HEAD = 5 };

template <int HD>
__global__ void __launch_bounds__(kPsThreads, 1) k_decode_persist(const PersistArgs a) {
    extern __shared__ __align__(128) unsigned char ps_smem_raw[];
    unsigned char* smem = ps_smem_raw;
    constexpr int LPK = HD / 8;                  // lanes per key row (16-byte pieces)
    constexpr int KPI = 32 / LPK;                // keys per warp instruction
    constexpr int DP = HD / 2;                   // threads across a value row (two dims each)
    constexpr int KG = kPsThreads / DP;          // key groups in the PV product
    const ModelDims& m = a.m;
    const int D = m.D, F = m.F, H = m.H, NL = m.L, V = m.V;
    const int cta = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const PsLayout lay = ps_layout(m, a.na, a.s_max, a.pps_max, a.kv.pages_per_seq);
    __nv_bfloat16* s_wqkv = reinterpret_cast<__nv_bfloat16*>(smem + lay.o_wqkv);
    __nv_bfloat16* s_wo = reinterpret_cast<__nv_bfloat16*>(smem + lay.o_wo);
    __nv_bfloat16* s_wgu = reinterpret_cast<__nv_bfloat16*>(smem + lay.o_wgu);
    __nv_bfloat16* s_wd = reinterpret_cast<__nv_bfloat16*>(smem + lay.o_wd);
    __nv_bfloat16* s_kv = reinterpret_cast<__nv_bfloat16*>(smem + lay.o_kv);
    float* s_gattn = reinterpret_cast<float*>(smem + lay.o_gattn);
    float* s_gffn = reinterpret_cast<float*>(smem + lay.o_gffn);
    float* s_gfinal = reinterpret_cast<float*>(smem + lay.o_gfinal);
    float* xraw = reinterpret_cast<float*>(smem + lay.o_xraw);
    float* xn = reinterpret_cast<float*>(smem + lay.o_xn);
    float* s_att = reinterpret_cast<float*>(smem + lay.o_att);
    float* s_hid = reinterpret_cast<float*>(smem + lay.o_hid);
    float* s_ap = reinterpret_cast<float*>(smem + lay.o_ap);
    float* s_sc = reinterpret_cast<float*>(smem + lay.o_sc);
    float* s_qh = reinterpret_cast<float*>(smem + lay.o_qh);
    float* s_redo = reinterpret_cast<float*>(smem + lay.o_redo);       // [KG][HD + 1]: partial outputs and sums of the key groups
    float2* s_rope = reinterpret_cast<float2*>(smem + lay.o_rope);
    int* s_pages = reinterpret_cast<int*>(smem + lay.o_pages);
    float* s_red = reinterpret_cast<float*>(smem + lay.o_red);
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_red + 32);
    const uint32_t bar0 = ps_smem(smem + lay.o_bars);
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    // this block's rows of every product
    int pp0, pp1, d0, d1, u0, u1, v0, v1;
    ps_part(3 * D / 2, a.na, cta, pp0, pp1);     // QKV row pairs (a RoPE pair stays in one block)
    ps_part(D, a.na, cta, d0, d1);               // residual rows: out- and down-projection
    ps_part(F, a.na, cta, u0, u1);               // hidden units: gate / up row pairs
    ps_part(V, a.na, cta, v0, v1);               // vocabulary rows of the head
    const int nq = 2 * (pp1 - pp0), nx = d1 - d0, nu = u1 - u0;

    if (tid == 0) {
        for (int i = 0; i < 5 + kPsMaxHeadStages; ++i) ps_bar_init(BAR(i));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *s_abort = 0;
    }
    __syncthreads();
    // loads issued / waited per barrier, identical in every thread (uniform control flow)
    int n_issued[5] = {0, 0, 0, 0, 0}, n_waited[5] = {0, 0, 0, 0, 0};
    auto issue_qkv = [&](int l) {
        if (tid == 0) {
            const uint32_t bytes = (uint32_t)nq * D * 2;
            ps_expect(BAR(PS_B_QKV), bytes + (uint32_t)D * 4);
            ps_bulk(ps_smem(s_wqkv), reinterpret_cast<const __nv_bfloat16*>(a.layers[l].wqkv) + (size_t)2 * pp0 * D, bytes, BAR(PS_B_QKV));
            ps_bulk(ps_smem(s_gattn), a.layers[l].g_attn, (uint32_t)D * 4, BAR(PS_B_QKV));
        }
        n_issued[PS_B_QKV] += 1;
    };
    auto issue_o = [&](int l) {
        if (tid == 0) {
            const uint32_t bytes = (uint32_t)nx * D * 2;
            ps_expect(BAR(PS_B_O), bytes);
            ps_bulk(ps_smem(s_wo), reinterpret_cast<const __nv_bfloat16*>(a.layers[l].wo) + (size_t)d0 * D, bytes, BAR(PS_B_O));
        }
        n_issued[PS_B_O] += 1;
    };
    auto issue_gu = [&](int l) {
        if (tid == 0) {
            const uint32_t bytes = (uint32_t)2 * nu * D * 2;
            ps_expect(BAR(PS_B_GU), bytes + (uint32_t)D * 4);
            ps_bulk(ps_smem(s_wgu), reinterpret_cast<const __nv_bfloat16*>(a.layers[l].wgu) + (size_t)2 * u0 * D, bytes, BAR(PS_B_GU));
            ps_bulk(ps_smem(s_gffn), a.layers[l].g_ffn, (uint32_t)D * 4, BAR(PS_B_GU));
        }
        n_issued[PS_B_GU] += 1;
    };
    auto issue_d = [&](int l) {
        if (tid == 0) {
            const uint32_t bytes = (uint32_t)nx * F * 2;
            ps_expect(BAR(PS_B_D), bytes);
            ps_bulk(ps_smem(s_wd), reinterpret_cast<const __nv_bfloat16*>(a.layers[l].wd) + (size_t)d0 * F, bytes, BAR(PS_B_D));
        }
        n_issued[PS_B_D] += 1;
    };
    // every thread waits for the copy (cheap once it has landed); the block barrier that follows makes the verdict
    // uniform: false = a wait ran out somewhere in the block
    auto wait_bar = [&](int b, unsigned int code) -> bool {
        const bool ok = mbar_wait_bounded(BAR(b), (uint32_t)(n_waited[b] & 1), c_wait_limit_ns);
        n_waited[b] += 1;
        if (!ok) { *s_abort = 1; atomicExch(a.status, code); }
        __syncthreads();
        return *s_abort == 0;
    };

    // the first layer's weights do not depend on the previous kernel: fetch them before the dependency wait
    issue_qkv(0); issue_o(0); issue_gu(0); issue_d(0);
    for (int k = tid; k < D; k += kPsThreads) s_gfinal[k] = a.g_final[k];
    SLLM_TL(400);
    pdl_launch_dependents();
    pdl_wait();
    SLLM_TL(401);

    bool live = *reinterpret_cast<volatile unsigned int*>(a.status) == 0u;     // an earlier failure: do nothing but drain
    const uint32_t epoch = *a.epoch;
    const int pos = a.tok_pos[0], slot = a.tok_slot[0];
    const uint32_t tok = a.tok_id[0];
    const int n_pages = pos / kPage + 1;
    for (int i = tid; i < HD / 2; i += kPsThreads) s_rope[i] = a.rope[(size_t)pos * (HD / 2) + i];
    for (int i = tid; i < n_pages; i += kPsThreads) s_pages[i] = a.kv.block_table[(size_t)slot * a.kv.pages_per_seq + i];
    for (int k = tid; k < D; k += kPsThreads) xraw[k] = a.emb_f32[(size_t)tok * D + k];
    // attention role: head ah, key range as of S; ranges of pps consecutive pages
    const int pps = max(2, ps_ceil_div(n_pages, a.s_max));
    const int S = ps_ceil_div(n_pages, pps);
    const bool attn_cta = cta < H * S;
    const int ah = attn_cta ? cta / S : 0, as = attn_cta ? cta % S : 0;
    const int p_lo = min(n_pages, as * pps), p_hi = attn_cta ? min(n_pages, p_lo + pps) : p_lo;
    const int my_pages = p_hi - p_lo;
    const size_t page_elems = (size_t)kPage * HD;
    __syncthreads();
    auto issue_kv = [&](int l) {
        if (my_pages > 0) {
            if (tid == 0) {
                ps_expect(BAR(PS_B_KV), (uint32_t)(my_pages * 2 * page_elems * 2));
                for (int p = 0; p < my_pages; ++p) {
                    const int page = s_pages[p_lo + p];
                    ps_bulk(ps_smem(s_kv + (size_t)(2 * p) * page_elems), kv_ptr<__nv_bfloat16>(a.kv, m, l, page, 0, ah, 0),
                            (uint32_t)(page_elems * 2), BAR(PS_B_KV));
                    ps_bulk(ps_smem(s_kv + (size_t)(2 * p + 1) * page_elems), kv_ptr<__nv_bfloat16>(a.kv, m, l, page, 1, ah, 0),
                            (uint32_t)(page_elems * 2), BAR(PS_B_KV));
                }
            }
            n_issued[PS_B_KV] += 1;
        }
    };
    if (live) issue_kv(0);
    const int page_new = s_pages[pos / kPage];

    for (int l = 0; l < NL && live; ++l) {
        const uint32_t tg = epoch * 1024u + (uint32_t)l * 8u;
        // ---- x entering the layer (layer 0: the embedding row, already in xraw) ----------------------------------
        if (l > 0) {
            ll_gather(a.xa, D, tg + 0u, xraw, s_abort, a.status, 70u);
            __syncthreads();
            if (*s_abort) { live = false; break; }
        }
        SLLM_TL(410);
        if (!wait_bar(PS_B_QKV, 71u)) { live = false; break; }
        SLLM_TL(411);
        ps_norm(xraw, s_gattn, xn, s_red, D, m.eps);
        SLLM_TL(412);
        // ---- this block's QKV row pairs: RoPE, K/V to the cache, all three to the consumers -----------------------
        for (int pi = warp; pi < pp1 - pp0; pi += kPsWarps) {
            float r0, r1;
            ps_dot2(s_wqkv + (size_t)(2 * pi) * D, s_wqkv + (size_t)(2 * pi + 1) * D, xn, D, r0, r1);
            const int row = 2 * (pp0 + pi);
            const int which = row / D, col = row - which * D, head = col / HD, d = col - head * HD;
            float o0 = r0, o1 = r1;
            if (which < 2) {                               // interleaved-pair rotation, src/ops/rope.cpp:60-76
                const float2 cs = s_rope[d >> 1];
                o0 = r0 * cs.x - r1 * cs.y;
                o1 = r0 * cs.y + r1 * cs.x;
            }
            if (which > 0) {                               // the cache holds the rounded value; attention must see the same
                const __nv_bfloat16 b0 = __float2bfloat16_rn(o0), b1 = __float2bfloat16_rn(o1);
                o0 = __bfloat162float(b0); o1 = __bfloat162float(b1);
                if (lane == 0) {
                    __nv_bfloat16* dst = kv_ptr<__nv_bfloat16>(a.kv, m, l, page_new, which - 1, head, pos % kPage) + d;
                    *reinterpret_cast<__nv_bfloat162*>(dst) = __halves2bfloat162(b0, b1);
                }
            }
            if (lane == 0) { ll_st(a.qkv + row, o0, tg + 1u); ll_st(a.qkv + row + 1, o1, tg + 1u); }
        }
        __syncthreads();                                   // every warp is done with s_wqkv, s_gattn
        SLLM_TL(413);
        if (l + 1 < NL) { if (tid == 0) ps_fence_async(); issue_qkv(l + 1); }
        // ---- attention over this block's key range -------------------------------------------------------------------
        if (attn_cta) {
            ll_gather(a.qkv + (size_t)ah * HD, HD, tg + 1u, s_qh, s_abort, a.status, 72u);
            ll_gather(a.qkv + (size_t)D + (size_t)ah * HD, HD, tg + 1u, s_qh + HD, s_abort, a.status, 72u);
            ll_gather(a.qkv + (size_t)2 * D + (size_t)ah * HD, HD, tg + 1u, s_qh + 2 * HD, s_abort, a.status, 72u);
            __syncthreads();
            if (*s_abort) { live = false; break; }
            SLLM_TL(414);
            float part = 0.f;                              // thread i < HD + 2: out[i] | max | sum of this key range
            if (my_pages > 0) {
                if (!wait_bar(PS_B_KV, 73u)) { live = false; break; }
                SLLM_TL(415);
                const int kb = p_lo * kPage;
                const int nk = min(my_pages * kPage, pos + 1 - kb);            // keys of this range that exist
                const int sub = lane % LPK, rsub = lane / LPK;
                float qf[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) qf[e] = s_qh[sub * 8 + e];
                for (int j0 = warp * KPI; j0 < nk; j0 += kPsWarps * KPI) {
                    const int j = j0 + rsub;
                    float s = 0.f;
                    if (j < nk) {
                        if (kb + j == pos) {               // the new key: its cache row is being written right now
#pragma unroll
                            for (int e = 0; e < 8; ++e) s += qf[e] * s_qh[HD + sub * 8 + e];
                        } else {
                            const __nv_bfloat16* kr = s_kv + (size_t)(2 * (j / kPage)) * page_elems + (size_t)(j % kPage) * HD + sub * 8;
                            float kf[8];
                            unpack16<__nv_bfloat16>(*reinterpret_cast<const uint4*>(kr), kf);
#pragma unroll
                            for (int e = 0; e < 8; ++e) s += qf[e] * kf[e];
                        }
                    }
#pragma unroll
                    for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    if (sub == 0 && j < nk) s_sc[j] = s * m.scale;
                }
                __syncthreads();
                float mx = -INFINITY;                      // every warp finds the range's maximum for itself
                for (int j = lane; j < nk; j += 32) mx = fmaxf(mx, s_sc[j]);
                mx = warp_max(mx);
                const int dp = tid % DP, kg = tid / DP;
                float o0 = 0.f, o1 = 0.f, lsum = 0.f;
                for (int j = kg; j < nk; j += KG) {
                    const float p = expf(s_sc[j] - mx);
                    float w0, w1;
                    if (kb + j == pos) { w0 = s_qh[2 * HD + 2 * dp]; w1 = s_qh[2 * HD + 2 * dp + 1]; }
                    else {
                        const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(
                            s_kv + (size_t)(2 * (j / kPage) + 1) * page_elems + (size_t)(j % kPage) * HD + 2 * dp);
                        w0 = __low2float(vv); w1 = __high2float(vv);
                    }
                    lsum += p; o0 += p * w0; o1 += p * w1;
                }
                s_redo[kg * (HD + 1) + 2 * dp] = o0;
                s_redo[kg * (HD + 1) + 2 * dp + 1] = o1;
                if (dp == 0) s_redo[kg * (HD + 1) + HD] = lsum;
                __syncthreads();
                if (tid < HD) { for (int g = 0; g < KG; ++g) part += s_redo[g * (HD + 1) + tid]; }
                else if (tid == HD) part = mx;
                else if (tid == HD + 1) { for (int g = 0; g < KG; ++g) part += s_redo[g * (HD + 1) + HD]; }
            } else if (tid == HD) {
                part = -INFINITY;                          // an empty range: ignored by the merge
            }
            if (tid < HD + 2) ll_st(a.ap + ((size_t)(ah * S + as) * (HD + 2) + tid), part, tg + 2u);
            __syncthreads();                               // s_kv is free: fetch the next layer's pages
            SLLM_TL(416);
            if (l + 1 < NL) { if (tid == 0) ps_fence_async(); issue_kv(l + 1); }
        }
        // ---- merge the key ranges of every head (in range order), out-projection rows, residual --------------------
        ll_gather(a.ap, H * S * (HD + 2), tg + 2u, s_ap, s_abort, a.status, 74u);
        __syncthreads();
        if (*s_abort) { live = false; break; }
        SLLM_TL(417);
        for (int t = tid; t < D; t += kPsThreads) {
            const int h = t / HD, d = t - h * HD;
            const float* ph = s_ap + (size_t)h * S * (HD + 2);
            float mx = -INFINITY;
            for (int s = 0; s < S; ++s) mx = fmaxf(mx, ph[s * (HD + 2) + HD]);
            float num = 0.f, den = 0.f;
            for (int s = 0; s < S; ++s) {
                const float mr = ph[s * (HD + 2) + HD];
                if (mr == -INFINITY) continue;
                const float w = expf(mr - mx);
                den += w * ph[s * (HD + 2) + HD + 1];
                num += w * ph[s * (HD + 2) + d];
            }
            s_att[t] = num / den;
        }
        if (!wait_bar(PS_B_O, 75u)) { live = false; break; }      // its barrier also publishes s_att
        SLLM_TL(418);
        for (int r = warp; r < nx; r += kPsWarps) {
            const float y = ps_dot(s_wo + (size_t)r * D, s_att, D);
            if (lane == 0) ll_st(a.xb + d0 + r, xraw[d0 + r] + y, tg + 3u);
        }
        __syncthreads();
        SLLM_TL(419);
        if (l + 1 < NL) { if (tid == 0) ps_fence_async(); issue_o(l + 1); }
        // ---- x after the attention half, norm, this block's hidden units ---------------------------------------------
        ll_gather(a.xb, D, tg + 3u, xraw, s_abort, a.status, 76u);
        __syncthreads();
        if (*s_abort) { live = false; break; }
        SLLM_TL(420);
        if (!wait_bar(PS_B_GU, 77u)) { live = false; break; }
        ps_norm(xraw, s_gffn, xn, s_red, D, m.eps);
        SLLM_TL(421);
        for (int u = warp; u < nu; u += kPsWarps) {
            float g, up;
            ps_dot2(s_wgu + (size_t)(2 * u) * D, s_wgu + (size_t)(2 * u + 1) * D, xn, D, g, up);
            if (lane == 0) {                               // silu(g) * up, src/nn/swiglu.cpp:37-57
                const float sig = 1.0f / (1.0f + expf(-g));
                ll_st(a.hb + u0 + u, (g * sig) * up, tg + 4u);
            }
        }
        __syncthreads();
        SLLM_TL(422);
        if (l + 1 < NL) { if (tid == 0) ps_fence_async(); issue_gu(l + 1); }
        // ---- all hidden units, down-projection rows, residual -----------------------------------------------------------
        ll_gather(a.hb, F, tg + 4u, s_hid, s_abort, a.status, 78u);
        __syncthreads();
        if (*s_abort) { live = false; break; }
        SLLM_TL(423);
        if (!wait_bar(PS_B_D, 79u)) { live = false; break; }
        SLLM_TL(424);
        for (int r = warp; r < nx; r += kPsWarps) {
            const float y = ps_dot(s_wd + (size_t)r * F, s_hid, F);
            if (lane == 0) {
                const float xnew = xraw[d0 + r] + y;
                ll_st(a.xa + d0 + r, xnew, tg + 8u);        // tag of the next layer's (or the head's) x
                if (l + 1 == NL && a.logits == nullptr) a.x_out[d0 + r] = xnew;
            }
        }
        __syncthreads();
        SLLM_TL(425);
        if (l + 1 < NL) { if (tid == 0) ps_fence_async(); issue_d(l + 1); }
    }

    // ---- final norm and the tied head: this block's vocabulary rows streamed through the freed weight buffers ------
    if (live && a.logits != nullptr) {
        const uint32_t stage_bytes = (uint32_t)kPsHeadRows * D * 2;
        const int n_rows = v1 - v0, n_st = ps_ceil_div(n_rows, kPsHeadRows), ns = lay.head_stages;
        auto issue_head = [&](int st) {
            if (tid == 0) {
                const int rows = min(kPsHeadRows, n_rows - st * kPsHeadRows);
                const uint32_t bytes = (uint32_t)rows * D * 2;
                ps_expect(BAR(PS_B_HEAD + st % ns), bytes);
                ps_bulk(ps_smem(smem + lay.o_wqkv) + (uint32_t)(st % ns) * stage_bytes, a.emb_w + (size_t)(v0 + st * kPsHeadRows) * D, bytes,
                        BAR(PS_B_HEAD + st % ns));
            }
        };
        if (tid == 0) ps_fence_async();
        int issued = 0;
        for (; issued < min(ns, n_st); ++issued) issue_head(issued);
        ll_gather(a.xa, D, epoch * 1024u + (uint32_t)NL * 8u, xraw, s_abort, a.status, 80u);
        __syncthreads();
        bool go = *s_abort == 0;
        SLLM_TL(430);
        if (go) ps_norm(xraw, s_gfinal, xn, s_red, D, m.eps);
        for (int st = 0; st < issued; ++st) {              // after a failure nothing more is issued: the loop drains
            const bool ok = mbar_wait_bounded(BAR(PS_B_HEAD + st % ns), (uint32_t)((st / ns) & 1), c_wait_limit_ns);
            if (!ok) { *s_abort = 1; atomicExch(a.status, 81u); }
            const int row = st * kPsHeadRows + warp;
            if (go && ok && row < n_rows) {
                const float y = ps_dot(reinterpret_cast<const __nv_bfloat16*>(smem + lay.o_wqkv + (size_t)(st % ns) * stage_bytes) + (size_t)warp * D, xn, D);
                if (lane == 0) a.logits[v0 + row] = y;
            }
            __syncthreads();
            go = go && *s_abort == 0;
            if (go && issued < n_st) { if (tid == 0) ps_fence_async(); issue_head(issued); ++issued; }
        }
    } else {
        // a wait ran out (or an earlier kernel's did): let this block's copies in flight land before its shared
        // memory is given to another block
        for (int b = 0; b < 5; ++b)
            while (n_waited[b] < n_issued[b]) { mbar_wait_bounded(BAR(b), (uint32_t)(n_waited[b] & 1), c_wait_limit_ns); n_waited[b] += 1; }
    }
    SLLM_TL(432);
    if (cta == 0 && tid == 0) *a.epoch = epoch + 1u;
}

}  // namespace sllm
