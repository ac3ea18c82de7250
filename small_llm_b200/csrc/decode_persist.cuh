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
// Measured and dropped: requesting every polled word three times 0.15 us apart (slower: 354 against 329 us per token
// on the same GPU), sleeping 50-300 ns between two polls of a word (284 -> 364-383 us), letting the blocks without an attention role sleep
// 0.2-2.5 us before they poll for the partials (262.5 -> 258.2 us at best, 270.5 at worst), splitting a down-projection row over several warps (two more block barriers cost more than the
// shorter sums saved).
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
#include "sampler.cuh"

namespace sllm {

constexpr int kPsThreads = 512;         // threads that compute; one more warp only issues the bulk copies
constexpr int kPsWarps = kPsThreads / 32;
constexpr int kPsBlock = kPsThreads + 32;
constexpr int kPsHeadRows = 32;          // vocabulary rows per head stage (two per warp)
constexpr int kPsMaxHeadStages = 12;

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
    uint32_t smem_total;                 // dynamic shared memory of the launch
    // The first two kernels of the sampler that follows (k_samp_max, k_samp_hist) done here, by the blocks that hold
    // the logits: per-block first maximum of the penalised scores, the slot's maximum (one more hand-off), the weights
    // expf((s - max) / T) and their level-0 histogram.  Off when fold_temperature < 0.
    float fold_temperature, fold_penalty;
    SeqState st;
    unsigned long long* g_mass; unsigned int* g_cnt; float* g_w; float* g_pmax_val; int* g_pmax_idx;
    unsigned long long* mxb;             // [2 * na] tagged words: every block's (maximum, index)
};

// ---- shared-memory layout, the same arithmetic on host and device ---------------------------------------------
struct PsLayout {
    int rq, rx, ru;                      // most QKV rows, residual rows, hidden units of any block
    uint32_t o_wqkv, o_wo, o_wgu, o_wd, o_kv, o_region_end;      // [o_wqkv, o_region_end) is reused by the head stages
    uint32_t o_gattn, o_gffn, o_gfinal, o_xraw, o_xn, o_att, o_hid, o_ap, o_sc, o_qh, o_redo, o_rope, o_pages, o_red, o_bars, o_logits, o_head_pre;
    uint32_t total;                      // bytes the layers need; the head's early stages take what is left of smem_total
    int head_stages, head_pre;
};
__host__ __device__ inline uint32_t ps_align(uint32_t v) { return (v + 127u) & ~127u; }
__host__ __device__ inline int ps_ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline PsLayout ps_layout(const ModelDims& m, int na, int s_max, int pps_max, int pages_per_seq, uint32_t smem_total) {
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
    L.o_sc = o;     o = ps_align(o + (uint32_t)(pps_max * kPage > m.H * s_max ? pps_max * kPage : m.H * s_max) * 4);   // scores of a key range; later one weight per (head, range)
    L.o_qh = o;     o = ps_align(o + (uint32_t)3 * m.hd * 4);
    L.o_redo = o;   o = ps_align(o + (uint32_t)kPsWarps * (m.hd + 2) * 4);
    L.o_rope = o;   o = ps_align(o + (uint32_t)(m.hd / 2) * 8);
    L.o_pages = o;  o = ps_align(o + (uint32_t)pages_per_seq * 4);
    L.o_red = o;    o = ps_align(o + 64 * 4);
    L.o_bars = o;   o = ps_align(o + 2 * (5 + kPsMaxHeadStages) * 8);
    L.o_logits = o; o = ps_align(o + (uint32_t)ps_ceil_div(m.V, na) * 4);
    L.o_head_pre = o;
    L.total = o;
    const uint32_t stage = (uint32_t)kPsHeadRows * m.D * 2;
    int hs = (int)((L.o_region_end - L.o_wqkv) / stage);
    L.head_stages = hs > kPsMaxHeadStages / 2 ? kPsMaxHeadStages / 2 : hs;
    int pre = smem_total > o ? (int)((smem_total - o) / stage) : 0;
    L.head_pre = pre > kPsMaxHeadStages - L.head_stages ? kPsMaxHeadStages - L.head_stages : pre;
    return L;
}

// barrier of the kPsThreads computing threads (the copy-issuing warp is not part of it)
__device__ __forceinline__ void ps_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kPsThreads) : "memory"); }
__device__ __forceinline__ void ps_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

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
// seg_len / seg_stride: the words are n / seg_len runs of seg_len consecutive words, seg_stride apart in buf
// (one run: seg_len = n).  With `gain`, dst2[i] = value * gain[i] is stored too and the thread's sum of squares of
// the values is returned (for the RMSNorm that follows: y = (x * r) * g is applied as r * (W . (x * g))).
template <int IF>
__device__ __forceinline__ float ll_gather(const unsigned long long* buf, int n, int seg_len, int seg_stride, uint32_t tag, float* dst,
                                           const float* gain, float* dst2, volatile int* s_abort, unsigned int* status,
                                           unsigned int code) {
    float ss = 0.f;
    for (int base = threadIdx.x; base < n; base += kPsThreads * IF) {
        unsigned long long v[IF];
        const unsigned long long* src[IF];
#pragma unroll
        for (int j = 0; j < IF; ++j) {
            const int idx = base + j * kPsThreads;
            const int seg = idx / seg_len;
            src[j] = buf + (size_t)seg * seg_stride + (idx - seg * seg_len);
            v[j] = idx < n ? ll_ld(src[j]) : ((unsigned long long)tag << 32);
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
                v[j] = ll_ld(src[j]);
            }
            const float x = __uint_as_float((uint32_t)v[j]);
            dst[idx] = x;
            if (gain) { dst2[idx] = x * gain[idx]; ss += x * x; }
        }
    }
    return ss;
}

// Block-wide 1 / sqrt(mean(x^2) + eps) from the threads' partial sums of squares; contains the block barrier that also
// publishes what the threads wrote to shared memory before the call.
__device__ __forceinline__ float ps_inv_rms(float ss, float* red, int D, float eps) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    ps_sync();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kPsWarps; ++w) s += red[w];
    return rsqrtf(s / (float)D + eps);
}

// ---- shared-memory arithmetic -------------------------------------------------------------------------------------
// dot products of one / two bf16 rows in shared memory with an fp32 vector in shared memory; every lane gets the sums
__device__ __forceinline__ float ps_dot_part(const __nv_bfloat16* w, const float* x, int c_begin, int c_end) {
    float a0 = 0.f, a1 = 0.f;                // two chains: the sum's latency is what bounds these products
    for (int c = c_begin + (threadIdx.x & 31); c < c_end; c += 32) {
        float f[8];
        unpack16<__nv_bfloat16>(*reinterpret_cast<const uint4*>(w + c * 8), f);
        const float4 x0 = *reinterpret_cast<const float4*>(x + c * 8), x1 = *reinterpret_cast<const float4*>(x + c * 8 + 4);
        a0 += f[0] * x0.x + f[1] * x0.y + f[2] * x0.z + f[3] * x0.w;
        a1 += f[4] * x1.x + f[5] * x1.y + f[6] * x1.z + f[7] * x1.w;
    }
    return a0 + a1;
}
__device__ __forceinline__ float ps_dot(const __nv_bfloat16* w, const float* x, int K) { return warp_sum(ps_dot_part(w, x, 0, K / 8)); }
__device__ __forceinline__ void ps_dot2(const __nv_bfloat16* w0, const __nv_bfloat16* w1, const float* x, int K, float& r0, float& r1) {
    const int lane = threadIdx.x & 31;
    float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
    for (int c = lane; c < K / 8; c += 32) {
        float f[8], g[8];
        unpack16<__nv_bfloat16>(*reinterpret_cast<const uint4*>(w0 + c * 8), f);
        unpack16<__nv_bfloat16>(*reinterpret_cast<const uint4*>(w1 + c * 8), g);
        const float4 x0 = *reinterpret_cast<const float4*>(x + c * 8), x1 = *reinterpret_cast<const float4*>(x + c * 8 + 4);
        a0 += f[0] * x0.x + f[1] * x0.y + f[2] * x0.z + f[3] * x0.w;
        a1 += f[4] * x1.x + f[5] * x1.y + f[6] * x1.z + f[7] * x1.w;
        b0 += g[0] * x0.x + g[1] * x0.y + g[2] * x0.z + g[3] * x0.w;
        b1 += g[4] * x1.x + g[5] * x1.y + g[6] * x1.z + g[7] * x1.w;
    }
    a0 += a1; b0 += b1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {           // the two reductions interleaved
        a0 += __shfl_xor_sync(0xffffffffu, a0, o);
        b0 += __shfl_xor_sync(0xffffffffu, b0, o);
    }
    r0 = a0; r1 = b0;
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

enum { PS_B_QKV = 0, PS_B_O = 1, PS_B_GU = 2, PS_B_D = 3, PS_B_KV = 4, PS_B_HEAD = 5, PS_N_BARS = 5 + kPsMaxHeadStages };

template <int HD>
__global__ void __launch_bounds__(kPsBlock, 1) k_decode_persist(const PersistArgs a) {
    extern __shared__ __align__(128) unsigned char ps_smem_raw[];
    unsigned char* smem = ps_smem_raw;
    constexpr int LPK = HD / 8;                  // lanes per key row (16-byte pieces)
    constexpr int KPI = 32 / LPK;                // keys per warp instruction
    const ModelDims& m = a.m;
    const int D = m.D, F = m.F, H = m.H, NL = m.L, V = m.V;
    const int cta = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const PsLayout lay = ps_layout(m, a.na, a.s_max, a.pps_max, a.kv.pages_per_seq, a.smem_total);
    __nv_bfloat16* s_wqkv = reinterpret_cast<__nv_bfloat16*>(smem + lay.o_wqkv);
    __nv_bfloat16* s_wo = reinterpret_cast<__nv_bfloat16*>(smem + lay.o_wo);
    __nv_bfloat16* s_wgu = reinterpret_cast<__nv_bfloat16*>(smem + lay.o_wgu);
    __nv_bfloat16* s_wd = reinterpret_cast<__nv_bfloat16*>(smem + lay.o_wd);
    __nv_bfloat16* s_kv = reinterpret_cast<__nv_bfloat16*>(smem + lay.o_kv);
    float* s_gattn = reinterpret_cast<float*>(smem + lay.o_gattn);
    float* s_gffn = reinterpret_cast<float*>(smem + lay.o_gffn);
    float* s_gfinal = reinterpret_cast<float*>(smem + lay.o_gfinal);
    float* xraw = reinterpret_cast<float*>(smem + lay.o_xraw);
    float* xg = reinterpret_cast<float*>(smem + lay.o_xn);             // x * gain of the norm ahead (1/rms is applied to the products)
    float* s_att = reinterpret_cast<float*>(smem + lay.o_att);
    float* s_hid = reinterpret_cast<float*>(smem + lay.o_hid);
    float* s_ap = reinterpret_cast<float*>(smem + lay.o_ap);
    float* s_sc = reinterpret_cast<float*>(smem + lay.o_sc);
    float* s_qh = reinterpret_cast<float*>(smem + lay.o_qh);
    float* s_redo = reinterpret_cast<float*>(smem + lay.o_redo);       // [warp][HD + 2]: partial attention results of the warps
    float2* s_rope = reinterpret_cast<float2*>(smem + lay.o_rope);
    int* s_pages = reinterpret_cast<int*>(smem + lay.o_pages);
    float* s_red = reinterpret_cast<float*>(smem + lay.o_red);
    float* s_logits = reinterpret_cast<float*>(smem + lay.o_logits);   // this block's logits, for the folded sampler kernels
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_red + 32);
    const uint32_t bar0 = ps_smem(smem + lay.o_bars);
    auto FULL = [&](int i) { return bar0 + 8u * (uint32_t)i; };                   // "the copy has landed"
    auto FREE = [&](int i) { return bar0 + 8u * (uint32_t)(PS_N_BARS + i); };     // "the buffer may be overwritten"

    // this block's rows of every product
    int pp0, pp1, d0, d1, u0, u1, v0, v1;
    ps_part(3 * D / 2, a.na, cta, pp0, pp1);     // QKV row pairs (a RoPE pair stays in one block)
    ps_part(D, a.na, cta, d0, d1);               // residual rows: out- and down-projection
    ps_part(F, a.na, cta, u0, u1);               // hidden units: gate / up row pairs
    ps_part(V, a.na, cta, v0, v1);               // vocabulary rows of the head
    const int nq = 2 * (pp1 - pp0), nx = d1 - d0, nu = u1 - u0;
    // the head's stages: slot i < n_pre lives in shared memory that nothing else uses, the others reuse the layers'
    // weight and KV buffers once the last layer is done
    const uint32_t stage_bytes = (uint32_t)kPsHeadRows * D * 2;
    const int n_head_rows = v1 - v0, n_st = a.logits ? ps_ceil_div(n_head_rows, kPsHeadRows) : 0;
    const int n_pre = lay.head_pre, ns = lay.head_pre + lay.head_stages;
    auto head_slot = [&](int slot) -> unsigned char* {
        return slot < n_pre ? smem + lay.o_head_pre + (size_t)slot * stage_bytes : smem + lay.o_wqkv + (size_t)(slot - n_pre) * stage_bytes;
    };
    const size_t page_elems = (size_t)kPage * HD;

    PS_TL_INIT(20 * NL + 8);
    if (tid == 0) {
        for (int i = 0; i < 2 * PS_N_BARS; ++i) ps_bar_init(bar0 + 8u * (uint32_t)i);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *s_abort = 0;
    }
    __syncthreads();

    // ============================================================================================================
    // The copy warp: one thread issues every bulk copy of the block, a layer ahead of its use, so that the computing
    // threads never spend their time on it.  It learns that a buffer may be refilled from the FREE barriers, on which
    // a computing thread arrives after the block barrier that ends the buffer's last use.
    // ============================================================================================================
    if (warp == kPsWarps) {
        if (lane != 0) return;
        auto issue = [&](int b, void* dst, const void* src, uint32_t bytes, const void* src2, void* dst2, uint32_t bytes2) {
            ps_expect(FULL(b), bytes + bytes2);
            ps_bulk(ps_smem(dst), src, bytes, FULL(b));
            if (bytes2) ps_bulk(ps_smem(dst2), src2, bytes2, FULL(b));
        };
        auto issue_qkv = [&](int l) {
            issue(PS_B_QKV, s_wqkv, reinterpret_cast<const __nv_bfloat16*>(a.layers[l].wqkv) + (size_t)2 * pp0 * D, (uint32_t)nq * D * 2,
                  a.layers[l].g_attn, s_gattn, (uint32_t)D * 4);
        };
        auto issue_o = [&](int l) {
            issue(PS_B_O, s_wo, reinterpret_cast<const __nv_bfloat16*>(a.layers[l].wo) + (size_t)d0 * D, (uint32_t)nx * D * 2, nullptr, nullptr, 0u);
        };
        auto issue_gu = [&](int l) {
            issue(PS_B_GU, s_wgu, reinterpret_cast<const __nv_bfloat16*>(a.layers[l].wgu) + (size_t)2 * u0 * D, (uint32_t)2 * nu * D * 2,
                  a.layers[l].g_ffn, s_gffn, (uint32_t)D * 4);
        };
        auto issue_d = [&](int l) {
            issue(PS_B_D, s_wd, reinterpret_cast<const __nv_bfloat16*>(a.layers[l].wd) + (size_t)d0 * F, (uint32_t)nx * F * 2, nullptr, nullptr, 0u);
        };
        auto issue_head = [&](int st) {
            const int rows = min(kPsHeadRows, n_head_rows - st * kPsHeadRows);
            issue(PS_B_HEAD + st % ns, head_slot(st % ns), a.emb_w + (size_t)(v0 + st * kPsHeadRows) * D, (uint32_t)rows * D * 2, nullptr, nullptr, 0u);
        };
        // bounded wait that also gives up when the block has aborted; false = stop issuing
        auto wait_free = [&](uint32_t bar, uint32_t parity) -> bool {
            unsigned long long t0 = 0;
            for (uint32_t i = 0;; ++i) {
                if (mbar_try_parity(bar, parity)) return true;
                if ((i & 63u) != 63u) continue;
                if (*s_abort) return false;
                const unsigned long long now = ps_now();
                if (t0 == 0) t0 = now;
                else if (now - t0 > c_wait_limit_ns) { *s_abort = 1; atomicExch(a.status, 82u); return false; }
            }
        };
        int full_uses[5] = {1, 1, 1, 1, 0};
        int head_issued = 0;
        // weights do not depend on the previous kernel: the first layer's slices and the first head stages are
        // requested before the dependency wait
        issue_qkv(0); issue_o(0); issue_gu(0); issue_d(0);
        for (; head_issued < min(n_pre, n_st); ++head_issued) issue_head(head_issued);
        pdl_launch_dependents();
        pdl_wait();
        bool go = *reinterpret_cast<volatile unsigned int*>(a.status) == 0u;
        const int pos = a.tok_pos[0], slot = a.tok_slot[0];
        const int n_pages = pos / kPage + 1;
        const int pps = max(2, ps_ceil_div(n_pages, a.s_max));
        const int S = ps_ceil_div(n_pages, pps);
        const bool attn_cta = cta < H * S;
        const int ah = attn_cta ? cta / S : 0, as = attn_cta ? cta % S : 0;
        const int p_lo = min(n_pages, as * pps), p_hi = attn_cta ? min(n_pages, p_lo + pps) : p_lo;
        const int my_pages = p_hi - p_lo;
        int pages[8];
        for (int p = 0; p < my_pages && p < 8; ++p) pages[p] = a.kv.block_table[(size_t)slot * a.kv.pages_per_seq + p_lo + p];
        auto issue_kv = [&](int l) {
            ps_expect(FULL(PS_B_KV), (uint32_t)(my_pages * 2 * page_elems * 2));
            for (int p = 0; p < my_pages; ++p) {
                ps_bulk(ps_smem(s_kv + (size_t)(2 * p) * page_elems), kv_ptr<__nv_bfloat16>(a.kv, m, l, pages[p], 0, ah, 0),
                        (uint32_t)(page_elems * 2), FULL(PS_B_KV));
                ps_bulk(ps_smem(s_kv + (size_t)(2 * p + 1) * page_elems), kv_ptr<__nv_bfloat16>(a.kv, m, l, pages[p], 1, ah, 0),
                        (uint32_t)(page_elems * 2), FULL(PS_B_KV));
            }
            full_uses[PS_B_KV] += 1;
        };
        if (go && my_pages > 0) issue_kv(0);
        for (int l = 1; l < NL && go; ++l) {               // refills, in the order in which the layer before frees the buffers
            const uint32_t par = (uint32_t)((l - 1) & 1);
            go = wait_free(FREE(PS_B_QKV), par);
            if (go) { issue_qkv(l); full_uses[PS_B_QKV] += 1; }
            if (go && my_pages > 0) { go = wait_free(FREE(PS_B_KV), par); if (go) issue_kv(l); }
            if (go) go = wait_free(FREE(PS_B_O), par);
            if (go) { issue_o(l); full_uses[PS_B_O] += 1; }
            if (go) go = wait_free(FREE(PS_B_GU), par);
            if (go) { issue_gu(l); full_uses[PS_B_GU] += 1; }
            if (go) go = wait_free(FREE(PS_B_D), par);
            if (go) { issue_d(l); full_uses[PS_B_D] += 1; }
        }
        if (go && n_st > head_issued) {
            // the rest of the head's stages go through the layers' buffers: all of them are free once the last layer is done
            const uint32_t par = (uint32_t)((NL - 1) & 1);
            go = wait_free(FREE(PS_B_QKV), par) && (my_pages == 0 || wait_free(FREE(PS_B_KV), par)) && wait_free(FREE(PS_B_O), par) &&
                 wait_free(FREE(PS_B_GU), par) && wait_free(FREE(PS_B_D), par);
            for (; go && head_issued < min(ns, n_st); ++head_issued) issue_head(head_issued);
            for (; go && head_issued < n_st; ++head_issued) {
                go = wait_free(FREE(PS_B_HEAD + head_issued % ns), (uint32_t)((head_issued / ns - 1) & 1));
                if (go) issue_head(head_issued); else break;
            }
        }
        // let every copy in flight land before the block's shared memory is given to another block
        for (int b = 0; b < 5; ++b)
            if (full_uses[b] > 0) mbar_wait_bounded(FULL(b), (uint32_t)((full_uses[b] - 1) & 1), c_wait_limit_ns);
        for (int st = max(0, head_issued - ns); st < head_issued; ++st)
            mbar_wait_bounded(FULL(PS_B_HEAD + st % ns), (uint32_t)((st / ns) & 1), c_wait_limit_ns);
        return;
    }

    // ============================================================================================================
    // The computing threads
    // ============================================================================================================
    int n_waited[5] = {0, 0, 0, 0, 0};
    // Every thread waits for the copy itself (a single probe once it has landed, which is the usual case: the copies
    // run a layer ahead).  A wait that runs out raises the abort flag; the block acts on it at its next barrier.
    auto wait_full = [&](int b, unsigned int code) {
        if (!mbar_wait_bounded(FULL(b), (uint32_t)(n_waited[b] & 1), c_wait_limit_ns)) { *s_abort = 1; atomicExch(a.status, code); }
        n_waited[b] += 1;
    };
    auto release = [&](int b) { if (tid == 0) ps_arrive(FREE(b)); };         // call after the barrier that ends the buffer's use

    for (int k = tid; k < D; k += kPsThreads) s_gfinal[k] = a.g_final[k];
    PS_TL(400);
    pdl_launch_dependents();
    pdl_wait();
    PS_TL(401);

    bool live = *reinterpret_cast<volatile unsigned int*>(a.status) == 0u;     // an earlier failure: do nothing
    const uint32_t epoch = *a.epoch;
    const int pos = a.tok_pos[0], slot = a.tok_slot[0];
    const uint32_t tok = a.tok_id[0];
    const int n_pages = pos / kPage + 1;
    for (int i = tid; i < HD / 2; i += kPsThreads) s_rope[i] = a.rope[(size_t)pos * (HD / 2) + i];
    if (tid == 0) s_pages[0] = a.kv.block_table[(size_t)slot * a.kv.pages_per_seq + pos / kPage];
    wait_full(PS_B_QKV, 71u);                    // the first layer's QKV slice and gain
    float ss = 0.f;                              // layer 0: the embedding row takes the place of the gathered x
    for (int k = tid; k < D; k += kPsThreads) {
        const float x = a.emb_f32[(size_t)tok * D + k];
        xraw[k] = x; xg[k] = x * s_gattn[k]; ss += x * x;
    }
    // attention role: head ah, key range as of S; ranges of pps consecutive pages
    const int pps = max(2, ps_ceil_div(n_pages, a.s_max));
    const int S = ps_ceil_div(n_pages, pps);
    const bool attn_cta = cta < H * S;
    const int ah = attn_cta ? cta / S : 0, as = attn_cta ? cta % S : 0;
    const int p_lo = min(n_pages, as * pps), p_hi = attn_cta ? min(n_pages, p_lo + pps) : p_lo;
    const int my_pages = p_hi - p_lo;
    float inv = ps_inv_rms(ss, s_red, D, m.eps);         // its barrier publishes s_pages, s_rope, xraw, xg
    const int page_new = s_pages[0];

    for (int l = 0; l < NL && live; ++l) {
        const uint32_t tg = epoch * 1024u + (uint32_t)l * 8u;
        // ---- x entering the layer (layer 0: done above), with the gain product and the sum of squares ------------
        if (l > 0) {
            wait_full(PS_B_QKV, 71u);
            ss = ll_gather<4>(a.xa, D, D, 0, tg + 0u, xraw, s_gattn, xg, s_abort, a.status, 70u);
            inv = ps_inv_rms(ss, s_red, D, m.eps);
            if (*s_abort) { live = false; break; }
        }
        PS_TL(412);
        // ---- this block's QKV row pairs: RoPE, K/V to the cache, all three to the consumers -----------------------
        for (int pi = warp; pi < pp1 - pp0; pi += kPsWarps) {
            float r0, r1;
            ps_dot2(s_wqkv + (size_t)(2 * pi) * D, s_wqkv + (size_t)(2 * pi + 1) * D, xg, D, r0, r1);
            r0 *= inv; r1 *= inv;
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
        ps_sync();                                         // every warp is done with s_wqkv, s_gattn
        release(PS_B_QKV);
        PS_TL(413);
        // ---- attention over this block's key range -------------------------------------------------------------------
        if (attn_cta) {
            if (my_pages > 0) wait_full(PS_B_KV, 73u);
            ll_gather<1>(a.qkv + (size_t)ah * HD, 3 * HD, HD, D, tg + 1u, s_qh, nullptr, nullptr, s_abort, a.status, 72u);   // q | k | v of the head
            ps_sync();
            if (*s_abort) { live = false; break; }
            PS_TL(414);
            float part = 0.f;                              // thread i < HD + 2: out[i] | max | sum of this key range
            if (my_pages > 0) {
                // Each warp takes a run of consecutive keys through scores, softmax weights and the value product on its
                // own (no block barrier inside); the 16 partial results are combined once at the end.
                const int kb = p_lo * kPage;
                const int nk = min(my_pages * kPage, pos + 1 - kb);            // keys of this range that exist
                const int chunk = ps_ceil_div(nk, kPsWarps);                   // <= 32 (at most 8 pages per range)
                const int j_lo = min(nk, warp * chunk), cnt = min(nk, j_lo + chunk) - j_lo;
                const int sub = lane % LPK, rsub = lane / LPK;
                float* wsc = s_sc + j_lo;                                      // this warp's scores, then weights
                float qf[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) qf[e] = s_qh[sub * 8 + e];
#pragma unroll 2
                for (int i0 = 0; i0 < cnt; i0 += KPI) {
                    const int i = i0 + rsub, j = j_lo + i;
                    float sc = 0.f;
                    if (i < cnt) {
                        if (kb + j == pos) {               // the new key: its cache row is being written right now
#pragma unroll
                            for (int e = 0; e < 8; ++e) sc += qf[e] * s_qh[HD + sub * 8 + e];
                        } else {
                            const __nv_bfloat16* kr = s_kv + (size_t)(2 * (j / kPage)) * page_elems + (size_t)(j % kPage) * HD + sub * 8;
                            float kf[8];
                            unpack16<__nv_bfloat16>(*reinterpret_cast<const uint4*>(kr), kf);
#pragma unroll
                            for (int e = 0; e < 8; ++e) sc += qf[e] * kf[e];
                        }
                    }
#pragma unroll
                    for (int o = LPK / 2; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
                    if (sub == 0 && i < cnt) wsc[i] = sc * m.scale;
                }
                __syncwarp();
                PS_TL(4141);
                const float sv = lane < cnt ? wsc[lane] : -INFINITY;
                const float mw = warp_max(sv);
                const float pw = lane < cnt ? __expf(sv - mw) : 0.f;
                const float lw = warp_sum(pw);
                if (lane < cnt) wsc[lane] = pw;
                __syncwarp();
                PS_TL(4142);
                constexpr int DL = HD >= 32 ? HD / 32 : 1;                     // value dims per lane
                const bool owns = lane * DL < HD;
                float ov[DL];
#pragma unroll
                for (int e = 0; e < DL; ++e) ov[e] = 0.f;
                const int i_new = pos - kb - j_lo;                             // the new key's place in this warp's run, if it is there
                if (owns) {
#pragma unroll 4
                    for (int i = 0; i < cnt; ++i) {
                        const int j = j_lo + i;
                        const float pj = i == i_new ? 0.f : wsc[i];            // its cache row is not final yet (it holds finite values)
                        const __nv_bfloat16* vr = s_kv + (size_t)(2 * (j / kPage) + 1) * page_elems + (size_t)(j % kPage) * HD + lane * DL;
                        if (DL == 1) ov[0] += pj * __bfloat162float(vr[0]);
                        else {
#pragma unroll
                            for (int e = 0; e < DL; e += 2) {
                                const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(vr + e);
                                ov[e] += pj * __low2float(vv); ov[e + 1] += pj * __high2float(vv);
                            }
                        }
                    }
                    if (i_new >= 0 && i_new < cnt) {
                        const float pj = wsc[i_new];
#pragma unroll
                        for (int e = 0; e < DL; ++e) ov[e] += pj * s_qh[2 * HD + lane * DL + e];
                    }
                }
                float* wp = s_redo + (size_t)warp * (HD + 2);                  // [warp][out | max | sum]
                if (owns) {
#pragma unroll
                    for (int e = 0; e < DL; ++e) wp[lane * DL + e] = ov[e];
                }
                if (lane == 0) { wp[HD] = cnt > 0 ? mw : -INFINITY; wp[HD + 1] = lw; }
                PS_TL(4143);
                ps_sync();
                PS_TL(4144);
                release(PS_B_KV);                          // s_kv is free: the next layer's pages may come
                if (tid < kPsWarps) {                      // weight of every warp's partial result
                    float mx = -INFINITY;
#pragma unroll
                    for (int w = 0; w < kPsWarps; ++w) mx = fmaxf(mx, s_redo[w * (HD + 2) + HD]);
                    const float mr = s_redo[tid * (HD + 2) + HD];
                    s_sc[tid] = mr == -INFINITY ? 0.f : __expf(mr - mx);
                    if (tid == 0) s_sc[kPsWarps] = mx;
                }
                ps_sync();
                if (tid == HD) part = s_sc[kPsWarps];
                else if (tid < HD + 2) {                   // combine the warps in warp order
                    const int col = tid < HD ? tid : HD + 1;
#pragma unroll
                    for (int w = 0; w < kPsWarps; ++w) part += s_sc[w] * s_redo[w * (HD + 2) + col];
                }
            } else if (tid == HD) {
                part = -INFINITY;                          // an empty range: ignored by the merge
            }
            if (tid < HD + 2) ll_st(a.ap + ((size_t)(ah * S + as) * (HD + 2) + tid), part, tg + 2u);
            PS_TL(416);
        }
        // ---- merge the key ranges of every head (in range order), out-projection rows, residual --------------------
        wait_full(PS_B_O, 75u);
        ll_gather<4>(a.ap, H * S * (HD + 2), H * S * (HD + 2), 0, tg + 2u, s_ap, nullptr, nullptr, s_abort, a.status, 74u);
        ps_sync();
        if (*s_abort) { live = false; break; }
        PS_TL(417);
        if (tid < H * S) {                                 // weight of every key range in its head's result: exp(max_r - max) / sum
            const int h = tid / S;
            const float* ph = s_ap + (size_t)h * S * (HD + 2);
            float mx = -INFINITY;
#pragma unroll 4
            for (int r = 0; r < S; ++r) mx = fmaxf(mx, ph[r * (HD + 2) + HD]);
            float den = 0.f;
#pragma unroll 4
            for (int r = 0; r < S; ++r) {
                const float mr = ph[r * (HD + 2) + HD];
                den += (mr == -INFINITY ? 0.f : __expf(mr - mx)) * ph[r * (HD + 2) + HD + 1];
            }
            const float mine = s_ap[(size_t)tid * (HD + 2) + HD];
            s_sc[tid] = mine == -INFINITY ? 0.f : __fdividef(__expf(mine - mx), den);
        }
        PS_TL(4171);
        ps_sync();
        PS_TL(4172);
        for (int t = tid; t < D; t += kPsThreads) {
            const int h = t / HD, d = t - h * HD;
            float acc = 0.f;
#pragma unroll 4
            for (int r = 0; r < S; ++r) acc += s_sc[h * S + r] * s_ap[(size_t)(h * S + r) * (HD + 2) + d];
            s_att[t] = acc;
        }
        PS_TL(4173);
        ps_sync();
        PS_TL(418);
        for (int r = warp; r < nx; r += kPsWarps) {
            const float y = ps_dot(s_wo + (size_t)r * D, s_att, D);
            if (lane == 0) ll_st(a.xb + d0 + r, xraw[d0 + r] + y, tg + 3u);
        }
        ps_sync();
        release(PS_B_O);
        PS_TL(419);
        // ---- x after the attention half with the FFN norm's gain product, this block's hidden units ----------------
        wait_full(PS_B_GU, 77u);
        ss = ll_gather<4>(a.xb, D, D, 0, tg + 3u, xraw, s_gffn, xg, s_abort, a.status, 76u);
        inv = ps_inv_rms(ss, s_red, D, m.eps);
        if (*s_abort) { live = false; break; }
        PS_TL(421);
        for (int u = warp; u < nu; u += kPsWarps) {
            float g, up;
            ps_dot2(s_wgu + (size_t)(2 * u) * D, s_wgu + (size_t)(2 * u + 1) * D, xg, D, g, up);
            if (lane == 0) {                               // silu(g) * up, src/nn/swiglu.cpp:37-57
                g *= inv; up *= inv;
                const float sig = 1.0f / (1.0f + expf(-g));
                ll_st(a.hb + u0 + u, (g * sig) * up, tg + 4u);
            }
        }
        ps_sync();
        release(PS_B_GU);
        PS_TL(422);
        // ---- all hidden units, down-projection rows, residual -----------------------------------------------------------
        wait_full(PS_B_D, 79u);
        ll_gather<4>(a.hb, F, F, 0, tg + 4u, s_hid, nullptr, nullptr, s_abort, a.status, 78u);
        ps_sync();
        if (*s_abort) { live = false; break; }
        PS_TL(424);
        for (int r = warp; r < nx; r += kPsWarps) {
            const float y = ps_dot(s_wd + (size_t)r * F, s_hid, F);
            if (lane == 0) {
                const float xnew = xraw[d0 + r] + y;
                ll_st(a.xa + d0 + r, xnew, tg + 8u);        // tag of the next layer's (or the head's) x
                if (l + 1 == NL && a.logits == nullptr) a.x_out[d0 + r] = xnew;
            }
        }
        ps_sync();
        release(PS_B_D);
        PS_TL(425);
    }

    // ---- final norm and the tied head: this block's vocabulary rows, streamed through shared memory --------------
    if (live && a.logits != nullptr) {
        ss = ll_gather<4>(a.xa, D, D, 0, epoch * 1024u + (uint32_t)NL * 8u, xraw, s_gfinal, xg, s_abort, a.status, 80u);
        inv = ps_inv_rms(ss, s_red, D, m.eps);
        PS_TL(430);
        for (int st = 0; st < n_st && *s_abort == 0; ++st) {
            const bool ok = mbar_wait_bounded(FULL(PS_B_HEAD + st % ns), (uint32_t)((st / ns) & 1), c_wait_limit_ns);
            if (!ok) { *s_abort = 1; atomicExch(a.status, 81u); }
            const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(head_slot(st % ns)) + (size_t)(2 * warp) * D;
            const int row = st * kPsHeadRows + 2 * warp;
            if (ok && row < n_head_rows) {
                float y0, y1;
                ps_dot2(w, row + 1 < n_head_rows ? w + D : w, xg, D, y0, y1);
                if (lane == 0) {
                    a.logits[v0 + row] = y0 * inv; s_logits[row] = y0 * inv;
                    if (row + 1 < n_head_rows) { a.logits[v0 + row + 1] = y1 * inv; s_logits[row + 1] = y1 * inv; }
                }
            }
            ps_sync();
            if (tid == 0) ps_arrive(FREE(PS_B_HEAD + st % ns));
        }
        PS_TL(431);
        // ---- the sampler's first two kernels, folded in (src/inference.cpp:104-131: penalty, maximum, weights) ----------
        if (a.fold_temperature >= 0.f && *s_abort == 0) {
            const float pen = a.fold_penalty;
            const uint32_t* seen = a.st.seen + (size_t)slot * (V / 32);
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int t = tid; t < n_head_rows; t += kPsThreads) {          // ascending ids per thread: a strict > keeps the first maximum
                const int i = v0 + t;
                float sv = s_logits[t];
                if (pen != 1.0f && ((seen[i >> 5] >> (i & 31)) & 1u)) sv = sv > 0.f ? sv / pen : sv * pen;
                s_logits[t] = sv;
                if (sv > bv) { bv = sv; bi = i; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) first_max(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
            int* s_redi = reinterpret_cast<int*>(s_red + 16);
            if (lane == 0) { s_red[warp] = bv; s_redi[warp] = bi; }
            ps_sync();
            const uint32_t tgm = epoch * 1024u + (uint32_t)NL * 8u + 1u;
            if (tid == 0) {
                for (int w = 1; w < kPsWarps; ++w) first_max(bv, bi, s_red[w], s_redi[w]);
                ll_st(a.mxb + 2 * cta, bv, tgm);
                ll_st(a.mxb + 2 * cta + 1, __int_as_float(bi), tgm);
                a.g_pmax_val[(size_t)slot * a.na + cta] = bv;               // what k_samp_pick reads: one part per block
                a.g_pmax_idx[(size_t)slot * a.na + cta] = bi;
            }
            ll_gather<1>(a.mxb, 2 * a.na, 2 * a.na, 0, tgm, s_ap, nullptr, nullptr, s_abort, a.status, 83u);
            ps_sync();
            float mx = -INFINITY; int arg = 0x7fffffff;                     // every warp finds the slot's maximum for itself
            for (int b = lane; b < a.na; b += 32) first_max(mx, arg, s_ap[2 * b], __float_as_int(s_ap[2 * b + 1]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) first_max(mx, arg, __shfl_xor_sync(0xffffffffu, mx, o), __shfl_xor_sync(0xffffffffu, arg, o));
            if (a.fold_temperature > 0.f && *s_abort == 0 && a.st.finished[slot] == 0 && isfinite(mx)) {
                float* w = a.g_w + (size_t)slot * V;
                unsigned long long* gm = a.g_mass + (size_t)slot * kL0Buckets;
                unsigned int* gc = a.g_cnt + (size_t)slot * kL0Buckets;
                for (int t = tid; t < n_head_rows; t += kPsThreads) {
                    const float e = expf((s_logits[t] - mx) / a.fold_temperature);
                    w[v0 + t] = e;
                    const int b = l0_bucket(__float_as_uint(e));
                    atomicAdd(gm + b, fix_of(e));                           // results unused: reductions performed in L2
                    atomicAdd(gc + b, 1u);
                }
            }
        }
    }
    PS_TL(432);
    if (cta == 0 && tid == 0) *a.epoch = epoch + 1u;
}

}  // namespace sllm
