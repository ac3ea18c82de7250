// Decode step for ONE new token: each transformer layer as two thread-block-cluster kernels.
//
// At batch 1 every projection is a latency problem, not a bandwidth problem: the weights of a
// layer (9.9 MB) stream in ~1.5 us, but a chain of kernels that each wait for the previous one's
// result costs several microseconds per link.  So the links are cut from five per layer to two,
// dependencies that stay inside one attention head or one slice of the FFN are resolved inside a
// cluster of 8 blocks through distributed shared memory, and every block fetches its weights into
// registers BEFORE it waits for its predecessor (griddepcontrol.wait).
//
//   k_attn_block  grid (8, H), cluster = the 8 blocks of a head.  x = x_in + sum(partials of the
//                 previous FFN), RMSNorm, this head's 3*hd rows of the QKV projection (hd/8 rows of
//                 each per block), RoPE, K/V appended to the paged cache and exchanged through DSMEM,
//                 attention over the cached keys with the pages dealt round-robin to the 8 blocks,
//                 partial (max, sum, out) exchanged through DSMEM and merged in rank order, then the
//                 head's share of the out-projection: partial[h][n] = sum_d att[d] * Wo[n][h*hd + d].
//   k_ffn_block   grid (nB), clusters of 8.  x = x_in + sum over heads of partial[h], RMSNorm, gate/up
//                 rows of this block's hidden units, SiLU(gate)*up, their share of the down-projection,
//                 summed over the cluster through DSMEM in rank order: partial[cluster][n].
// The residual stream is the sum "x + partials" in a fixed order, so results do not depend on timing.
// Same reference arithmetic as gemv.cuh / attn_decode.cuh (see the citations there).
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace sllm {
namespace cg = cooperative_groups;

constexpr int kFusedThreads = 384;
constexpr int kFusedWarps = kFusedThreads / 32;
constexpr int kCS = 8;                       // blocks per cluster

struct FusedArgs {
    ModelDims m;
    KvView kv;
    int layer;
    const uint32_t* tok_id;                  // the pass holds one token: index 0
    const int* tok_slot;
    const int* tok_pos;
    const float* x_in;                       // [D] residual before the partial sums
    const float* parts_in;                   // [n_parts_in][D]
    int n_parts_in;
    float* x_out;                            // [D] residual after the partial sums (written by one block)
    const float* gain;                       // [D]
    const void* w1;                          // attention: wqkv [3D][D];  FFN: wgu [2F][D]
    const void* w2;                          // attention: wo [D][D];     FFN: down weights as [F][D]
    float* parts_out;                        // attention: [H][D];        FFN: [gridDim.x / 8][D]
    const float2* rope;
    const float* emb;                        // layer 0: the token's row replaces x_in
    int upc;                                 // FFN: hidden units per block
};

// RMSNorm gains of the (up to two) elements a thread normalises; weights, so they can be fetched before the wait
struct GainPf { float g[2]; };
__device__ __forceinline__ GainPf gain_prefetch(const FusedArgs& a) {
    GainPf p;
    p.g[0] = threadIdx.x < a.m.D ? a.gain[threadIdx.x] : 0.f;
    p.g[1] = threadIdx.x + kFusedThreads < a.m.D ? a.gain[threadIdx.x + kFusedThreads] : 0.f;
    return p;
}

// x = x_in (+ partial sums), stored as the new residual by the designated block; xs = RMSNorm(x) * gain.
// The 1 + n_parts source vectors are split into up to 3 groups of threads, each thread requests its group's
// 16-byte pieces together (one round trip to L2 for up to 10 sources), the groups are combined in shared
// memory in a fixed order.  `scratch` holds 2 * D floats.  `after_issue` runs once the first batch of loads
// is in flight and before its data is needed: the place for other loads that should overlap with it.
template <typename F>
__device__ __forceinline__ void fused_prologue(const FusedArgs& a, float* xs, float* scratch, float* red, bool store,
                                               const GainPf& gp, F after_issue) {
    const int D = a.m.D, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* base = a.emb ? a.emb + (size_t)a.tok_id[0] * D : a.x_in;
    const int nch = D / 4;
    const int ng = max(1, min(3, kFusedThreads / nch));
    const int nsrc = 1 + a.n_parts_in, per = (nsrc + ng - 1) / ng;
    bool called = false;
    for (int item = tid; item < ng * nch || !called; item += kFusedThreads) {
        const bool live = item < ng * nch;
        const int g = live ? item / nch : 0, c = live ? item - g * nch : 0;
        const int s_end = live ? min(nsrc, (g + 1) * per) : 0;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = g * per; s0 < s_end || !called; s0 += 10) {
            float4 t[10];
#pragma unroll
            for (int i = 0; i < 10; ++i) {
                const int sidx = s0 + i;
                const float* src = sidx == 0 ? base : a.parts_in + (size_t)(sidx - 1) * D;
                t[i] = sidx < s_end ? __ldcg(reinterpret_cast<const float4*>(src) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (!called) { after_issue(); called = true; }
#pragma unroll
            for (int i = 0; i < 10; ++i) { acc.x += t[i].x; acc.y += t[i].y; acc.z += t[i].z; acc.w += t[i].w; }
        }
        if (live) *reinterpret_cast<float4*>((g == 0 ? xs : scratch + (size_t)(g - 1) * D) + c * 4) = acc;
    }
    __syncthreads();
    float ss = 0.f;
    for (int k = tid; k < D; k += kFusedThreads) {
        float v = xs[k];
        for (int g = 1; g < ng; ++g) v += scratch[(size_t)(g - 1) * D + k];
        xs[k] = v;
        ss += v * v;
        if (store) a.x_out[k] = v;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kFusedWarps; ++w) s += red[w];
    const float inv = 1.0f / sqrtf(s / (float)D + a.m.eps);
    for (int k = tid, j = 0; k < D; k += kFusedThreads, ++j) xs[k] = xs[k] * inv * (j < 2 ? gp.g[j] : a.gain[k]);
    __syncthreads();
}

// dot products of two adjacent weight rows with xs; PF chunks per lane come prefetched
template <typename WT, int PF>
__device__ __forceinline__ void pair_dot(const WT* w0p, const WT* w1p, const uint4* pf0, const uint4* pf1, bool prefetched,
                                         const float* xs, int K, float& r0, float& r1) {
    constexpr int EPC = Elems<WT>::per16;
    const int lane = threadIdx.x & 31, nchunk = K / EPC;
    const uint4* w0 = reinterpret_cast<const uint4*>(w0p);
    const uint4* w1 = reinterpret_cast<const uint4*>(w1p);
    float a0 = 0.f, a1 = 0.f;
    auto fma_chunk = [&](const uint4& v0, const uint4& v1, int c) {
        float f0[EPC], f1[EPC];
        unpack16<WT>(v0, f0);
        unpack16<WT>(v1, f1);
#pragma unroll
        for (int e = 0; e < EPC; e += 4) {
            const float4 x4 = *reinterpret_cast<const float4*>(xs + c * EPC + e);
            a0 += f0[e] * x4.x + f0[e + 1] * x4.y + f0[e + 2] * x4.z + f0[e + 3] * x4.w;
            a1 += f1[e] * x4.x + f1[e + 1] * x4.y + f1[e + 2] * x4.z + f1[e + 3] * x4.w;
        }
    };
    int c_begin = lane;
    if (prefetched) {
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            const int c = lane + 32 * i;
            if (c < nchunk) fma_chunk(pf0[i], pf1[i], c);
        }
        c_begin = lane + 32 * PF;
    }
#pragma unroll 2
    for (int c = c_begin; c < nchunk; c += 32) fma_chunk(ldg_stream(w0 + c), ldg_stream(w1 + c), c);
    r0 = warp_sum(a0);
    r1 = warp_sum(a1);
}

template <typename WT, int HD, int PF>
__global__ void __launch_bounds__(kFusedThreads, 2) k_attn_block(const FusedArgs a) {
    constexpr int EPC = Elems<WT>::per16;
    constexpr int RP = HD / kCS;                 // rows of q (and of k, of v) per block
    constexpr int NP = 3 * RP / 2;               // row pairs per block
    constexpr int LPK = HD / EPC;                // lanes per key row / per Wo row slice
    constexpr int KPI = 32 / LPK;
    constexpr int DP = HD / 2;
    constexpr int KG = kFusedThreads / DP;
    static_assert(RP >= 2 && RP % 2 == 0, "head_dim must give each block whole RoPE pairs");
    static_assert(kFusedThreads % DP == 0 && LPK <= 32, "unsupported head_dim");

    extern __shared__ __align__(16) float xs[];          // [D] + 2 * D of prologue scratch
    __shared__ float red[kFusedWarps];
    __shared__ float s_q[HD], s_k[HD], s_v[HD];          // filled by all 8 blocks of the head
    __shared__ float s_part[kCS][HD + 2];                // (out[HD], max, sum) of every block
    __shared__ float s_att[HD];
    __shared__ float sc[kPage];
    __shared__ float red_o[KG][HD];
    __shared__ float red_l[KG];

    cg::cluster_group cluster = cg::this_cluster();
    const int c = (int)cluster.block_rank();
    const int head = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int D = a.m.D;
    const WT* W1 = reinterpret_cast<const WT*>(a.w1);
    const WT* W2 = reinterpret_cast<const WT*>(a.w2);

    // ---- before the dependency wait: weights into registers ------------------------------------------
    SLLM_TL(100);
    pdl_launch_dependents();
    auto pair_row = [&](int pi) {                 // first of the two wqkv rows of pair pi
        const int which = pi / (RP / 2), lp = pi - which * (RP / 2);
        return which * D + head * HD + c * RP + 2 * lp;
    };
    uint4 pf0[PF], pf1[PF];
    if (warp < NP) {
        const uint4* w0 = reinterpret_cast<const uint4*>(W1 + (size_t)pair_row(warp) * D);
        const uint4* w1 = reinterpret_cast<const uint4*>(W1 + (size_t)(pair_row(warp) + 1) * D);
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            const int ch = lane + 32 * i;
            if (ch < D / EPC) { pf0[i] = ldg_stream(w0 + ch); pf1[i] = ldg_stream(w1 + ch); }
        }
    }
    // out-projection slice: rows n0..n0+NR, columns head*HD..+HD; LPK lanes per row
    const int NR = D / kCS, n0 = c * NR;
    const int sub = lane % LPK, rsub = lane / LPK;
    uint4 wo_pf[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int n = (warp + kFusedWarps * i) * KPI + rsub;
        if (n < NR) wo_pf[i] = ldg_stream(reinterpret_cast<const uint4*>(W2 + (size_t)(n0 + n) * D + head * HD) + sub);
    }
    const GainPf gp = gain_prefetch(a);
    cluster.sync();                            // every block of the head is running: its shared memory may be written
    SLLM_TL(101);
    pdl_wait();
    SLLM_TL(102);

    // ---- residual, norm, this block's rows of q, k, v ----------------------------------------------------
    // position and slot are requested together with the residual; what depends on them (RoPE factors, the
    // page of the new key, this block's first page) is requested as soon as they arrive, while the norm runs
    const int pos = a.tok_pos[0], slot = a.tok_slot[0];
    float2 cs_first = make_float2(1.f, 0.f);
    int n_pages = 1, page_new = 0, page_first = 0;
    fused_prologue(a, xs, xs + D, red, c == 0 && head == 0, gp, [&]() {
        if (warp < NP && warp / (RP / 2) < 2)
            cs_first = a.rope[(size_t)pos * (HD / 2) + ((c * RP + 2 * (warp % (RP / 2))) >> 1)];
        n_pages = pos / kPage + 1;
        page_new = a.kv.block_table[(size_t)slot * a.kv.pages_per_seq + pos / kPage];
        page_first = a.kv.block_table[(size_t)slot * a.kv.pages_per_seq + min(c, n_pages - 1)];
    });
    SLLM_TL(103);
    for (int pi = warp; pi < NP; pi += kFusedWarps) {
        const int row = pair_row(pi);
        float v0, v1;
        pair_dot<WT, PF>(W1 + (size_t)row * D, W1 + (size_t)(row + 1) * D, pf0, pf1, pi == warp, xs, D, v0, v1);
        const int which = pi / (RP / 2), d0 = c * RP + 2 * (pi - which * (RP / 2));
        float o0 = v0, o1 = v1;
        if (which < 2) {                       // interleaved-pair rotation, src/ops/rope.cpp:60-76
            const float2 cs = pi == warp ? cs_first : a.rope[(size_t)pos * (HD / 2) + (d0 >> 1)];
            o0 = v0 * cs.x - v1 * cs.y;
            o1 = v0 * cs.y + v1 * cs.x;
        }
        float* dst_local = which == 0 ? s_q : (which == 1 ? s_k : s_v);
        if (which > 0) {                       // the cache holds the rounded value; attention must see the same
            const WT r0 = from_float<WT>(o0), r1 = from_float<WT>(o1);
            o0 = to_float(r0); o1 = to_float(r1);
            if (lane == 0) {
                WT* dst = kv_ptr<WT>(a.kv, a.m, a.layer, page_new, which - 1, head, pos % kPage) + d0;
                dst[0] = r0; dst[1] = r1;
            }
        }
        if (lane < kCS) {                      // lane r hands the pair to block r of the cluster
            float* remote = cluster.map_shared_rank(dst_local, lane);
            remote[d0] = o0; remote[d0 + 1] = o1;
        }
    }
    // this block's first page of keys and values: requested before the exchange, used after it
    constexpr int KIT = (kPage + kFusedWarps * KPI - 1) / (kFusedWarps * KPI);
    constexpr int VIT = (kPage + KG - 1) / KG;
    const int dp = tid % DP, kg = tid / DP;
    uint4 k_pf[KIT];
    float v_pf0[VIT], v_pf1[VIT];
    auto load_v = [&](const WT* Vp, int j, float& v0, float& v1) {
        if (sizeof(WT) == 2) {
            const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(Vp + (size_t)j * HD + 2 * dp);
            v0 = __low2float(vv); v1 = __high2float(vv);
        } else {
            const float2 vv = *reinterpret_cast<const float2*>(Vp + (size_t)j * HD + 2 * dp);
            v0 = vv.x; v1 = vv.y;
        }
    };
    if (c < n_pages) {
        const WT* Kp = kv_ptr<WT>(a.kv, a.m, a.layer, page_first, 0, head, 0);
        const WT* Vp = kv_ptr<WT>(a.kv, a.m, a.layer, page_first, 1, head, 0);
        const int nk = min(kPage, pos + 1 - c * kPage);
#pragma unroll
        for (int i = 0; i < KIT; ++i) {
            const int j = warp * KPI + rsub + i * kFusedWarps * KPI;
            if (j < nk && c * kPage + j != pos) k_pf[i] = *reinterpret_cast<const uint4*>(Kp + (size_t)j * HD + sub * EPC);
        }
#pragma unroll
        for (int i = 0; i < VIT; ++i) {
            const int j = kg + KG * i;
            if (j < nk && c * kPage + j != pos) load_v(Vp, j, v_pf0[i], v_pf1[i]);
        }
    }
    SLLM_TL(104);
    cluster.sync();
    SLLM_TL(105);

    // ---- attention over this block's pages (round-robin over the cluster) ---------------------------------
    float qf[EPC];
#pragma unroll
    for (int e = 0; e < EPC; ++e) qf[e] = s_q[sub * EPC + e];
    float m_run = -INFINITY, l_run = 0.f, o0 = 0.f, o1 = 0.f;
    for (int pg = c; pg < n_pages; pg += kCS) {
        const int kb = pg * kPage;
        const bool first = pg == c;
        const int page = first ? page_first : a.kv.block_table[(size_t)slot * a.kv.pages_per_seq + pg];
        const WT* Kp = kv_ptr<WT>(a.kv, a.m, a.layer, page, 0, head, 0);
        const WT* Vp = kv_ptr<WT>(a.kv, a.m, a.layer, page, 1, head, 0);
        const int nk = min(kPage, pos + 1 - kb);
#pragma unroll
        for (int i = 0; i < KIT; ++i) {
            const int j = warp * KPI + rsub + i * kFusedWarps * KPI;
            if (j - rsub >= kPage) break;      // warp-uniform
            float s = 0.f;
            if (j < nk) {
                if (kb + j == pos) {           // the new key lives in shared memory (its cache row is being written)
#pragma unroll
                    for (int e = 0; e < EPC; ++e) s += qf[e] * s_k[sub * EPC + e];
                } else {
                    const uint4 v = first ? k_pf[i] : *reinterpret_cast<const uint4*>(Kp + (size_t)j * HD + sub * EPC);
                    float kf[EPC];
                    unpack16<WT>(v, kf);
#pragma unroll
                    for (int e = 0; e < EPC; ++e) s += qf[e] * kf[e];
                }
            }
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (sub == 0) sc[j] = (j < nk) ? s * a.m.scale : -INFINITY;
        }
        __syncthreads();
        float pm = -INFINITY;
        for (int j = lane; j < kPage; j += 32) pm = fmaxf(pm, sc[j]);
        pm = warp_max(pm);
        const float m_new = fmaxf(m_run, pm);
        const float corr = expf(m_run - m_new);
        l_run *= corr; o0 *= corr; o1 *= corr;
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < VIT; ++i) {
            const int j = kg + KG * i;
            if (j >= nk) break;
            const float p = expf(sc[j] - m_new);
            float v0, v1;
            if (kb + j == pos) { v0 = s_v[2 * dp]; v1 = s_v[2 * dp + 1]; }
            else if (first) { v0 = v_pf0[i]; v1 = v_pf1[i]; }
            else load_v(Vp, j, v0, v1);
            l_run += p; o0 += p * v0; o1 += p * v1;
        }
        __syncthreads();
    }
    red_o[kg][2 * dp] = o0;
    red_o[kg][2 * dp + 1] = o1;
    if (dp == 0) red_l[kg] = l_run;
    __syncthreads();
    if (tid < HD + 2) {                        // hand (out, max, sum) to every block of the head
        float val;
        if (tid < HD) { val = 0.f; for (int g = 0; g < KG; ++g) val += red_o[g][tid]; }
        else if (tid == HD) val = m_run;
        else { val = 0.f; for (int g = 0; g < KG; ++g) val += red_l[g]; }
        for (int r = 0; r < kCS; ++r) cluster.map_shared_rank(&s_part[0][0], r)[c * (HD + 2) + tid] = val;
    }
    SLLM_TL(106);
    cluster.sync();
    SLLM_TL(107);
    if (tid < HD) {                            // merge in rank order
        float mx = -INFINITY;
        for (int r = 0; r < kCS; ++r) mx = fmaxf(mx, s_part[r][HD]);
        float num = 0.f, den = 0.f;
        for (int r = 0; r < kCS; ++r) {
            const float mr = s_part[r][HD];
            if (mr == -INFINITY) continue;
            const float w = expf(mr - mx);
            den += w * s_part[r][HD + 1];
            num += w * s_part[r][tid];
        }
        s_att[tid] = num / den;
    }
    __syncthreads();

    // ---- this head's share of the out-projection, rows n0..n0+NR -------------------------------------------
    float af[EPC];
#pragma unroll
    for (int e = 0; e < EPC; ++e) af[e] = s_att[sub * EPC + e];
    auto out_row = [&](const uint4& v, int n) {
        float s = 0.f;
        if (n < NR) {
            float wf[EPC];
            unpack16<WT>(v, wf);
#pragma unroll
            for (int e = 0; e < EPC; ++e) s += af[e] * wf[e];
        }
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (sub == 0 && n < NR) a.parts_out[(size_t)head * D + n0 + n] = s;
    };
    const int nbase = warp * KPI;                       // warp-uniform loop bounds: the shuffles need whole warps
#pragma unroll
    for (int i = 0; i < 2; ++i)
        if (nbase + kFusedWarps * KPI * i < NR) out_row(wo_pf[i], nbase + kFusedWarps * KPI * i + rsub);
    for (int nb = nbase + 2 * kFusedWarps * KPI; nb < NR; nb += kFusedWarps * KPI) {
        const int n = nb + rsub;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (n < NR) v = ldg_stream(reinterpret_cast<const uint4*>(W2 + (size_t)(n0 + n) * D + head * HD) + sub);
        out_row(v, n);
    }
    SLLM_TL(108);
}

template <typename WT, int PF>
__global__ void __launch_bounds__(kFusedThreads, 2) k_ffn_block(const FusedArgs a) {
    constexpr int EPC = Elems<WT>::per16;
    constexpr int DPF = 3;                       // prefetched down-projection chunks per thread
    extern __shared__ __align__(16) float smem[];
    const int D = a.m.D, F = a.m.F;
    float* xs = smem;                            // [D]
    float* s_y = xs + D;                         // [G][D], then [D] in place of group 0
    __shared__ float red[kFusedWarps];
    __shared__ float s_hid[64];

    cg::cluster_group cluster = cg::this_cluster();
    const int c = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const WT* W1 = reinterpret_cast<const WT*>(a.w1);
    const WT* W2 = reinterpret_cast<const WT*>(a.w2);
    const int upc = a.upc;
    const int j0 = blockIdx.x * upc;
    const int nu = max(0, min(upc, F - j0));     // hidden units of this block
    const int NCH = D / EPC;                     // 16-byte chunks of a down-projection row
    const int G = kFusedThreads / NCH;           // unit groups in the down phase (>= 1 by launch condition)
    const int ch = tid % NCH, ug = tid / NCH;

    SLLM_TL(200);
    pdl_launch_dependents();
    uint4 pf0[PF], pf1[PF];
    if (warp < nu) {
        const uint4* w0 = reinterpret_cast<const uint4*>(W1 + (size_t)(2 * (j0 + warp)) * D);
        const uint4* w1 = reinterpret_cast<const uint4*>(W1 + (size_t)(2 * (j0 + warp) + 1) * D);
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            const int cc = lane + 32 * i;
            if (cc < NCH) { pf0[i] = ldg_stream(w0 + cc); pf1[i] = ldg_stream(w1 + cc); }
        }
    }
    uint4 dpf[DPF];
#pragma unroll
    for (int i = 0; i < DPF; ++i) {
        const int u = ug + G * i;
        if (ug < G && u < nu) dpf[i] = ldg_stream(reinterpret_cast<const uint4*>(W2 + (size_t)(j0 + u) * D) + ch);
    }
    const GainPf gp = gain_prefetch(a);
    cluster.sync();                              // all 8 blocks are running: their shared memory may be written later
    SLLM_TL(201);
    pdl_wait();
    SLLM_TL(202);

    fused_prologue(a, xs, s_y, red, blockIdx.x == 0, gp, []() {});
    SLLM_TL(203);
    // gate / up rows of this block's hidden units: silu(g) * u, src/nn/swiglu.cpp:37-57
    for (int u = warp; u < nu; u += kFusedWarps) {
        float g, up;
        pair_dot<WT, PF>(W1 + (size_t)(2 * (j0 + u)) * D, W1 + (size_t)(2 * (j0 + u) + 1) * D, pf0, pf1, u == warp, xs, D, g, up);
        if (lane == 0) {
            const float sig = 1.0f / (1.0f + expf(-g));
            s_hid[u] = (g * sig) * up;
        }
    }
    __syncthreads();
    SLLM_TL(204);
    // share of the down-projection: y[n] = sum_u hid[u] * Wd[j0+u][n]
    if (ug < G) {
        float acc[EPC];
#pragma unroll
        for (int e = 0; e < EPC; ++e) acc[e] = 0.f;
        auto down_row = [&](const uint4& v, int u) {
            float wf[EPC];
            unpack16<WT>(v, wf);
            const float h = s_hid[u];
#pragma unroll
            for (int e = 0; e < EPC; ++e) acc[e] += h * wf[e];
        };
#pragma unroll
        for (int i = 0; i < DPF; ++i)
            if (ug + G * i < nu) down_row(dpf[i], ug + G * i);
        for (int u = ug + G * DPF; u < nu; u += G)
            down_row(ldg_stream(reinterpret_cast<const uint4*>(W2 + (size_t)(j0 + u) * D) + ch), u);
#pragma unroll
        for (int e = 0; e < EPC; ++e) s_y[(size_t)ug * D + ch * EPC + e] = acc[e];
    }
    __syncthreads();
    // every block hands each column to the block of its cluster that owns it (columns [r*D/8, (r+1)*D/8) belong
    // to rank r), one barrier, then the owner adds the 8 contributions from its own shared memory in rank order
    const int NR = D / kCS;
    float* rx = s_y + (size_t)max(G, 2) * D;     // [kCS][NR], written by the peers
    for (int n = tid; n < D; n += kFusedThreads) {
        float v = s_y[n];
        for (int g = 1; g < G; ++g) v += s_y[(size_t)g * D + n];
        const int owner = n / NR;
        cluster.map_shared_rank(rx, owner)[c * NR + (n - owner * NR)] = v;
    }
    SLLM_TL(205);
    cluster.sync();
    SLLM_TL(206);
    for (int n = tid; n < NR; n += kFusedThreads) {
        float v = 0.f;
#pragma unroll
        for (int r = 0; r < kCS; ++r) v += rx[r * NR + n];
        a.parts_out[(size_t)(blockIdx.x / kCS) * D + c * NR + n] = v;
    }
    SLLM_TL(208);
}

// Final RMSNorm of the single-token path, once: xn = RMSNorm(base + sum of partials) * gain.  The head kernel
// then starts from 2.5 KB instead of every one of its blocks re-reading 19 vectors.
__global__ void __launch_bounds__(kFusedThreads) k_final_norm(const float* __restrict__ base, const float* __restrict__ parts,
                                                              int n_parts, int D, const float* __restrict__ gain, float eps,
                                                              float* __restrict__ xn) {
    extern __shared__ __align__(16) float fx[];          // [3 * D]
    __shared__ float red[kFusedWarps];
    FusedArgs a{};
    a.m.D = D; a.m.eps = eps; a.x_in = base; a.parts_in = parts; a.n_parts_in = n_parts; a.gain = gain;
    pdl_launch_dependents();
    const GainPf gp = gain_prefetch(a);
    pdl_wait();
    fused_prologue(a, fx, fx + D, red, false, gp, []() {});
    for (int k = threadIdx.x; k < D; k += kFusedThreads) xn[k] = fx[k];
}

// x[k] = base[k] + sum of partials, for callers that want the finished residual stream in one buffer
__global__ void __launch_bounds__(256) k_sum_parts(const float* __restrict__ base, const float* __restrict__ parts, int n_parts,
                                                   int D, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < D; k += gridDim.x * blockDim.x) {
        float v = base[k];
        for (int p0 = 0; p0 < n_parts; p0 += 16) {
            float t[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) t[i] = (p0 + i < n_parts) ? __ldcg(parts + (size_t)(p0 + i) * D + k) : 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) v += t[i];
        }
        out[k] = v;
    }
}

}  // namespace sllm
