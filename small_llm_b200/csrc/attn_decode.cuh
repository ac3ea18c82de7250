// Causal attention for one query position per (token, head) over the paged KV cache:
// split-K flash-decode.  Replaces, for the cached case, the reference's
// scores = Q K^T, * 1/sqrt(hd), causal softmax, P V chain (src/ops/attention.cpp:45-50,179-183,
// src/ops/softmax.cpp:24-40); there are as many KV heads as query heads (no GQA).
//
// grid = (n_splits, H, n_tok).  Split s of a query at position p covers keys
// [s*keys_per_split, min((s+1)*keys_per_split, p+1)).  Each block keeps a running (max, sum, out)
// over its keys; with more than one split the partial triples go to scratch memory and the block
// that finishes last for a (token, head) merges them in split order, so the result does not
// depend on which block that is.  No block ever waits for another.
#pragma once
#include "common.cuh"

namespace sllm {

struct AttnDecArgs {
    const float* q;        // [n_tok][D] rotated queries (fp32)
    float* out;            // [n_tok][D] merged heads
    __nv_bfloat16* out_bf16; // when set, the result is also stored as bf16 (operand of the tensor-core out-projection)
    ModelDims m;
    KvView kv;
    PassView pass;
    int layer;
    int n_splits;
    int keys_per_split;    // multiple of kPage
    // scratch for n_splits > 1
    float* part_o;         // [n_tok][H][n_splits][hd]
    float* part_ml;        // [n_tok][H][n_splits][2]
    unsigned int* ticket;  // [n_tok][H], zero between launches
    int prefer_stream;     // host side: take the page-streaming kernel although there are fewer pairs than SMs
};

constexpr int kAttnThreads = 128;

template <typename KVT, int HD>
__global__ void __launch_bounds__(kAttnThreads) k_attn_decode(const AttnDecArgs a) {
    constexpr int EPC = Elems<KVT>::per16;        // elements per 16-byte load
    constexpr int LPK = HD / EPC;                 // lanes per key in the score phase
    constexpr int KPI = 32 / LPK;                 // keys per warp iteration
    constexpr int WARPS = kAttnThreads / 32;
    constexpr int DP = HD / 2;                    // output pairs
    constexpr int KG = kAttnThreads / DP;         // key groups in the PV phase
    static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "head_dim must map to a power-of-two lane group");
    static_assert(kAttnThreads % DP == 0, "threads must tile the output pairs");

    __shared__ float sc[kPage];
    __shared__ float red_o[KG][HD];
    __shared__ float s_q[HD];
    __shared__ unsigned int s_last;

    const int split = blockIdx.x, head = blockIdx.y, tok = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    pdl_launch_dependents();        // successors may start fetching their weights now
    pdl_wait();

    const int pos = a.pass.tok_pos[tok];
    const int slot = a.pass.tok_slot[tok];
    const int k_begin = split * a.keys_per_split;
    const int k_end = min(k_begin + a.keys_per_split, pos + 1);
    const int D = a.m.D;

    if (tid < HD) s_q[tid] = a.q[(size_t)tok * D + head * HD + tid];
    __syncthreads();

    // this lane's slice of q for the score phase
    const int sub = lane % LPK;
    float qf[EPC];
#pragma unroll
    for (int e = 0; e < EPC; ++e) qf[e] = s_q[sub * EPC + e];

    const int dp = tid % DP, kg = tid / DP;
    float m_run = -INFINITY, l_run = 0.f, o0 = 0.f, o1 = 0.f;

    for (int kb = k_begin; kb < k_end; kb += kPage) {
        const int page = a.kv.block_table[(size_t)slot * a.kv.pages_per_seq + kb / kPage];
        const KVT* Kp = kv_ptr<KVT>(a.kv, a.m, a.layer, page, 0, head, 0);
        const KVT* Vp = kv_ptr<KVT>(a.kv, a.m, a.layer, page, 1, head, 0);
        const int nk = min(kPage, k_end - kb);

        // scores: LPK lanes share one key row
        for (int j = warp * KPI + lane / LPK; j < kPage; j += WARPS * KPI) {
            float s = 0.f;
            if (j < nk) {
                const uint4 v = *reinterpret_cast<const uint4*>(Kp + (size_t)j * HD + sub * EPC);
                float kf[EPC];
                unpack16<KVT>(v, kf);
#pragma unroll
                for (int e = 0; e < EPC; ++e) s += qf[e] * kf[e];
            }
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (sub == 0) sc[j] = (j < nk) ? s * a.m.scale : -INFINITY;
        }
        __syncthreads();

        // page maximum (every warp computes the same value)
        float pm = -INFINITY;
        for (int j = lane; j < kPage; j += 32) pm = fmaxf(pm, sc[j]);
        pm = warp_max(pm);
        const float m_new = fmaxf(m_run, pm);
        const float corr = expf(m_run - m_new);       // 0 on the first page (m_run = -inf)
        l_run *= corr; o0 *= corr; o1 *= corr;
        m_run = m_new;

        // P V: thread (kg, dp) takes keys kg, kg+KG, ... and output dims 2dp, 2dp+1
        for (int j = kg; j < nk; j += KG) {
            const float p = expf(sc[j] - m_new);
            float v0, v1;
            if (sizeof(KVT) == 2) {
                const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(Vp + (size_t)j * HD + 2 * dp);
                v0 = __low2float(vv); v1 = __high2float(vv);
            } else {
                const float2 vv = *reinterpret_cast<const float2*>(Vp + (size_t)j * HD + 2 * dp);
                v0 = vv.x; v1 = vv.y;
            }
            l_run += p;
            o0 += p * v0;
            o1 += p * v1;
        }
        __syncthreads();
    }

    // combine the KG key groups (l_run differs per group: each saw different keys)
    __shared__ float red_l[KG];
    red_o[kg][2 * dp] = o0;
    red_o[kg][2 * dp + 1] = o1;
    if (dp == 0) red_l[kg] = l_run;
    __syncthreads();
    float o = 0.f, l = 0.f;
    if (tid < HD) {
#pragma unroll
        for (int g = 0; g < KG; ++g) { o += red_o[g][tid]; l += red_l[g]; }
    }

    if (a.n_splits == 1) {
        if (tid < HD) {
            a.out[(size_t)tok * D + head * HD + tid] = o / l;
            if (a.out_bf16) a.out_bf16[(size_t)tok * D + head * HD + tid] = __float2bfloat16_rn(o / l);
        }
        return;
    }

    // ---- several splits: publish the partial, the last block merges ---------------------------
    const size_t pidx = ((size_t)tok * a.m.H + head) * a.n_splits + split;
    if (tid < HD) a.part_o[pidx * HD + tid] = o;
    if (tid == 0) { a.part_ml[pidx * 2] = m_run; a.part_ml[pidx * 2 + 1] = l; }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int done = atomicAdd(&a.ticket[(size_t)tok * a.m.H + head], 1u);
        s_last = (done == (unsigned int)a.n_splits - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const size_t base = ((size_t)tok * a.m.H + head) * a.n_splits;
    float mx = -INFINITY;
    for (int s = 0; s < a.n_splits; ++s) mx = fmaxf(mx, __ldcg(a.part_ml + (base + s) * 2));
    if (tid < HD) {
        float num = 0.f, den = 0.f;
        for (int s = 0; s < a.n_splits; ++s) {
            const float ms = __ldcg(a.part_ml + (base + s) * 2);
            if (ms == -INFINITY) continue;            // split had no keys
            const float w = expf(ms - mx);
            den += w * __ldcg(a.part_ml + (base + s) * 2 + 1);
            num += w * __ldcg(a.part_o + (base + s) * HD + tid);
        }
        a.out[(size_t)tok * D + head * HD + tid] = num / den;
        if (a.out_bf16) a.out_bf16[(size_t)tok * D + head * HD + tid] = __float2bfloat16_rn(num / den);
    }
    if (tid == 0) a.ticket[(size_t)tok * a.m.H + head] = 0;   // ready for the next launch
}

}  // namespace sllm
