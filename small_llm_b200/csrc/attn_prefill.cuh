// Causal attention for runs of consecutive query positions of one sequence (prefill): tiles of up to 64
// queries per block share every K/V page, which is staged into shared memory by bulk asynchronous copies
// (cp.async.bulk; per page and head K is one contiguous run and V another), two pages in flight.
// Replaces the reference's materialised scores / causal softmax / PV chain for T > 1
// (src/ops/attention.cpp:45-50,179-183, src/ops/softmax.cpp:24-40) with an online softmax per query row.
// A query tile reads each page once instead of once per query: 64x less KV traffic than the per-query kernels.
//
// grid (n_tiles, H), 256 threads.  Phase 1 per page: S = Q K^T (thread = 2 queries x 8 keys), scale, causal
// mask.  Phase 2: per-row running max / sum, P = exp(S - max) (4 threads per row).  Phase 3: O = O*corr + P V
// (thread = 2 queries x 8 dims).  All waits on mbarriers are bounded.
#pragma once
#include "attn_stream.cuh"
#include "common.cuh"

namespace sllm {

constexpr int kPfThreads = 256;
constexpr int kPfQ = 64;                 // queries per tile
constexpr int kPfStages = 2;

struct AttnPfArgs {
    const float* q;            // [n_tok][D]
    float* out;                // [n_tok][D]
    __nv_bfloat16* out_bf16;   // optional
    ModelDims m;
    KvView kv;
    const PfTile* tiles;
    int layer;
    unsigned int* status;
};

// n consecutive elements of a K or V row as floats, with the widest loads the type allows
template <int N> __device__ __forceinline__ void load_row(const __nv_bfloat16* p, float* f) {
    if (N % 8 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 8) unpack16<__nv_bfloat16>(*reinterpret_cast<const uint4*>(p + i), f + i);
    } else if (N % 4 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 4) {
            const uint2 v = *reinterpret_cast<const uint2*>(p + i);
            f[i] = __uint_as_float(v.x << 16); f[i + 1] = __uint_as_float(v.x & 0xffff0000u);
            f[i + 2] = __uint_as_float(v.y << 16); f[i + 3] = __uint_as_float(v.y & 0xffff0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p + i);
            f[i] = __low2float(v); f[i + 1] = __high2float(v);
        }
    }
}
template <int N> __device__ __forceinline__ void load_row(const float* p, float* f) {
    if (N % 4 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 4) { const float4 v = *reinterpret_cast<const float4*>(p + i); f[i] = v.x; f[i + 1] = v.y; f[i + 2] = v.z; f[i + 3] = v.w; }
    } else {
#pragma unroll
        for (int i = 0; i < N; i += 2) { const float2 v = *reinterpret_cast<const float2*>(p + i); f[i] = v.x; f[i + 1] = v.y; }
    }
}

template <typename KVT, int HD> constexpr size_t attn_prefill_smem() {
    return (size_t)kPfStages * 2 * kPage * HD * sizeof(KVT)      // K | V stages
           + (size_t)kPfQ * (HD + 4) * sizeof(float)              // Q, rows padded by 4 floats
           + (size_t)kPfQ * (kPage + 1) * sizeof(float);          // S / P, rows padded by 1
}

template <typename KVT, int HD>
__global__ void __launch_bounds__(kPfThreads) k_attn_prefill(const AttnPfArgs a) {
    constexpr uint32_t BLK = kPage * HD * sizeof(KVT);
    constexpr int QS = HD + 4, SS = kPage + 1;
    constexpr int DPT = HD / 8;                          // output dims per thread in phase 3 (8 warps)
    static_assert(HD % 8 == 0, "head_dim must be a multiple of 8");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* kvs = smem_raw;
    float* sQ = reinterpret_cast<float*>(smem_raw + (size_t)kPfStages * 2 * BLK);
    float* sS = sQ + kPfQ * QS;
    __shared__ __align__(8) unsigned long long bars[kPfStages];
    __shared__ float s_m[kPfQ], s_l[kPfQ], s_corr[kPfQ];
    __shared__ int s_ok;

    const PfTile t = a.tiles[blockIdx.x];
    const int head = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int D = a.m.D;

    if (tid == 0) {
        for (int s = 0; s < kPfStages; ++s) bar_init(as_smem(&bars[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_ok = 1;
    }
    pdl_launch_dependents();
    pdl_wait();

    const int n_pages = (t.pos0 + t.n_q - 1) / kPage + 1;
    const int* table = a.kv.block_table + (size_t)t.slot * a.kv.pages_per_seq;
    for (int i = tid; i < kPfQ * HD; i += kPfThreads) {
        const int qi = i / HD, d = i - qi * HD;
        sQ[qi * QS + d] = qi < t.n_q ? a.q[(size_t)(t.tok_begin + qi) * D + head * HD + d] : 0.f;
    }
    if (tid < kPfQ) { s_m[tid] = -INFINITY; s_l[tid] = 0.f; }
    __syncthreads();
    auto issue = [&](int pg) {
        const int s = pg % kPfStages;
        const int page = table[pg];
        const uint32_t bar = as_smem(&bars[s]);
        bar_expect(bar, 2 * BLK);
        bulk_g2s(as_smem(kvs + (size_t)s * 2 * BLK), kv_ptr<KVT>(a.kv, a.m, a.layer, page, 0, head, 0), BLK, bar);
        bulk_g2s(as_smem(kvs + (size_t)s * 2 * BLK + BLK), kv_ptr<KVT>(a.kv, a.m, a.layer, page, 1, head, 0), BLK, bar);
    };
    if (tid == 0)
        for (int pg = 0; pg < kPfStages && pg < n_pages; ++pg) issue(pg);

    float o[2][DPT];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int d = 0; d < DPT; ++d) o[i][d] = 0.f;

    for (int pg = 0; pg < n_pages; ++pg) {
        const int s = pg % kPfStages;
        if (!bar_wait(as_smem(&bars[s]), (pg / kPfStages) & 1)) { s_ok = 0; atomicExch(a.status, 22u); }
        __syncthreads();
        if (!s_ok) break;
        const KVT* Kp = reinterpret_cast<const KVT*>(kvs + (size_t)s * 2 * BLK);
        const KVT* Vp = reinterpret_cast<const KVT*>(kvs + (size_t)s * 2 * BLK + BLK);
        const int kb = pg * kPage;
        // ---- phase 1: scores; thread = queries {lane, lane+32} x keys {warp*8 .. warp*8+7} -------------
        {
            float acc[2][8];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
            for (int d = 0; d < HD; d += 4) {
                const float4 q0 = *reinterpret_cast<const float4*>(sQ + lane * QS + d);
                const float4 q1 = *reinterpret_cast<const float4*>(sQ + (lane + 32) * QS + d);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float kf[4];
                    load_row<4>(Kp + (size_t)(warp * 8 + j) * HD + d, kf);
                    acc[0][j] += q0.x * kf[0] + q0.y * kf[1] + q0.z * kf[2] + q0.w * kf[3];
                    acc[1][j] += q1.x * kf[0] + q1.y * kf[1] + q1.z * kf[2] + q1.w * kf[3];
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int qi = lane + 32 * i;
                const int qpos = t.pos0 + qi;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int kj = warp * 8 + j;
                    sS[qi * SS + kj] = (qi < t.n_q && kb + kj <= qpos) ? acc[i][j] * a.m.scale : -INFINITY;
                }
            }
        }
        __syncthreads();
        // ---- phase 2: online softmax; 4 threads per query row, 16 keys each --------------------------------
        {
            const int qi = tid >> 2, part = tid & 3;
            float* row = sS + qi * SS + part * 16;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 16; ++j) mx = fmaxf(mx, row[j]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_old = s_m[qi];
            const float m_new = fmaxf(m_old, mx);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float p = m_new == -INFINITY ? 0.f : expf(row[j] - m_new);
                row[j] = p;
                sum += p;
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            __syncwarp();
            if (part == 0) {
                const float corr = m_new == -INFINITY ? 1.f : expf(m_old - m_new);
                s_corr[qi] = corr;
                s_l[qi] = s_l[qi] * corr + sum;
                s_m[qi] = m_new;
            }
        }
        __syncthreads();
        // ---- phase 3: O = O * corr + P V; thread = queries {lane, lane+32} x dims {warp*DPT ..} -------------
        {
            const float c0 = s_corr[lane], c1 = s_corr[lane + 32];
#pragma unroll
            for (int d = 0; d < DPT; ++d) { o[0][d] *= c0; o[1][d] *= c1; }
            const int nk = min(kPage, t.pos0 + t.n_q - kb);          // keys beyond the last query are all masked
            for (int kj = 0; kj < nk; ++kj) {
                const float p0 = sS[lane * SS + kj], p1 = sS[(lane + 32) * SS + kj];
                float vf[DPT];
                load_row<DPT>(Vp + (size_t)kj * HD + warp * DPT, vf);
#pragma unroll
                for (int d = 0; d < DPT; ++d) {
                    o[0][d] += p0 * vf[d];
                    o[1][d] += p1 * vf[d];
                }
            }
        }
        __syncthreads();                                             // stage s and sS are free again
        if (tid == 0 && pg + kPfStages < n_pages) issue(pg + kPfStages);
    }
    if (!s_ok) {
        for (int i = 0; i < 32; ++i) __nanosleep(16384);
        return;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int qi = lane + 32 * i;
        if (qi >= t.n_q) continue;
        const float inv = 1.0f / s_l[qi];
        const size_t base = (size_t)(t.tok_begin + qi) * D + head * HD + warp * DPT;
#pragma unroll
        for (int d = 0; d < DPT; ++d) {
            const float r = o[i][d] * inv;
            a.out[base + d] = r;
            if (a.out_bf16) a.out_bf16[base + d] = __float2bfloat16_rn(r);
        }
    }
}

}  // namespace sllm
