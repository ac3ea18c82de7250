// Causal attention for one query position per (token, head) when there are many (token, head) pairs
// (decode at large batch, prefill chunks): one block per pair streams that head's K and V pages through
// shared memory with bulk asynchronous copies (cp.async.bulk, the 1-D form of TMA: each page holds the
// head's 64 keys as one contiguous run, and its 64 values as another), three pages in flight per warp quarter,
// completion signalled on mbarriers.  The arithmetic is that of attn_decode.cuh (online softmax over pages;
// reference: src/ops/attention.cpp:45-50,179-183, src/ops/softmax.cpp:24-40); only the data movement differs:
// the kernel is bound by HBM bandwidth (2 * head_dim * bytes per cached position and head), and bulk copies
// keep ~32 KB per block in flight without spending registers or issue slots on it.
// Every mbarrier wait is bounded; on expiry the block raises the engine's status word and returns.
#pragma once
#include "attn_decode.cuh"
#include "common.cuh"

namespace sllm {

constexpr int kStreamThreads = 128;
constexpr int kStreamStages = 3;         // pages in flight per warp (6 measured slower at 32..64 sequences: fewer blocks fit an SM)

__device__ __forceinline__ uint32_t as_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// false = gave up (the engine's wait limit, see common.cuh)
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) { return mbar_wait_bounded(bar, parity, c_wait_limit_ns); }
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// DL consecutive elements of a V row as floats
template <int DL> __device__ __forceinline__ void load_vals(const __nv_bfloat16* p, float* f) {
    if (DL == 1) f[0] = __bfloat162float(*p);
    else if (DL == 2) { const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p); f[0] = __low2float(v); f[1] = __high2float(v); }
    else {
#pragma unroll
        for (int i = 0; i < DL; i += 4) {
            const uint2 v = *reinterpret_cast<const uint2*>(p + i);
            f[i] = __uint_as_float(v.x << 16); f[i + 1] = __uint_as_float(v.x & 0xffff0000u);
            f[i + 2] = __uint_as_float(v.y << 16); f[i + 3] = __uint_as_float(v.y & 0xffff0000u);
        }
    }
}
template <int DL> __device__ __forceinline__ void load_vals(const float* p, float* f) {
    if (DL == 1) f[0] = *p;
    else if (DL == 2) { const float2 v = *reinterpret_cast<const float2*>(p); f[0] = v.x; f[1] = v.y; }
    else {
#pragma unroll
        for (int i = 0; i < DL; i += 4) { const float4 v = *reinterpret_cast<const float4*>(p + i); f[i] = v.x; f[i + 1] = v.y; f[i + 2] = v.z; f[i + 3] = v.w; }
    }
}

// Each of the four warps owns a quarter of every page (16 consecutive keys and their values) and runs its own
// copy pipeline over it: own stages, own mbarriers, own running softmax state.  The main loop therefore has no
// block-wide barrier; the four states are merged once at the end.
template <typename KVT, int HD, int ST>
__global__ void __launch_bounds__(kStreamThreads) k_attn_stream(const AttnDecArgs a, unsigned int* status) {
    constexpr int EPC = Elems<KVT>::per16;
    constexpr int LPK = HD / EPC;                 // lanes per key in the score phase
    constexpr int KPI = 32 / LPK;                 // keys per warp pass
    constexpr int WARPS = kStreamThreads / 32;
    constexpr int KW = kPage / WARPS;             // keys of a page owned by one warp
    constexpr int PASSES = KW / KPI;
    constexpr int DL = HD >= 32 ? HD / 32 : 1;    // output dims per lane in the value phase
    constexpr int LPV = HD / DL;                  // lanes per key in the value phase
    constexpr int KGW = 32 / LPV;                 // keys handled side by side in the value phase
    constexpr uint32_t WBLK = KW * HD * sizeof(KVT);             // one warp's K (or V) rows of one page
    constexpr int kTableCache = 128;
    static_assert(LPK >= 2 && LPK <= 32 && KW % KPI == 0 && KPI % KGW == 0, "unsupported head_dim");

    extern __shared__ __align__(128) unsigned char smem_raw[];   // [warp][stage][K rows | V rows]
    __shared__ __align__(8) unsigned long long bars[WARPS][ST];
    __shared__ float red_o[WARPS][HD];
    __shared__ float red_m[WARPS], red_l[WARPS];
    __shared__ float s_q[HD];
    __shared__ int s_table[kTableCache];
    __shared__ int s_ok;
    __shared__ unsigned int s_last;

    const int split = blockIdx.x, head = blockIdx.y;
    const int tok = a.pass.order ? a.pass.order[blockIdx.z] : (int)blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (tid == 0) {
        for (int w = 0; w < WARPS; ++w)
            for (int s = 0; s < ST; ++s) bar_init(as_smem(&bars[w][s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_ok = 1;
    }
    SLLM_TL(600);
    pdl_launch_dependents();
    pdl_wait();
    SLLM_TL(601);

    const int pos = a.pass.tok_pos[tok];
    const int slot = a.pass.tok_slot[tok];
    const int D = a.m.D;
    const int all_pages = pos / kPage + 1;
    // with several splits each block takes an equal share of the pages this query actually has
    const int per_split = (all_pages + a.n_splits - 1) / a.n_splits;
    const int pg0 = split * per_split;
    const int n_pages = max(0, min(all_pages, pg0 + per_split) - pg0);
    const int* table = a.kv.block_table + (size_t)slot * a.kv.pages_per_seq + pg0;
    if (tid < HD) s_q[tid] = a.q[(size_t)tok * D + head * HD + tid];
    for (int i = tid; i < n_pages && i < kTableCache; i += kStreamThreads) s_table[i] = table[i];
    __syncthreads();

    const int wk0 = warp * KW;                                    // this warp's first key inside a page
    // the last page may hold fewer keys than this warp's offset: then the warp has one page less
    const int last_nk = n_pages > 0 ? min(kPage, pos + 1 - (pg0 + n_pages - 1) * kPage) : 0;
    const int my_pages = n_pages - ((n_pages > 0 && last_nk <= wk0) ? 1 : 0);
    unsigned char* my_smem = smem_raw + (size_t)warp * ST * 2 * WBLK;
    auto issue = [&](int pg) {                    // one lane: this warp's K and V rows of page pg into stage pg % stages
        const int s = pg % ST;
        const int page = pg < kTableCache ? s_table[pg] : table[pg];
        const uint32_t bar = as_smem(&bars[warp][s]);
        bar_expect(bar, 2 * WBLK);
        bulk_g2s(as_smem(my_smem + (size_t)s * 2 * WBLK), kv_ptr<KVT>(a.kv, a.m, a.layer, page, 0, head, wk0), WBLK, bar);
        bulk_g2s(as_smem(my_smem + (size_t)s * 2 * WBLK + WBLK), kv_ptr<KVT>(a.kv, a.m, a.layer, page, 1, head, wk0), WBLK, bar);
    };
    if (lane == 0)
        for (int pg = 0; pg < ST && pg < my_pages; ++pg) issue(pg);

    const int sub = lane % LPK, grp = lane / LPK;
    float qf[EPC];
#pragma unroll
    for (int e = 0; e < EPC; ++e) qf[e] = s_q[sub * EPC + e];
    const int dv = (lane % LPV) * DL, kgw = lane / LPV;
    float m_run = -INFINITY, l_run = 0.f, o[DL];
#pragma unroll
    for (int d = 0; d < DL; ++d) o[d] = 0.f;

    bool ok = true;
    for (int pg = 0; pg < my_pages; ++pg) {
        const int s = pg % ST;
        ok = bar_wait(as_smem(&bars[warp][s]), (pg / ST) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const KVT* Kp = reinterpret_cast<const KVT*>(my_smem + (size_t)s * 2 * WBLK);
        const KVT* Vp = reinterpret_cast<const KVT*>(my_smem + (size_t)s * 2 * WBLK + WBLK);
        const int nkw = pos + 1 - (pg0 + pg) * kPage - wk0;     // valid keys among this warp's KW (>= 1)
        float sc[PASSES];
        float mx = -INFINITY;
#pragma unroll
        for (int pi = 0; pi < PASSES; ++pi) {
            const int j = pi * KPI + grp;
            const uint4 v = *reinterpret_cast<const uint4*>(Kp + (size_t)j * HD + sub * EPC);
            float kf[EPC];
            unpack16<KVT>(v, kf);
            float sdot = 0.f;
#pragma unroll
            for (int e = 0; e < EPC; ++e) sdot += qf[e] * kf[e];
#pragma unroll
            for (int of = LPK / 2; of > 0; of >>= 1) sdot += __shfl_xor_sync(0xffffffffu, sdot, of);
            sc[pi] = j < nkw ? sdot * a.m.scale : -INFINITY;
            mx = fmaxf(mx, sc[pi]);
        }
#pragma unroll
        for (int of = 16; of >= LPK; of >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, of));
        const float m_new = fmaxf(m_run, mx);                    // finite: key wk0 of this page is valid
        const float corr = expf(m_run - m_new);
        m_run = m_new;
        float psum = 0.f;
#pragma unroll
        for (int pi = 0; pi < PASSES; ++pi) { sc[pi] = expf(sc[pi] - m_new); psum += sc[pi]; }
        l_run = l_run * corr + psum;                             // per key group; groups are summed at the end
#pragma unroll
        for (int d = 0; d < DL; ++d) o[d] *= corr;
        if (nkw >= KW) {
#pragma unroll
            for (int pi = 0; pi < PASSES; ++pi)
#pragma unroll
                for (int g = 0; g < KPI; g += KGW) {
                    const float p = __shfl_sync(0xffffffffu, sc[pi], (g + kgw) * LPK);
                    float vf[DL];
                    load_vals<DL>(Vp + (size_t)(pi * KPI + g + kgw) * HD + dv, vf);
#pragma unroll
                    for (int d = 0; d < DL; ++d) o[d] += p * vf[d];
                }
        } else {                                                 // rows past the last position hold arbitrary bits
#pragma unroll
            for (int pi = 0; pi < PASSES; ++pi)
#pragma unroll
                for (int g = 0; g < KPI; g += KGW) {
                    const float p = __shfl_sync(0xffffffffu, sc[pi], (g + kgw) * LPK);
                    float vf[DL];
                    load_vals<DL>(Vp + (size_t)(pi * KPI + g + kgw) * HD + dv, vf);
                    const bool valid = pi * KPI + g + kgw < nkw;
#pragma unroll
                    for (int d = 0; d < DL; ++d) o[d] += valid ? p * vf[d] : 0.f;
                }
        }
        __syncwarp();                                            // every lane is done with stage s
        if (lane == 0 && pg + ST < my_pages) issue(pg + ST);
    }
    if (!ok) { s_ok = 0; atomicExch(status, 21u); }
    // merge the four warps' states
#pragma unroll
    for (int of = 16; of >= LPK; of >>= 1) l_run += __shfl_xor_sync(0xffffffffu, l_run, of);
    if (KGW == 2) {
#pragma unroll
        for (int d = 0; d < DL; ++d) o[d] += __shfl_xor_sync(0xffffffffu, o[d], LPV & 31);
    }
    if (kgw == 0) {
#pragma unroll
        for (int d = 0; d < DL; ++d) red_o[warp][dv + d] = o[d];
    }
    if (lane == 0) { red_m[warp] = m_run; red_l[warp] = l_run; }
    __syncthreads();
    if (!s_ok) {                                  // let copies in flight land before shared memory is released
        for (int i = 0; i < 32; ++i) __nanosleep(16384);
        return;
    }
    float blk_m = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) blk_m = fmaxf(blk_m, red_m[w]);
    float ov = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        const float wt = red_m[w] == -INFINITY ? 0.f : expf(red_m[w] - blk_m);
        l += wt * red_l[w];
        if (tid < HD) ov += wt * red_o[w][tid];
    }
    if (a.n_splits == 1) {
        if (tid < HD) {
            const float r = ov / l;
            a.out[(size_t)tok * D + head * HD + tid] = r;
            if (a.out_bf16) a.out_bf16[(size_t)tok * D + head * HD + tid] = __float2bfloat16_rn(r);
        }
        return;
    }
    // several splits: publish the partial; the block that takes the last ticket merges in split order
    const size_t pidx = ((size_t)tok * a.m.H + head) * a.n_splits + split;
    if (tid < HD) a.part_o[pidx * HD + tid] = ov;
    if (tid == 0) { a.part_ml[pidx * 2] = blk_m; a.part_ml[pidx * 2 + 1] = l; }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&a.ticket[(size_t)tok * a.m.H + head], 1u) == (unsigned int)a.n_splits - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const size_t base = ((size_t)tok * a.m.H + head) * a.n_splits;
    float mx = -INFINITY;
    for (int sp = 0; sp < a.n_splits; ++sp) mx = fmaxf(mx, __ldcg(a.part_ml + (base + sp) * 2));
    if (tid < HD) {
        float num = 0.f, den = 0.f;
        for (int sp = 0; sp < a.n_splits; ++sp) {
            const float ms = __ldcg(a.part_ml + (base + sp) * 2);
            if (ms == -INFINITY) continue;
            const float w = expf(ms - mx);
            den += w * __ldcg(a.part_ml + (base + sp) * 2 + 1);
            num += w * __ldcg(a.part_o + (base + sp) * HD + tid);
        }
        const float r = num / den;
        a.out[(size_t)tok * D + head * HD + tid] = r;
        if (a.out_bf16) a.out_bf16[(size_t)tok * D + head * HD + tid] = __float2bfloat16_rn(r);
    }
    if (tid == 0) a.ticket[(size_t)tok * a.m.H + head] = 0;
}

template <typename KVT, int HD, int ST> constexpr size_t attn_stream_smem() {
    return (size_t)ST * 2 * kPage * HD * sizeof(KVT);
}

}  // namespace sllm
