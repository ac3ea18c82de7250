// Causal attention for one query position per (token, head) when there are many (token, head) pairs
// (decode at large batch, prefill chunks): one block per pair streams that head's K and V pages through
// shared memory with bulk asynchronous copies (cp.async.bulk, the 1-D form of TMA: each page holds the
// head's 64 keys as one contiguous run, and its 64 values as another), three pages in flight per block,
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
constexpr int kStreamStages = 3;

__device__ __forceinline__ uint32_t as_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// false = gave up after two seconds
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (bar_try(bar, parity)) return true;
        if (i < 64) continue;
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > 2000000000ull) return false;
        __nanosleep(64);
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <typename KVT, int HD>
__global__ void __launch_bounds__(kStreamThreads) k_attn_stream(const AttnDecArgs a, unsigned int* status) {
    constexpr int EPC = Elems<KVT>::per16;
    constexpr int LPK = HD / EPC;
    constexpr int KPI = 32 / LPK;
    constexpr int WARPS = kStreamThreads / 32;
    constexpr int DP = HD / 2;
    constexpr int KG = kStreamThreads / DP;
    constexpr uint32_t BLK = kPage * HD * sizeof(KVT);           // bytes of one page's K (or V) for one head
    static_assert(kStreamThreads % DP == 0 && LPK <= 32, "unsupported head_dim");

    extern __shared__ __align__(128) unsigned char smem_raw[];   // [stages][K block | V block]
    __shared__ __align__(8) unsigned long long bars[kStreamStages];
    __shared__ float sc[kPage];
    __shared__ float red_o[KG][HD];
    __shared__ float red_l[KG];
    __shared__ float s_q[HD];
    __shared__ int s_ok;
    __shared__ unsigned int s_last;

    const int split = blockIdx.x, head = blockIdx.y, tok = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (tid == 0) {
        for (int s = 0; s < kStreamStages; ++s) bar_init(as_smem(&bars[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_ok = 1;
    }
    pdl_launch_dependents();
    pdl_wait();

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
    __syncthreads();

    auto issue = [&](int pg) {                   // one thread: both copies of page pg into stage pg % stages
        const int s = pg % kStreamStages;
        const int page = table[pg];
        const uint32_t bar = as_smem(&bars[s]);
        bar_expect(bar, 2 * BLK);
        bulk_g2s(as_smem(smem_raw + (size_t)s * 2 * BLK), kv_ptr<KVT>(a.kv, a.m, a.layer, page, 0, head, 0), BLK, bar);
        bulk_g2s(as_smem(smem_raw + (size_t)s * 2 * BLK + BLK), kv_ptr<KVT>(a.kv, a.m, a.layer, page, 1, head, 0), BLK, bar);
    };
    if (tid == 0)
        for (int pg = 0; pg < kStreamStages && pg < n_pages; ++pg) issue(pg);

    const int sub = lane % LPK;
    float qf[EPC];
#pragma unroll
    for (int e = 0; e < EPC; ++e) qf[e] = s_q[sub * EPC + e];
    const int dp = tid % DP, kg = tid / DP;
    float m_run = -INFINITY, l_run = 0.f, o0 = 0.f, o1 = 0.f;

    for (int pg = 0; pg < n_pages; ++pg) {
        const int s = pg % kStreamStages;
        if (!bar_wait(as_smem(&bars[s]), (pg / kStreamStages) & 1)) { s_ok = 0; atomicExch(status, 21u); }
        __syncthreads();
        if (!s_ok) break;                         // uniform after the barrier
        const KVT* Kp = reinterpret_cast<const KVT*>(smem_raw + (size_t)s * 2 * BLK);
        const KVT* Vp = reinterpret_cast<const KVT*>(smem_raw + (size_t)s * 2 * BLK + BLK);
        const int nk = min(kPage, pos + 1 - (pg0 + pg) * kPage);
        for (int j = warp * KPI + lane / LPK; j < kPage; j += WARPS * KPI) {
            float sdot = 0.f;
            if (j < nk) {
                const uint4 v = *reinterpret_cast<const uint4*>(Kp + (size_t)j * HD + sub * EPC);
                float kf[EPC];
                unpack16<KVT>(v, kf);
#pragma unroll
                for (int e = 0; e < EPC; ++e) sdot += qf[e] * kf[e];
            }
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) sdot += __shfl_xor_sync(0xffffffffu, sdot, o);
            if (sub == 0) sc[j] = (j < nk) ? sdot * a.m.scale : -INFINITY;
        }
        __syncthreads();
        float pm = -INFINITY;
        for (int j = lane; j < kPage; j += 32) pm = fmaxf(pm, sc[j]);
        pm = warp_max(pm);
        const float m_new = fmaxf(m_run, pm);
        const float corr = expf(m_run - m_new);
        l_run *= corr; o0 *= corr; o1 *= corr;
        m_run = m_new;
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
            l_run += p; o0 += p * v0; o1 += p * v1;
        }
        __syncthreads();                          // everyone is done with stage s
        if (tid == 0 && pg + kStreamStages < n_pages) issue(pg + kStreamStages);
    }
    if (!s_ok) {                                  // let copies in flight land before shared memory is released
        for (int i = 0; i < 32; ++i) __nanosleep(16384);
        return;
    }
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
            const float r = o / l;
            a.out[(size_t)tok * D + head * HD + tid] = r;
            if (a.out_bf16) a.out_bf16[(size_t)tok * D + head * HD + tid] = __float2bfloat16_rn(r);
        }
        return;
    }
    // several splits: publish the partial; the block that takes the last ticket merges in split order
    const size_t pidx = ((size_t)tok * a.m.H + head) * a.n_splits + split;
    if (tid < HD) a.part_o[pidx * HD + tid] = o;
    if (tid == 0) { a.part_ml[pidx * 2] = m_run; a.part_ml[pidx * 2 + 1] = l; }
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

template <typename KVT, int HD> constexpr size_t attn_stream_smem() {
    return (size_t)kStreamStages * 2 * kPage * HD * sizeof(KVT);
}

}  // namespace sllm
