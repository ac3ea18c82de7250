// Causal attention for runs of consecutive query positions (prefill) on the 5th-generation tensor cores, for
// bf16 KV pages and head_dim 64: one block per (tile of up to 128 queries, head).
//
// Replaces the reference's materialised scores / causal softmax / PV chain for T > 1
// (src/ops/attention.cpp:45-50,179-183, src/ops/softmax.cpp:24-40) with an online softmax per query row:
//   per KV page (64 keys):  S = Q K^T        tcgen05.mma, 128 x 64 x 64, accumulator in tensor memory
//                           P = exp(S*scale - max) as bf16 in shared memory, row sums / maxima in registers
//                           PV = P V         tcgen05.mma, 128 x 64 x 64
//                           O = O * corr + PV  in registers (one thread owns one query row = one TMEM lane)
// Operands in shared memory carry the 128-byte swizzle.  K and V pages come in by TMA over the whole KV pool (a
// [rows][64] bf16 tensor) exactly as they lie in the cache, [key][dim]: for S the K page is the K-major B operand
// (dim is the contraction), for PV the V page is the MN-major B operand (key is the contraction, dim contiguous), so
// nothing is transposed.  Q (fp32 from the projection) and P are written by the threads themselves in the swizzled
// K-major layout.  exp(x) is evaluated as exp2(x * log2 e); the causal mask is applied only on pages that reach the
// tile's first query.
// Warps: 0 = copy producer, 1 = MMA issuer and TMEM owner, 2-5 = softmax (TMEM lane quarters 2,3,0,1).  S is
// double-buffered in TMEM so that S of the next page is computed while the softmax of this one runs.  192 threads at
// <= 168 registers and 81 KB of shared memory: two blocks per SM, which overlap each other's dependency chains.
// Every mbarrier wait is bounded (two seconds), as in gemm_tc.cuh.
#pragma once
#include "attn_stream.cuh"
#include "gemm_tc.cuh"

namespace sllm {

constexpr int kPtThreads = 192;
constexpr int kPtQ = 128;                    // query rows per tile (UMMA M)
constexpr int kPtStages = 3;                 // K / raw-V pages in flight
constexpr uint32_t kPtPageBytes = kPage * 64 * 2;           // one page of K (or V) of one head: 8 KB

struct AttnPtArgs {
    const float* q;            // [n_tok][D] rotated queries (fp32)
    float* out;                // [n_tok][D]
    __nv_bfloat16* out_bf16;   // optional
    ModelDims m;
    KvView kv;
    const PfTile* tiles;       // up to kPtQ queries each
    int layer;
    unsigned int* status;
};

constexpr size_t attn_prefill_tc_smem() {
    return 1024 + (size_t)kPtQ * 128                       // Q
           + (size_t)kPtStages * kPtPageBytes * 2          // K stages, V stages
           + (size_t)kPtQ * 128                            // P
           + 256;                                          // barriers, TMEM slot
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// byte offset of 16-byte chunk c of row r in a K-major tile with 128-byte rows and the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__global__ void __launch_bounds__(kPtThreads, 2) k_attn_prefill_tc(const __grid_constant__ CUtensorMap map_kv, const AttnPtArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + kPtQ * 128;
    uint8_t* sV = sK + kPtStages * kPtPageBytes;
    uint8_t* sP = sV + kPtStages * kPtPageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kPtQ * 128);
    // barrier indices
    enum { K_FULL = 0, V_FULL = 3, K_FREE = 6, V_FREE = 9, S_READY = 12, S_FREE = 14, P_READY = 16, PV_READY = 17, N_BARS = 18 };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
    const uint32_t bar0 = smem_u32(bars);
    auto B = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    const PfTile t = a.tiles[blockIdx.x];
    const int head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = a.m.D;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 3; ++i) { mbar_init(B(K_FULL + i), 1); mbar_init(B(V_FULL + i), 1); mbar_init(B(K_FREE + i), 1); mbar_init(B(V_FREE + i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(B(S_READY + i), 1); mbar_init(B(S_FREE + i), 4); }
        mbar_init(B(P_READY), 4); mbar_init(B(PV_READY), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    pdl_launch_dependents();
    pdl_wait();

    // Q tile: fp32 rows -> bf16, K-major swizzled; rows past the tile's queries are zero
    for (int i = threadIdx.x; i < kPtQ * 8; i += kPtThreads) {
        const int r = i >> 3, c = i & 7;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < t.n_q) {
            const float4* src = reinterpret_cast<const float4*>(a.q + (size_t)(t.tok_begin + r) * D + head * 64 + c * 8);
            const float4 x = src[0], y = src[1];
            v = make_uint4(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w), pack_bf16(y.x, y.y), pack_bf16(y.z, y.w));
        }
        *reinterpret_cast<uint4*>(sQ + sw128(r, c)) = v;
    }
    fence_async_smem();
    __syncthreads();

    const int n_pages = (t.pos0 + t.n_q - 1) / kPage + 1;
    const int* table = a.kv.block_table + (size_t)t.slot * a.kv.pages_per_seq;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < n_pages && ok; ++i) {
                const int s = i % kPtStages;
                if (i >= kPtStages) {
                    const uint32_t par = ((i / kPtStages) - 1) & 1;
                    ok = mbar_wait(B(K_FREE + s), par, a.status, 31) && mbar_wait(B(V_FREE + s), par, a.status, 32);
                    if (!ok) break;
                }
                const int page = table[i];
                const long long row = ((((long long)a.layer * a.kv.n_pages + page) * 2) * a.m.H + head) * kPage;
                mbar_expect_tx(B(K_FULL + s), kPtPageBytes);
                tma_load_2d(smem_u32(sK + s * kPtPageBytes), &map_kv, 0, (int)row, B(K_FULL + s));
                mbar_expect_tx(B(V_FULL + s), kPtPageBytes);
                tma_load_2d(smem_u32(sV + s * kPtPageBytes), &map_kv, 0, (int)(row + (long long)a.m.H * kPage), B(V_FULL + s));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = tc_idesc(kPtQ, 64);
            auto issue_qk = [&](int i) -> bool {
                const int s = i % kPtStages, b = i & 1;
                if (!mbar_wait(B(K_FULL + s), (i / kPtStages) & 1, a.status, 33)) return false;
                if (i >= 2 && !mbar_wait(B(S_FREE + b), ((i >> 1) - 1) & 1, a.status, 34)) return false;
                tc_fence_after();
                const uint32_t qa = smem_u32(sQ), kb = smem_u32(sK + s * kPtPageBytes);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tc_mma_bf16(tmem + (uint32_t)(b * 64), tc_smem_desc(qa + k * 32), tc_smem_desc(kb + k * 32), idesc, k != 0);
                tc_commit(B(S_READY + b));
                tc_commit(B(K_FREE + s));
                return true;
            };
            ok = issue_qk(0);
            for (int i = 0; i < n_pages && ok; ++i) {
                if (i + 1 < n_pages) { ok = issue_qk(i + 1); if (!ok) break; }
                const int sv_ = i % kPtStages;
                ok = mbar_wait(B(P_READY), i & 1, a.status, 35) && mbar_wait(B(V_FULL + sv_), (i / kPtStages) & 1, a.status, 36);
                if (!ok) break;
                tc_fence_after();
                // V page as it lies in the cache, [key][dim]: the B operand in MN-major form (dim contiguous), 16 keys
                // (two 8-row groups of 1024 bytes) per MMA
                const uint32_t pa = smem_u32(sP), vb = smem_u32(sV + sv_ * kPtPageBytes);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tc_mma_bf16(tmem + 128u, tc_smem_desc(pa + k * 32), tc_smem_desc(vb + k * 2048), idesc | (1u << 16), k != 0);
                tc_commit(B(PV_READY));
                tc_commit(B(V_FREE + sv_));
            }
        }
    } else {
        // ---- softmax: thread = query row = TMEM lane; transposition of V: thread = (dim, half of the keys) ----
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int qpos = t.pos0 + r;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        float o[64];
#pragma unroll
        for (int d = 0; d < 64; ++d) o[d] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;
        const float sl2 = a.m.scale * 1.4426950408889634f;
        for (int i = 0; i < n_pages && ok; ++i) {
            const int b = i & 1;
            ok = mbar_wait(B(S_READY + b), (i >> 1) & 1, a.status, 37);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t sv[64];
            tc_ld32(lane_addr + (uint32_t)(b * 64), sv);
            tc_ld32(lane_addr + (uint32_t)(b * 64 + 32), sv + 32);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(B(S_FREE + b));
            // scores in units of log2(e): exp(x) = exp2(x * log2 e), one multiply and one ex2 per element
            const int kbase = i * kPage;
            float mxp[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four interleaved chains instead of one of 64
            if (kbase + kPage - 1 <= t.pos0) {                   // page entirely before the tile's first query: no mask
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    const float s = __uint_as_float(sv[j]) * sl2;
                    sv[j] = __float_as_uint(s);
                    mxp[j & 3] = fmaxf(mxp[j & 3], s);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    const float s = (kbase + j <= qpos) ? __uint_as_float(sv[j]) * sl2 : -INFINITY;
                    sv[j] = __float_as_uint(s);
                    mxp[j & 3] = fmaxf(mxp[j & 3], s);
                }
            }
            const float mx = fmaxf(fmaxf(mxp[0], mxp[1]), fmaxf(mxp[2], mxp[3]));
            const float m_new = fmaxf(m_run, mx);              // finite from the first page on: key 0 is never masked
            const float corr = exp2f(m_run - m_new);
            m_run = m_new;
            float sump[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[32];
#pragma unroll
            for (int j = 0; j < 64; j += 2) {
                const float p0 = exp2f(__uint_as_float(sv[j]) - m_new), p1 = exp2f(__uint_as_float(sv[j + 1]) - m_new);
                sump[(j >> 1) & 3] += p0 + p1;
                pk[j >> 1] = pack_bf16(p0, p1);
            }
            const float sum = (sump[0] + sump[1]) + (sump[2] + sump[3]);
            l_run = l_run * corr + sum;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(sP + sw128(r, c)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            fence_async_smem();
            tc_fence_before();                                   // the PV loads of the previous page are done before the next PV may start
            __syncwarp();
            if (lane == 0) mbar_arrive(B(P_READY));
            ok = mbar_wait(B(PV_READY), i & 1, a.status, 38);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            tc_ld32(lane_addr + 128u, sv);
            tc_ld32(lane_addr + 160u, sv + 32);
#pragma unroll
            for (int d = 0; d < 64; ++d) o[d] = o[d] * corr + __uint_as_float(sv[d]);
        }
        if (ok && r < t.n_q) {
            const float inv = 1.0f / l_run;
            float* dst = a.out + (size_t)(t.tok_begin + r) * D + head * 64;
#pragma unroll
            for (int d = 0; d < 64; d += 4)
                *reinterpret_cast<float4*>(dst + d) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
            if (a.out_bf16) {
                uint4* d16 = reinterpret_cast<uint4*>(a.out_bf16 + (size_t)(t.tok_begin + r) * D + head * 64);
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    d16[c] = make_uint4(pack_bf16(o[8 * c] * inv, o[8 * c + 1] * inv), pack_bf16(o[8 * c + 2] * inv, o[8 * c + 3] * inv),
                                        pack_bf16(o[8 * c + 4] * inv, o[8 * c + 5] * inv), pack_bf16(o[8 * c + 6] * inv, o[8 * c + 7] * inv));
            }
        }
    }
    if (!ok) {                       // a wait gave up: give copies in flight time to land before shared memory goes away
        for (int i = 0; i < 64; ++i) __nanosleep(16384);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256));
    }
}

}  // namespace sllm
