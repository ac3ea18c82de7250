// Causal attention for runs of consecutive query positions (prefill) on the 5th-generation tensor cores, for
// bf16 KV pages and head_dim 64: one block per (tile of up to 128 queries, head).
//
// Replaces the reference's materialised scores / causal softmax / PV chain for T > 1
// (src/ops/attention.cpp:45-50,179-183, src/ops/softmax.cpp:24-40) with an online softmax per query row:
//   per KV page (64 keys):  S = Q K^T        tcgen05.mma, 128 x 64 x 64, accumulator in tensor memory
//                           P = exp(S*scale - max) as bf16 in shared memory, row sums / maxima in registers
//                           PV = P V         tcgen05.mma, 128 x 64 x 64
//                           O = O * corr + PV  in registers (one thread owns one query row = one TMEM lane)
// Operands in shared memory are K-major with the 128-byte swizzle: K pages come in by TMA over the whole KV pool
// (a [rows][64] bf16 tensor), V pages by a bulk copy and are transposed to [dim][key] by four warps, Q (fp32 from
// the projection) and P are written by the threads themselves in the swizzled layout.
// Warps: 0 = copy producer, 1 = MMA issuer and TMEM owner, 2-5 = softmax (TMEM lane quarters 2,3,0,1); the softmax
// warps also transpose the next page's V while the PV product of this page runs.  S is double-buffered in TMEM so that
// S of the next page is computed while the softmax of this one runs.  192 threads at <= 168 registers and 97 KB of
// shared memory: two blocks per SM, which overlap each other's dependency chains.  Every mbarrier wait is bounded
// (two seconds), as in gemm_tc.cuh.
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
           + (size_t)kPtStages * kPtPageBytes * 2          // K stages, raw V stages
           + 2 * (size_t)kPtPageBytes                      // transposed V, two buffers
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
    uint8_t* sVraw = sK + kPtStages * kPtPageBytes;
    uint8_t* sVt = sVraw + kPtStages * kPtPageBytes;
    uint8_t* sP = sVt + 2 * kPtPageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kPtQ * 128);
    // barrier indices
    enum { K_FULL = 0, V_FULL = 3, K_FREE = 6, V_FREE = 9, S_READY = 12, S_FREE = 14, VT_READY = 16, P_READY = 18,
           PV_READY = 19, N_BARS = 20 };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
    const uint32_t bar0 = smem_u32(bars);
    auto B = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    const PfTile t = a.tiles[blockIdx.x];
    const int head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = a.m.D;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 3; ++i) { mbar_init(B(K_FULL + i), 1); mbar_init(B(V_FULL + i), 1); mbar_init(B(K_FREE + i), 1); mbar_init(B(V_FREE + i), 4); }
        for (int i = 0; i < 2; ++i) { mbar_init(B(S_READY + i), 1); mbar_init(B(S_FREE + i), 4); mbar_init(B(VT_READY + i), 4); }
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
                bulk_g2s(smem_u32(sVraw + s * kPtPageBytes), kv_ptr<__nv_bfloat16>(a.kv, a.m, a.layer, page, 1, head, 0), kPtPageBytes,
                         B(V_FULL + s));
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
                const int b = i & 1;
                ok = mbar_wait(B(P_READY), i & 1, a.status, 35) && mbar_wait(B(VT_READY + b), (i >> 1) & 1, a.status, 36);
                if (!ok) break;
                tc_fence_after();
                const uint32_t pa = smem_u32(sP), vb = smem_u32(sVt + b * kPtPageBytes);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tc_mma_bf16(tmem + 128u, tc_smem_desc(pa + k * 32), tc_smem_desc(vb + k * 32), idesc, k != 0);
                tc_commit(B(PV_READY));
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
        const int tt = threadIdx.x - 64, h = tt & 63, half = tt >> 6;
        // page [key][dim] -> [dim][key], K-major swizzled, into buffer i & 1.  The buffer was last read by the PV
        // product of page i - 2, whose completion this thread has already waited for.
        auto transpose_v = [&](int i) -> bool {
            const int s = i % kPtStages;
            bool good = mbar_wait(B(V_FULL + s), (i / kPtStages) & 1, a.status, 39);
            good = __all_sync(0xffffffffu, good);
            if (!good) return false;
            const unsigned short* src = reinterpret_cast<const unsigned short*>(sVraw + s * kPtPageBytes) + (half * 32) * 64 + h;
            uint8_t* dst = sVt + (i & 1) * kPtPageBytes;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t lo = src[(c * 8 + 2 * e) * 64], hi = src[(c * 8 + 2 * e + 1) * 64];
                    w[e] = lo | (hi << 16);
                }
                *reinterpret_cast<uint4*>(dst + sw128(h, half * 4 + c)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) { mbar_arrive(B(VT_READY + (i & 1))); mbar_arrive(B(V_FREE + s)); }
            return true;
        };
        ok = transpose_v(0);
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
            const int kbase = i * kPage;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 64; ++j) {
                const float s = (kbase + j <= qpos) ? __uint_as_float(sv[j]) * a.m.scale : -INFINITY;
                sv[j] = __float_as_uint(s);
                mx = fmaxf(mx, s);
            }
            const float m_new = fmaxf(m_run, mx);              // finite from the first page on: key 0 is never masked
            const float corr = expf(m_run - m_new);
            m_run = m_new;
            float sum = 0.f;
            uint32_t pk[32];
#pragma unroll
            for (int j = 0; j < 64; j += 2) {
                const float p0 = expf(__uint_as_float(sv[j]) - m_new), p1 = expf(__uint_as_float(sv[j + 1]) - m_new);
                sum += p0 + p1;
                pk[j >> 1] = pack_bf16(p0, p1);
            }
            l_run = l_run * corr + sum;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(sP + sw128(r, c)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            fence_async_smem();
            tc_fence_before();                                   // the PV loads of the previous page are done before the next PV may start
            __syncwarp();
            if (lane == 0) mbar_arrive(B(P_READY));
            if (i + 1 < n_pages && !transpose_v(i + 1)) { ok = false; break; }   // while the PV product of this page runs
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
