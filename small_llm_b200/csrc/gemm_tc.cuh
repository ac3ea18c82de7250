// Dense projections for two and more tokens (prefill, batched decode) on the 5th-generation tensor
// cores: tcgen05.mma with the accumulator in tensor memory, operands staged in shared memory by
// TMA (cp.async.bulk.tensor, no multicast), bf16 x bf16 -> fp32.
//
//   out[tok][r] = sum_k X[tok][k] * W[r][k]        X: [tokens][K] bf16,  W: [R][K] bf16, both K-major
//
// The weight tile is the MMA's M side (128 rows = 128 TMEM lanes), the token tile its N side
// (32..256 columns), so the batch does not have to fill a 128-row tile.  A thread block computes 128 x BN tiles --
// one, or, when there are more tiles than SMs, its share of them with two accumulators in tensor memory so that a
// tile's epilogue overlaps the next tile's main loop:  warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2.. (8 or 16 of them) = epilogue.  The epilogue reads the accumulator as thread = weight row, registers =
// tokens, and (row counts that are multiples of 4) transposes it through shared memory so that a lane stores 16 bytes
// of consecutive rows of one token; the same fused epilogues as the GEMV family: RoPE + paged-KV append, residual
// add, SiLU(gate)*up, fp32 logits.
// Every mbarrier wait is bounded; on expiry the block raises the engine's status word, lets its
// copies land, frees its tensor memory and returns.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "gemv.cuh"

namespace sllm {

constexpr int kTcBM = 128;          // weight rows per tile (UMMA M)
constexpr int kTcBK = 64;           // K elements per stage = one 128-byte swizzle row of bf16
// Epilogue warps: 8 (two per TMEM lane quarter) for 32-token tiles, 16 from 64 tokens on, where the epilogue takes
// longer than the main loop and the transposing form (TcArgs::wide_epi) needs groups of four warps per 16 columns
// (measured at 256..512 sequences per decode pass: 0.3-0.8 % per iteration over 8 warps with the thread-per-row form).
template <int BN> __host__ __device__ constexpr int tc_epi_warps() { return BN >= 64 ? 16 : 8; }
template <int BN> __host__ __device__ constexpr int tc_threads() { return 64 + 32 * tc_epi_warps<BN>(); }
constexpr int kTcMaxStages = 16;
constexpr int kTcMaxSplit = 8;

struct TcArgs {
    int R, K, n_tok;
    float* out;                     // QKV: q fp32 [tok][D]; Residual: x fp32 [tok][R]; Head: logits fp32 [tok][R]
    __nv_bfloat16* out_bf16;        // GateUp: hidden bf16 [tok][R/2]
    ModelDims m;
    KvView kv;
    PassView pass;
    int layer;
    const float2* rope;
    unsigned int* status;           // engine status word (0 = fine)
    // RMSNorm folded into the projections around it (src/ops/rmsnorm.cpp:38-60: y = x * r * g, r = 1/sqrt(mean(x^2) + eps)):
    // a Residual epilogue that knows the next norm's gain stores bf16(x_new * g) as the next projection's operand and
    // the sums of squares of its 32-row slices; the consuming epilogue multiplies its accumulator by r (the product is
    // linear in r), which it gets from those partial sums.
    const float* gain_next;         // Residual: gain of the norm that follows (null: nothing follows)
    __nv_bfloat16* xn_out;          // Residual: [tok][R] bf16(x_new * gain_next)
    float* ss_out;                  // Residual: [tok][n_parts] partial sums of squares, part = row tile * 4 + lane quarter
    const float* ss_in;             // QKV / GateUp: the same array, written by the producer (null: operand already normalised)
    int n_parts;
    float eps;
    // Split-K over a thread-block cluster (grid z = cluster z = split): block z accumulates its share of the K
    // blocks in its own tensor memory; blocks 1.. hand their accumulators to block 0 through distributed shared
    // memory, block 0 adds them in rank order and runs the epilogue.  With few tiles (small batches) this spreads a
    // tile's weight bytes over several SMs, each of which can only take in ~65 GB/s.
    int stages;                     // pipeline stages of this launch (<= kTcMaxStages)
    int split;                      // blocks per cluster (1 = no cluster)
    // More tiles than the GPU holds blocks (prefill): grid x = resident blocks, block b takes tiles b, b + grid x, ...
    // with two accumulators in tensor memory, so that the epilogue of one tile (loads and stores scattered by token,
    // longer than the main loop) runs while the tensor cores work on the next.  Otherwise one tile per block,
    // taken from the block index.
    int persistent;
    int n_tiles;                    // weight row tiles x token tiles
    // Transposing epilogue (every row count a multiple of 4): the four warps that share a column group transpose each
    // 16-column chunk of the accumulator (after adding the split-K peers' shares) through shared memory, after which a
    // lane holds four consecutive output rows of one token and loads / stores 16 bytes at a time -- a tenth of the
    // address arithmetic and memory instructions of the thread-per-row epilogue, which is bound by instruction issue on
    // wide tiles (prefill: 75 -> 44 us for the QKV projection of 8192 positions; decode at 64 sequences: 1.7 % per iteration).
    int wide_epi;
};

// Sums v[j] over the 32 lanes for every j at once: afterwards lane j holds the sum of all lanes' v[j] (31 shuffles,
// a fixed tree, so the result does not depend on timing).
__device__ __forceinline__ float warp_column_sums(float (&v)[32], int lane) {
#pragma unroll
    for (int step = 16; step >= 1; step >>= 1) {
        const bool up = (lane & step) != 0;
#pragma unroll
        for (int i = 0; i < step; ++i) {
            const float send = up ? v[i] : v[i + step];
            const float keep = up ? v[i + step] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, step);
        }
    }
    return v[0];
}

// ---- PTX wrappers -----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) { return mbar_try_parity(bar, parity); }
// bounded wait; false = gave up (status word raised)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned int* status, unsigned int code) {
    if (mbar_wait_bounded(bar, parity, c_wait_limit_ns)) return true;
    atomicExch(status, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
// K-major operand tile, rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16: D fp32, A and B bf16, both K-major, N and M encoded >>3 and >>4
__device__ __forceinline__ uint32_t tc_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
template <int CW> __device__ __forceinline__ void tc_ld(uint32_t taddr, uint32_t* r) {
    if (CW == 32) tc_ld32(taddr, r); else tc_ld16(taddr, r);
}

// Shared memory of one block: [1 KB alignment slack][stages x (weight tile | token tile)][barriers, TMEM slot: 512 B]
// [token metadata: per epilogue warp its columns' positions, pages and 1/rms: 12 x BN words in all][split > 1: (split - 1) accumulators of 128 x BN floats handed over
// by the peers][transposing epilogue: the column groups' buffers]
constexpr size_t tc_stage_bytes(int bn) { return (size_t)kTcBM * kTcBK * 2 + (size_t)bn * kTcBK * 2; }
// transposing epilogue: per column group (4 epilogue warps) 2 buffers of [16 columns][128 rows] floats
constexpr size_t tc_wide_bytes(int bn) { return (size_t)(bn >= 64 ? 4 : 2) * 2 * 16 * kTcBM * sizeof(float); }
constexpr size_t tc_fixed_bytes(int bn, int split, bool wide = false) {
    return 1024 + 512 + (size_t)12 * bn * sizeof(int) + (size_t)(split - 1) * kTcBM * bn * sizeof(float) +
           (wide ? tc_wide_bytes(bn) : 0);
}
constexpr size_t tc_smem_bytes(int bn, int stages, int split, bool wide = false) {
    return tc_fixed_bytes(bn, split, wide) + (size_t)stages * tc_stage_bytes(bn);
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in the cluster's block `rank`
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// barrier `id` over 128 threads (the four warps of a column group) that also ANDs a flag over them
__device__ __forceinline__ bool group_sync_and(int id, bool flag) {
    uint32_t out;
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.and.pred p, %2, 128, q;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(out) : "r"((uint32_t)flag), "r"(id) : "memory");
    return out != 0;
}
__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <int BN, int MODE>
__global__ void __launch_bounds__(tc_threads<BN>()) k_gemm_tc(const __grid_constant__ CUtensorMap map_w,
                                                        const __grid_constant__ CUtensorMap map_x, const TcArgs a) {
    constexpr uint32_t A_BYTES = kTcBM * kTcBK * 2, B_BYTES = BN * kTcBK * 2;
    const int STAGES = a.stages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * B_BYTES);   // full[16], empty[16], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kTcMaxStages + 4);
    int* tok_meta = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 512);   // [epilogue warps][pos | page of the warp's columns]
    float* tok_rs = reinterpret_cast<float*>(tok_meta + 8 * BN);            // [epilogue warps][its columns]: 1/rms of the warp's tokens
    float* handover = tok_rs + 4 * BN;                                      // [split - 1][BN][128] in block 0 of the cluster
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kTcMaxStages);
    const uint32_t accf0 = smem_u32(bars + 2 * kTcMaxStages), acce0 = accf0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (a.R + kTcBM - 1) / kTcBM;
    // this block's tiles: first, first + step, ... (one tile unless persistent)
    const int tile_first = a.persistent ? (int)blockIdx.x : (int)(blockIdx.y * tiles_m + blockIdx.x);
    const int tile_step = a.persistent ? (int)gridDim.x : a.n_tiles;
    const uint32_t n_acc = a.persistent ? 2u : 1u;                          // accumulators in tensor memory
    const int split = a.split, ks = blockIdx.z;                             // the cluster spans grid z
    const int nkb_all = (a.K + kTcBK - 1) / kTcBK;
    const int kb_first = (nkb_all * ks) / split;
    const int nkb = (nkb_all * (ks + 1)) / split - kb_first;                // this block's K blocks (>= 1)

    if (threadIdx.x == 32) {                     // the descriptors' first use would otherwise wait for their fetch
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf0 + 8 * b, 1); mbar_init(acce0 + 8 * b, tc_epi_warps<BN>()); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(n_acc * BN));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    SLLM_TL(500 + MODE * 10);
    pdl_launch_dependents();
    // The weight tiles do not depend on the predecessor kernel: the first STAGES of them (of the block's first tile)
    // are requested before the dependency wait (the barrier already expects the bytes of both operands of its stage).
    const int pre = nkb < STAGES ? nkb : STAGES;
    if (warp == 0 && lane == 0) {
        const int m0 = (tile_first % tiles_m) * kTcBM;
        for (int kb = 0; kb < pre; ++kb) {
            mbar_expect_tx(full0 + 8 * kb, A_BYTES + B_BYTES);
            tma_load_2d(smem_u32(sA + kb * A_BYTES), &map_w, (kb_first + kb) * kTcBK, m0, full0 + 8 * kb);
        }
    }
    pdl_wait();
    SLLM_TL(501 + MODE * 10);

    bool ok = true;
    if (warp == 0) {
        if (lane == 0) {
            // stage index and round kept as counters: the stage count is a launch parameter, and an integer
            // division per K block on this single thread would be on the critical path
            int s = 0; uint32_t round = 0;
            for (int tile = tile_first; tile < a.n_tiles && ok; tile += tile_step) {
                const int m0 = (tile % tiles_m) * kTcBM, t0 = (tile / tiles_m) * BN;
                for (int kb = 0; kb < nkb && ok; ++kb) {
                    if (tile != tile_first || kb >= pre) {
                        ok = mbar_wait(empty0 + 8 * s, (round - 1) & 1, a.status, 11);
                        if (!ok) break;
                        mbar_expect_tx(full0 + 8 * s, A_BYTES + B_BYTES);
                        tma_load_2d(smem_u32(sA + s * A_BYTES), &map_w, (kb_first + kb) * kTcBK, m0, full0 + 8 * s);
                    }
                    tma_load_2d(smem_u32(sB + s * B_BYTES), &map_x, (kb_first + kb) * kTcBK, t0, full0 + 8 * s);
                    if (++s == STAGES) { s = 0; ++round; }
                }
            }
        }
        __syncwarp();
        if (split > 1) cluster_sync_all();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = tc_idesc(kTcBM, BN);
            int s = 0; uint32_t round = 0, it = 0;
            for (int tile = tile_first; tile < a.n_tiles && ok; tile += tile_step, ++it) {
                // the accumulator this tile goes to must have been read out by the epilogue of the tile two before
                const uint32_t buf = it & (n_acc - 1), use = it / n_acc;
                ok = mbar_wait(acce0 + 8 * buf, (use - 1) & 1, a.status, 14);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem + buf * BN;
                for (int kb = 0; kb < nkb && ok; ++kb) {
                    ok = mbar_wait(full0 + 8 * s, round & 1, a.status, 12);
                    if (!ok) break;
                    tc_fence_after();
                    if (kb == 0) SLLM_TL_HERE(502 + MODE * 10);
                    if (kb == nkb - 1) SLLM_TL_HERE(505 + MODE * 10);
                    const uint32_t aaddr = smem_u32(sA + s * A_BYTES), baddr = smem_u32(sB + s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < kTcBK / 16; ++k)
                        tc_mma_bf16(acc, tc_smem_desc(aaddr + k * 32), tc_smem_desc(baddr + k * 32), idesc, (kb | k) != 0);
                    tc_commit(empty0 + 8 * s);          // the stage may be refilled once these MMAs have read it
                    if (++s == STAGES) { s = 0; ++round; }
                }
                if (ok) tc_commit(accf0 + 8 * buf);     // accumulator complete
            }
        }
        __syncwarp();
        if (split > 1) cluster_sync_all();
    } else {
        // ---- epilogue: warp w reads TMEM lane quarter w % 4, column group (w - 2) / 4 -------------------------
        constexpr int EW = tc_epi_warps<BN>();
        constexpr int HALF = BN / (EW / 4);                      // token columns per epilogue warp
        constexpr int CW = (EW == 16 || HALF < 32) ? 16 : 32;    // columns per TMEM load
        const int ew = warp - 2;
        const int quarter = warp & 3;
        const int cbeg = (ew >> 2) * HALF;
        uint32_t it = 0;
        for (int tile = tile_first; tile < a.n_tiles && ok; tile += tile_step, ++it) {
            const int mi = tile % tiles_m, m0 = mi * kTcBM, t0 = (tile / tiles_m) * BN;
            const uint32_t buf = it & (n_acc - 1);
            const uint32_t acc = tmem + buf * BN;                   // this tile's accumulator
            const int row = m0 + quarter * 32 + lane;
            const bool row_ok = row < a.R;
            const int D = a.m.D, hd = a.m.hd;
            int which = 0, col = 0, head = 0, d = 0;
            if (MODE == kModeQKV && row_ok) { which = row / D; col = row - which * D; head = col / hd; d = col - head * hd; }
            // While the tensor cores work, each epilogue warp fetches the positions and KV pages of its tokens into
            // its own shared-memory copy, and the operands of its first column chunk that do not depend on the
            // accumulator (rotation factors, residual values), so that little is left to wait for afterwards.
            // per token: its position (for the rotation factors) and the row of the KV pool, in units of head_dim
            // elements, at which head 0's K entry of that position lies
            int* my_pos = tok_meta + ew * 2 * HALF;
            uint32_t* my_kvrow = reinterpret_cast<uint32_t*>(my_pos + HALF);
            if (MODE == kModeQKV) {
                for (int j = lane; j < HALF; j += 32) {
                    const int tok = t0 + cbeg + j;
                    int pos = 0, page = 0;
                    if (tok < a.n_tok) {
                        pos = a.pass.tok_pos[tok];
                        page = a.kv.block_table[(size_t)a.pass.tok_slot[tok] * a.kv.pages_per_seq + pos / kPage];
                    }
                    my_pos[j] = pos;
                    my_kvrow[j] = (uint32_t)((((unsigned long long)a.layer * a.kv.n_pages + page) * 2 * a.m.H) * kPage + pos % kPage);
                }
                __syncwarp();
            }
            // this lane's constant part of the addresses it loads from and stores to
            float* const x_lane = a.out + row;                       // Residual / Head: [tok][R] fp32
            __nv_bfloat16* const xn_lane = a.xn_out + row;
            float* const q_lane = a.out + col;
            __nv_bfloat16* const kv_lane = reinterpret_cast<__nv_bfloat16*>(a.kv.pool) + d;
            const uint32_t kv_lane_row = (uint32_t)(((which > 0 ? which - 1 : 0) * a.m.H + head) * kPage);
            float2 cs[MODE == kModeQKV ? CW : 1];
            float xv[MODE == kModeResidual ? CW : 1];
            const bool scaled = (MODE == kModeQKV || MODE == kModeGateUp) && a.ss_in != nullptr;
            const float gnext = (MODE == kModeResidual && a.gain_next && row_ok) ? a.gain_next[row] : 0.f;
            // consumers of a folded norm: 1/rms of each of the warp's tokens, from the producer's partial sums of squares
            float* my_rs = tok_rs + ew * HALF;
            if (MODE == kModeQKV || MODE == kModeGateUp) {
                for (int j = lane; j < HALF; j += 32) {
                    const int tok = t0 + cbeg + j;
                    float r = 1.0f;
                    if (scaled && ks == 0 && tok < a.n_tok) {        // n_parts is a multiple of 4: 16-byte loads, 8 in flight per trip
                        const float4* pp = reinterpret_cast<const float4*>(a.ss_in + (size_t)tok * a.n_parts);
                        const int n4 = a.n_parts / 4;
                        float ss = 0.f;
                        for (int p0 = 0; p0 < n4; p0 += 8) {
                            float4 q[8];
    #pragma unroll
                            for (int i = 0; i < 8; ++i) q[i] = p0 + i < n4 ? pp[p0 + i] : make_float4(0.f, 0.f, 0.f, 0.f);
    #pragma unroll
                            for (int i = 0; i < 8; ++i) ss += (q[i].x + q[i].y) + (q[i].z + q[i].w);
                        }
                        r = 1.0f / sqrtf(ss / (float)a.K + a.eps);
                    }
                    my_rs[j] = r;
                }
                __syncwarp();
            }
            {
                if (a.wide_epi) {
                    // ---- wide tiles: transpose through shared memory, four consecutive rows per lane -----------------
                    const int grp = ew >> 2;
                    float* const stg = handover + (size_t)(split - 1) * BN * kTcBM + (size_t)grp * 2 * 16 * kTcBM;   // this group's two buffers [16][128]
                    const int r0 = m0 + 4 * lane;
                    const bool r_ok = r0 < a.R;                                      // R is a multiple of 4: all four rows or none
                    int w_which = 0, w_col = 0, w_head = 0, w_d = 0;
                    if (MODE == kModeQKV && r_ok) { w_which = r0 / D; w_col = r0 - w_which * D; w_head = w_col / hd; w_d = w_col - w_head * hd; }
                    float4 gn = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (MODE == kModeResidual && a.gain_next && r_ok) gn = *reinterpret_cast<const float4*>(a.gain_next + r0);
                    const uint32_t kv_head_row = (uint32_t)(((w_which > 0 ? w_which - 1 : 0) * a.m.H + w_head) * kPage);
                    ok = mbar_wait(accf0 + 8 * buf, (it / n_acc) & 1, a.status, 13);
                    ok = group_sync_and(1 + grp, ok);                // the four warps go on together or not at all
                    tc_fence_after();
                    if (warp == 2 && lane == 0) SLLM_TL_HERE(503 + MODE * 10);
                    if (split > 1) {                                 // split-K: the peers' accumulators come to block 0 first
                        if (ks > 0 && ok) {
                            const uint32_t base = cluster_map(smem_u32(handover), 0);
                            for (int c0 = cbeg; c0 < cbeg + HALF; c0 += 16) {
                                if (t0 + c0 >= a.n_tok) break;
                                uint32_t v[16];
                                tc_ld16(acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    st_cluster_f32(base + 4u * (uint32_t)(((ks - 1) * BN + c0 + j) * kTcBM + quarter * 32 + lane), __uint_as_float(v[j]));
                            }
                        }
                        cluster_sync_all();                          // every thread of every block of the cluster, exactly once
                    }
                    int chunk = 0;
                    for (int c0 = cbeg; c0 < cbeg + HALF && ok && ks == 0; c0 += 16, ++chunk) {
                        if (t0 + c0 >= a.n_tok) break;               // uniform over the group
                        const int cj = c0 + quarter * 4;             // this warp's four columns after the transposition
                        float4 opnd[4];                              // operands that do not depend on the accumulator
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int tok = t0 + cj + i;
                            const bool valid = r_ok && tok < a.n_tok;
                            if (MODE == kModeResidual)
                                opnd[i] = valid ? *reinterpret_cast<const float4*>(a.out + (size_t)tok * a.R + r0) : make_float4(0.f, 0.f, 0.f, 0.f);
                            else if (MODE == kModeQKV)
                                opnd[i] = (valid && w_which < 2)
                                              ? *reinterpret_cast<const float4*>(a.rope + (size_t)my_pos[cj - cbeg + i] * (hd / 2) + (w_d >> 1))
                                              : make_float4(1.f, 0.f, 1.f, 0.f);
                        }
                        uint32_t v[16];
                        tc_ld16(acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                        for (int p = 0; p + 1 < split; ++p) {        // peers' shares, in rank order
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                v[j] = __float_as_uint(__uint_as_float(v[j]) + handover[((p * BN + c0 + j) * kTcBM) + quarter * 32 + lane]);
                        }
                        float* const sb = stg + (chunk & 1) * 16 * kTcBM;
#pragma unroll
                        for (int j = 0; j < 16; ++j) sb[j * kTcBM + quarter * 32 + lane] = __uint_as_float(v[j]);
                        // One barrier per chunk is enough with two buffers: a warp that writes chunk k + 2 has passed
                        // the barrier of chunk k + 1, which every warp reaches only after its reads of chunk k.
                        group_sync(1 + grp);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int tok = t0 + cj + i;
                            if (tok >= a.n_tok) break;               // uniform over the warp
                            const float4 w = *reinterpret_cast<const float4*>(sb + (quarter * 4 + i) * kTcBM + 4 * lane);
                            if (MODE == kModeResidual) {
                                const float4 r = make_float4(opnd[i].x + w.x, opnd[i].y + w.y, opnd[i].z + w.z, opnd[i].w + w.w);
                                if (r_ok) {
                                    *reinterpret_cast<float4*>(a.out + (size_t)tok * a.R + r0) = r;
                                    if (a.gain_next)
                                        *reinterpret_cast<uint2*>(a.xn_out + (size_t)tok * a.R + r0) =
                                            make_uint2(pack_bf16x2(r.x * gn.x, r.y * gn.y), pack_bf16x2(r.z * gn.z, r.w * gn.w));
                                }
                                if (a.gain_next) {                   // uniform over the grid: the 32-row slices' sums of squares
                                    float sq = r_ok ? (r.x * r.x + r.y * r.y) + (r.z * r.z + r.w * r.w) : 0.f;
                                    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                                    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                                    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                                    if ((lane & 7) == 0) a.ss_out[(size_t)tok * a.n_parts + mi * 4 + (lane >> 3)] = sq;
                                }
                            } else if (MODE == kModeHead) {
                                if (r_ok) *reinterpret_cast<float4*>(a.out + (size_t)tok * a.R + r0) = w;
                            } else if (MODE == kModeGateUp) {        // rows: gate, up, gate, up of two hidden units
                                const float rs = my_rs[cj - cbeg + i];
                                const float g0 = w.x * rs, u0 = w.y * rs, g1 = w.z * rs, u1 = w.w * rs;
                                const float h0 = __fdividef(g0, 1.0f + __expf(-g0)) * u0;
                                const float h1 = __fdividef(g1, 1.0f + __expf(-g1)) * u1;
                                if (r_ok) *reinterpret_cast<uint32_t*>(a.out_bf16 + (size_t)tok * (a.R / 2) + (r0 >> 1)) = pack_bf16x2(h0, h1);
                            } else {                                 // QKV: two RoPE pairs per lane
                                const float rs = my_rs[cj - cbeg + i];
                                float4 r = make_float4(w.x * rs, w.y * rs, w.z * rs, w.w * rs);
                                if (w_which < 2) {
                                    const float4 cs4 = opnd[i];      // cos, sin of the two pairs
                                    r = make_float4(r.x * cs4.x - r.y * cs4.y, r.x * cs4.y + r.y * cs4.x,
                                                    r.z * cs4.z - r.w * cs4.w, r.z * cs4.w + r.w * cs4.z);
                                }
                                if (r_ok) {
                                    if (w_which == 0) *reinterpret_cast<float4*>(a.out + (size_t)tok * D + w_col) = r;
                                    else
                                        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.kv.pool) +
                                                                  (size_t)(my_kvrow[cj - cbeg + i] + kv_head_row) * (uint32_t)hd + w_d) =
                                            make_uint2(pack_bf16x2(r.x, r.y), pack_bf16x2(r.z, r.w));
                                }
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acce0 + 8 * buf) : "memory");
                    continue;
                }
            }
            auto fetch = [&](int c) {                                // operands of columns c .. c + CW - 1
                if (MODE == kModeQKV) {
    #pragma unroll
                    for (int j = 0; j < CW; ++j)
                        cs[j] = (which < 2 && row_ok) ? a.rope[(size_t)my_pos[c - cbeg + j] * (hd / 2) + (d >> 1)] : make_float2(1.f, 0.f);
                } else if (MODE == kModeResidual) {
    #pragma unroll
                    for (int j = 0; j < CW; ++j) {
                        const int tok = t0 + c + j;
                        xv[j] = (row_ok && tok < a.n_tok) ? x_lane[(size_t)((uint32_t)tok * (uint32_t)a.R)] : 0.f;
                    }
                }
            };
            if (ks == 0 && t0 + cbeg < a.n_tok) fetch(cbeg);
            ok = mbar_wait(accf0 + 8 * buf, (it / n_acc) & 1, a.status, 13);
            ok = __all_sync(0xffffffffu, ok);                        // the TMEM loads below need the whole warp
            tc_fence_after();
            if (warp == 2 && lane == 0) SLLM_TL_HERE(503 + MODE * 10);
            if (split > 1) {
                if (ks > 0 && ok) {                                  // hand this block's accumulator to block 0: [peer][column][row]
                    const uint32_t base = cluster_map(smem_u32(handover), 0);
                    for (int c0 = cbeg; c0 < cbeg + HALF; c0 += CW) {
                        if (t0 + c0 >= a.n_tok) break;
                        uint32_t v[CW];
                        tc_ld<CW>(acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
    #pragma unroll
                        for (int j = 0; j < CW; ++j)
                            st_cluster_f32(base + 4u * (uint32_t)(((ks - 1) * BN + c0 + j) * kTcBM + quarter * 32 + lane), __uint_as_float(v[j]));
                    }
                }
                cluster_sync_all();                                  // every thread of every block of the cluster, exactly once
            }
            for (int c0 = cbeg; c0 < cbeg + HALF && ok && ks == 0; c0 += CW) {
                if (t0 + c0 >= a.n_tok) break;                       // uniform over the warp
                const bool more = c0 + CW < cbeg + HALF && t0 + c0 + CW < a.n_tok;
                uint32_t v[CW];
                tc_ld<CW>(acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                for (int p = 0; p + 1 < split; ++p) {                // peers' shares, in rank order
    #pragma unroll
                    for (int j = 0; j < CW; ++j)
                        v[j] = __float_as_uint(__uint_as_float(v[j]) + handover[((p * BN + c0 + j) * kTcBM) + quarter * 32 + lane]);
                }
                if (MODE == kModeResidual) {
                    float r[CW];
    #pragma unroll
                    for (int j = 0; j < CW; ++j) r[j] = xv[j] + __uint_as_float(v[j]);
                    if (more) fetch(c0 + CW);
    #pragma unroll
                    for (int j = 0; j < CW; ++j) {
                        const int tok = t0 + c0 + j;
                        if (row_ok && tok < a.n_tok) {
                            x_lane[(size_t)((uint32_t)tok * (uint32_t)a.R)] = r[j];
                            if (a.gain_next) xn_lane[(size_t)((uint32_t)tok * (uint32_t)a.R)] = __float2bfloat16_rn(r[j] * gnext);
                        }
                    }
                    if (a.gain_next) {                               // uniform over the grid
                        float sq[32];
    #pragma unroll
                        for (int j = 0; j < 32; ++j) sq[j] = (j < CW && row_ok && t0 + c0 + j < a.n_tok) ? r[j < CW ? j : 0] * r[j < CW ? j : 0] : 0.f;
                        const float col = warp_column_sums(sq, lane);
                        const int tok = t0 + c0 + lane;
                        if (lane < CW && tok < a.n_tok) a.ss_out[(size_t)tok * a.n_parts + mi * 4 + quarter] = col;
                    }
                } else if (MODE == kModeHead) {
    #pragma unroll
                    for (int j = 0; j < CW; ++j) {
                        const int tok = t0 + c0 + j;
                        if (row_ok && tok < a.n_tok) x_lane[(size_t)tok * a.R] = __uint_as_float(v[j]);
                    }
                } else if (MODE == kModeGateUp) {
                    // (gate, up) of a hidden unit sit in adjacent lanes.  Two columns per step: the even lane finishes
                    // column j (its own gate, the neighbour's up), the odd lane column j + 1 (the neighbour's gate, its
                    // own up), so one exchange and one SiLU serve two tokens and every lane's result is stored
                    const bool odd = (row & 1) != 0;
                    __nv_bfloat16* const h_lane = a.out_bf16 + (row >> 1);
                    const uint32_t h_stride = (uint32_t)(a.R / 2);
    #pragma unroll
                    for (int j = 0; j < CW; j += 2) {
                        const float a0 = __uint_as_float(v[j]) * my_rs[c0 - cbeg + j];
                        const float a1 = __uint_as_float(v[j + 1]) * my_rs[c0 - cbeg + j + 1];
                        const float recv = __shfl_xor_sync(0xffffffffu, odd ? a0 : a1, 1);
                        const float g = odd ? recv : a0, u = odd ? a1 : recv;
                        const float hval = __fdividef(g, 1.0f + __expf(-g)) * u;
                        const int tok = t0 + c0 + j + (odd ? 1 : 0);
                        if (row_ok && tok < a.n_tok) h_lane[(size_t)((uint32_t)tok * h_stride)] = __float2bfloat16_rn(hval);
                    }
                } else {
                    // RoPE pairs sit in adjacent lanes
                    float r[CW];
    #pragma unroll
                    for (int j = 0; j < CW; ++j) {
                        const float mine = __uint_as_float(v[j]) * my_rs[c0 - cbeg + j];
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                        r[j] = mine;
                        if (which < 2) r[j] = (row & 1) ? (other * cs[j].y + mine * cs[j].x) : (mine * cs[j].x - other * cs[j].y);
                    }
                    if (more) fetch(c0 + CW);
    #pragma unroll
                    for (int j = 0; j < CW; ++j) {
                        const int tok = t0 + c0 + j;
                        if (!row_ok || tok >= a.n_tok) continue;
                        if (which == 0) q_lane[(uint32_t)tok * (uint32_t)D] = r[j];
                        else kv_lane[(size_t)(my_kvrow[c0 - cbeg + j] + kv_lane_row) * (uint32_t)hd] = __float2bfloat16_rn(r[j]);
                    }
                }
            }
            // the accumulator has been read out: the tensor cores may overwrite it (tile after next)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acce0 + 8 * buf) : "memory");
        }
    }
    if (warp == 2 && lane == 0) SLLM_TL_HERE(504 + MODE * 10);
    if (!ok) {                       // a wait gave up: give copies in flight time to land before shared memory goes away
        for (int i = 0; i < 64; ++i) __nanosleep(16384);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(n_acc * BN));
    }
}

// ---- small helper kernels of the tensor-core path ------------------------------------------------------

// First layer of a tensor-core pass: gathers the fp32 embedding rows (src/ops/embedding.cpp:20-44) into the residual
// stream and prepares the first projection's operand in the folded-norm form: bf16(x * gain) and the row's sum of
// squares in part 0 (the other parts 0).
__global__ void __launch_bounds__(256) k_embed_prep(const float* __restrict__ emb, const uint32_t* __restrict__ tok_id,
                                                     const float* __restrict__ gain, float* __restrict__ x_out,
                                                     __nv_bfloat16* __restrict__ xn, float* __restrict__ ss, int D, int n_parts) {
    __shared__ float red[8];
    SLLM_TL(700);
    pdl_wait();
    pdl_launch_dependents();
    const int tok = blockIdx.x;
    const float* src = emb + (size_t)tok_id[tok] * D;
    float sum = 0.f;
    for (int k = threadIdx.x; k < D; k += 256) {
        const float v = src[k];
        x_out[(size_t)tok * D + k] = v;
        xn[(size_t)tok * D + k] = __float2bfloat16_rn(v * gain[k]);
        sum += v * v;
    }
    sum = warp_sum(sum);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x < n_parts) {
        float t = 0.f;
        if (threadIdx.x == 0)
            for (int w = 0; w < 8; ++w) t += red[w];
        ss[(size_t)tok * n_parts + threadIdx.x] = t;
    }
}
// RMSNorm (src/ops/rmsnorm.cpp:38-60) of selected rows to bf16 [n_rows][D]; on layer 0 the row is first
// gathered from the fp32 embedding table and stored as the residual stream.
__global__ void __launch_bounds__(256) k_rmsnorm_bf16(const float* __restrict__ x, const float* __restrict__ gain,
                                                       __nv_bfloat16* __restrict__ out, int D, float eps, const int* row_tok,
                                                       const float* emb, const uint32_t* tok_id, float* x_out) {
    __shared__ float red[8];
    SLLM_TL(700);
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int tok = row_tok ? row_tok[r] : r;
    const float* src = emb ? emb + (size_t)tok_id[tok] * D : x + (size_t)tok * D;
    float ss = 0.f;
    for (int k = threadIdx.x; k < D; k += 256) {
        const float v = src[k];
        ss += v * v;
        if (emb) x_out[(size_t)tok * D + k] = v;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w];
    const float inv = 1.0f / sqrtf(s / (float)D + eps);
    for (int k = threadIdx.x; k < D; k += 256) out[(size_t)r * D + k] = __float2bfloat16_rn(src[k] * inv * gain[k]);
}

__global__ void __launch_bounds__(256) k_f32_to_bf16_rows(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
}

}  // namespace sllm
