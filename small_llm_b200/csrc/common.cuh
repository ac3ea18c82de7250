// Shared device-side definitions of the token-loop engine (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sllm {

constexpr int kPage = 64;            // positions per KV page
constexpr int kMaxSplits = 32;       // flash-decode splits per (token, head)

// ---- weight / KV element types -----------------------------------------------------------
// A 16-byte vector of weights: 8 bf16 or 4 fp32.
template <typename T> struct Elems;
template <> struct Elems<__nv_bfloat16> { static constexpr int per16 = 8; };
template <> struct Elems<float> { static constexpr int per16 = 4; };

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    // read-only, streamed once: do not keep the line in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <typename T> __device__ __forceinline__ void unpack16(const uint4& v, float* f);
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& v, float* f) {
    // bf16 -> fp32 is a 16-bit shift
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack16<float>(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_float(float x) { return x; }

// ---- reductions ----------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Programmatic dependent launch: a kernel may start while its predecessor in the stream is
// still running; everything before pdl_wait() must not touch data the predecessor writes.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- bounded mbarrier wait: the one wait loop of every kernel in this library ------------------------------
// A wait polls for kWaitLimitNs of wall-clock time at most (c_wait_limit_ns, two seconds unless the engine was
// created with SLLM_WAIT_LIMIT_MS set); then it gives up and the caller raises the engine's status word, leaves
// its loops, frees what it holds and returns, so that a lost signal ends as an error code on the host
// (SLLM_ERR_DEVICE_WAIT) and never as a hung GPU.
constexpr unsigned long long kWaitLimitNs = 2000000000ull;
__constant__ unsigned long long c_wait_limit_ns = kWaitLimitNs;

__device__ __forceinline__ bool mbar_try_parity(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// false = gave up after limit_ns
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_parity(bar, parity)) return true;
        if (i < 64) continue;
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > limit_ns) return false;
        __nanosleep(32);
    }
}

// ---- optional timeline stamps (debug builds with -DSLLM_TIMELINE only) ------------------------------------
#ifdef SLLM_TIMELINE
__device__ unsigned long long g_tl_buf[1 << 16];
__device__ unsigned int g_tl_n;
__device__ __forceinline__ void tl_stamp(unsigned int id) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        const unsigned int i = atomicAdd(&g_tl_n, 1u);
        if (i < (1u << 15)) { g_tl_buf[2 * i] = id; g_tl_buf[2 * i + 1] = t; }
    }
}
// stamp from whichever thread calls it (block 0 only): for single-thread roles such as an MMA issuer
__device__ __forceinline__ void tl_stamp_here(unsigned int id) {
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        const unsigned int i = atomicAdd(&g_tl_n, 1u);
        if (i < (1u << 15)) { g_tl_buf[2 * i] = id; g_tl_buf[2 * i + 1] = t; }
    }
}
#define SLLM_TL(id) tl_stamp(id)
#define SLLM_TL_HERE(id) tl_stamp_here(id)
// Stamps without a round trip per stamp: thread 0 of the chosen blocks reserves a run of entries once per launch
// (PS_TL_INIT), then every stamp (PS_TL) is two plain stores.
#ifndef SLLM_TL_BLOCKS            /* blocks whose thread 0 stamps: 0 only, or (debugging skew between blocks) 0, 37 and the last */
#define SLLM_TL_BLOCKS 1
#endif
#define PS_TL_INIT(n) unsigned int ps_tl_i = 0, ps_tl_end = 0, ps_tl_tag = 0; \
    if (threadIdx.x == 0 && (blockIdx.x == 0 || (SLLM_TL_BLOCKS > 1 && (blockIdx.x == 37 || blockIdx.x == gridDim.x - 1)))) { \
        ps_tl_i = atomicAdd(&g_tl_n, (unsigned int)(n)); ps_tl_end = ps_tl_i + (n); ps_tl_tag = blockIdx.x * 10000u; }
#define PS_TL(id) do { if (ps_tl_i < ps_tl_end && ps_tl_end <= (1u << 15)) { unsigned long long t_; \
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_)); g_tl_buf[2 * ps_tl_i] = (id) + ps_tl_tag; g_tl_buf[2 * ps_tl_i + 1] = t_; ++ps_tl_i; } } while (0)
#else
#define SLLM_TL(id)
#define SLLM_TL_HERE(id)
#define PS_TL_INIT(n)
#define PS_TL(id)
#endif

// ---- device-side view of the model and of the running sequences ----------------------------
struct LayerW {
    const void* wqkv;     // [3D][D]   rows: q | k | v       (reference: attn.q/k/v, each [D][D] as x@W)
    const void* wo;       // [D][D]    row n = output n      (attn.out transposed)
    const void* wgu;      // [2F][D]   row 2j = gate_j, 2j+1 = up_j
    const void* wd;       // [D][F]    (ffn.down transposed)
    const float* g_attn;  // [D]
    const float* g_ffn;   // [D]
};

struct ModelDims {
    int V, ctx, L, D, H, hd, F;
    float eps;
    float scale;          // 1/sqrt(hd), computed in fp32 like src/ops/attention.cpp:46
};

// Per-pass token list: token i of the pass belongs to slot tok_slot[i] at position tok_pos[i].
struct PfTile { int tok_begin, n_q, slot, pos0; };   // pass tokens [tok_begin, tok_begin+n_q) of one slot at positions pos0..

struct PassView {
    const uint32_t* tok_id;
    const int* tok_slot;
    const int* tok_pos;
    int n_tok;
    const PfTile* tiles;      // prefill passes: runs of consecutive positions, <= 64 queries each (else null)
    int n_tiles;
    const int* order;         // optional permutation, grid index -> pass token, longest context first (else null)
};

struct KvView {
    void* pool;            // [L][n_pages][2][H][kPage][hd]
    const int* block_table;// [max_batch][pages_per_seq]
    long long n_pages;
    int pages_per_seq;
};

template <typename KVT>
__device__ __forceinline__ KVT* kv_ptr(const KvView& kv, const ModelDims& m, int layer, int page, int which,
                                       int head, int slot_in_page) {
    size_t off = ((((size_t)layer * kv.n_pages + page) * 2 + which) * m.H + head) * kPage + slot_in_page;
    return reinterpret_cast<KVT*>(kv.pool) + off * m.hd;
}

}  // namespace sllm
