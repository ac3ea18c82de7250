// Weight-streaming projections: every pass with fp32 weights, the head of the one-token decode step, and bf16 passes
// when the driver offers no tensor-map encoder (bf16 passes of two and more tokens otherwise take gemm_tc.cuh).
//
// Every projection of the model is y[t][r] = sum_k x[t][k] * W[r][k] with W stored row-per-output
// ("[R][K]", the transpose of the reference's x@W matrices, re-laid-out once at load time), so a
// row is one contiguous run of K weights.  A warp owns RPW adjacent rows, its 32 lanes stride over
// the 16-byte chunks of those rows (coalesced 128-bit loads), the activation vectors of up to NT
// tokens sit in shared memory as fp32, partial sums are combined with warp shuffles.  The work
// that surrounds each projection in the reference is fused in:
//   QKV      : [embedding gather] + RMSNorm prologue; RoPE + paged-KV append epilogue
//              (src/ops/embedding.cpp:20-44, src/ops/rmsnorm.cpp:10-63, src/nn/attention.cpp:61-90,
//               src/ops/rope.cpp:14-79, src/ops/attention.cpp:90-114)
//   Residual : x += in @ W   (out-projection and FFN down-projection with the residual add,
//              src/nn/transformer_ block.cpp:19-31, src/ops/elementwise.cpp:19-55)
//   GateUp   : RMSNorm prologue; silu(gate)*up epilogue (src/nn/swiglu.cpp:37-57,
//              src/ops/elementwise.cpp:57-84,106-132)
//   Head     : final RMSNorm prologue; fp32 logits (src/model.cpp:55-60, src/ops/matmul.cpp:172-199)
#pragma once
#include "common.cuh"

namespace sllm {

enum GemvMode { kModeQKV = 0, kModeResidual = 1, kModeGateUp = 2, kModeHead = 3 };

struct GemvArgs {
    const void* W;            // [R][K]
    int R, K;
    const float* in;          // [n_tok][K] fp32 (x for the norm modes)
    const float* gain;        // [K] RMSNorm gain (norm modes)
    float* out;               // QKV: q [n_tok][D]; Residual: x [n_tok][R]; GateUp: hidden [n_tok][R/2]; Head: logits [n_rows][R]
    int n_tok;                // tokens (Head: rows) handled by this launch
    const int* row_tok;       // Head: pass-token index of each logits row (NULL = identity)
    // QKV only
    ModelDims m;
    KvView kv;
    PassView pass;
    int layer;
    const float2* rope;       // [ctx][hd/2] (cos, sin)
    const float* parts;       // single-token passes: [n_parts][K] partial sums that complete the residual `in`
    int n_parts;
    int prenorm;              // Head: `in` already holds the normalised vector (k_final_norm): no norm here
    const float* emb;         // layer 0: fp32 embedding table [V][D]; x is gathered from it ...
    float* x_out;             // ... and written here by block column 0
    float eps;
};

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;

// PF = 16-byte chunks per lane and row that are fetched into registers BEFORE the kernel waits for its
// predecessor (weights never change during a pass, so this overlaps the predecessor's tail).
template <typename WT, int NT, int MODE, int PF>
__global__ void __launch_bounds__(kGemvThreads) k_gemv(const GemvArgs a) {
    constexpr int EPC = Elems<WT>::per16;
    constexpr int RPW = 2;
    extern __shared__ __align__(16) float xs[];            // [NT][K]
    __shared__ float red[kGemvWarps][NT];
    __shared__ float inv_rms[NT];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = a.K;
    const int t0 = blockIdx.y * NT;
    const int nt = min(NT, a.n_tok - t0);
    const bool kNorm = (MODE != kModeResidual) && !(MODE == kModeHead && a.prenorm);

    // ---- weights of this warp's first row pair: in flight before anything else -------------------
    const int nchunk = K / EPC;
    const int groups = a.R / RPW;
    const int gw = blockIdx.x * kGemvWarps + warp;
    const int gstride = gridDim.x * kGemvWarps;
    const WT* Wt = reinterpret_cast<const WT*>(a.W);
    pdl_launch_dependents();
    uint4 pf0[PF], pf1[PF];
    if (gw < groups) {
        const uint4* w0 = reinterpret_cast<const uint4*>(Wt + (size_t)(gw * RPW) * K);
        const uint4* w1 = reinterpret_cast<const uint4*>(Wt + (size_t)(gw * RPW + 1) * K);
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            const int c = lane + 32 * i;
            if (c < nchunk) { pf0[i] = ldg_stream(w0 + c); pf1[i] = ldg_stream(w1 + c); }
        }
    }
    pdl_wait();
    if (MODE == kModeHead) SLLM_TL(400);

    // ---- prologue: activations to shared memory (+ RMSNorm) ---------------------------------
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        float ss = 0.f;
        if (t < nt) {
            const float* src;
            int ptok = t0 + t;
            if (MODE == kModeHead && a.row_tok) ptok = a.row_tok[t0 + t];
            if (MODE == kModeQKV && a.emb) src = a.emb + (size_t)a.pass.tok_id[ptok] * K;
            else src = a.in + (size_t)ptok * K;
            for (int k = tid * 4; k < K; k += kGemvThreads * 4) {
                float4 v = *reinterpret_cast<const float4*>(src + k);
                for (int p0 = 0; p0 < a.n_parts; p0 += 10) {   // 10 independent loads per round trip; fixed order of adds
                    float4 q[10];
#pragma unroll
                    for (int i = 0; i < 10; ++i)
                        q[i] = (p0 + i < a.n_parts) ? __ldcg(reinterpret_cast<const float4*>(a.parts + (size_t)(p0 + i) * K + k))
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int i = 0; i < 10; ++i) { v.x += q[i].x; v.y += q[i].y; v.z += q[i].z; v.w += q[i].w; }
                }
                *reinterpret_cast<float4*>(xs + t * K + k) = v;
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                if (MODE == kModeQKV && a.emb && blockIdx.x == 0)
                    *reinterpret_cast<float4*>(a.x_out + (size_t)ptok * K + k) = v;
            }
        }
        if (kNorm) {
            ss = warp_sum(ss);
            if (lane == 0) red[warp][t] = ss;
        }
    }
    __syncthreads();
    if (kNorm) {
        if (tid < NT) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kGemvWarps; ++w) s += red[w][tid];
            const float ms = s / (float)K;
            inv_rms[tid] = 1.0f / sqrtf(ms + a.eps);
        }
        __syncthreads();
        for (int i = tid; i < nt * K; i += kGemvThreads) {
            const int t = i / K, k = i - t * K;
            xs[i] = xs[i] * inv_rms[t] * a.gain[k];
        }
        __syncthreads();
    }

    // ---- stream the rows -------------------------------------------------------------------
    for (int g = gw; g < groups; g += gstride) {
        const int r = g * RPW;
        const uint4* w0 = reinterpret_cast<const uint4*>(Wt + (size_t)r * K);
        const uint4* w1 = reinterpret_cast<const uint4*>(Wt + (size_t)(r + 1) * K);
        float acc0[NT], acc1[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) { acc0[t] = 0.f; acc1[t] = 0.f; }
        auto fma_chunk = [&](const uint4& v0, const uint4& v1, int c) {
            float f0[EPC], f1[EPC];
            unpack16<WT>(v0, f0);
            unpack16<WT>(v1, f1);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const float* xv = xs + t * K + c * EPC;
#pragma unroll
                for (int e = 0; e < EPC; e += 4) {
                    const float4 x4 = *reinterpret_cast<const float4*>(xv + e);
                    acc0[t] += f0[e] * x4.x + f0[e + 1] * x4.y + f0[e + 2] * x4.z + f0[e + 3] * x4.w;
                    acc1[t] += f1[e] * x4.x + f1[e + 1] * x4.y + f1[e + 2] * x4.z + f1[e + 3] * x4.w;
                }
            }
        };
        int c_begin = lane;
        if (g == gw) {                       // first pair: the prefetched chunks
#pragma unroll
            for (int i = 0; i < PF; ++i) {
                const int c = lane + 32 * i;
                if (c < nchunk) fma_chunk(pf0[i], pf1[i], c);
            }
            c_begin = lane + 32 * PF;
        }
#pragma unroll 4
        for (int c = c_begin; c < nchunk; c += 32) {
            const uint4 v0 = ldg_stream(w0 + c);
            const uint4 v1 = ldg_stream(w1 + c);
            fma_chunk(v0, v1, c);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) { acc0[t] = warp_sum(acc0[t]); acc1[t] = warp_sum(acc1[t]); }

        // ---- epilogue: lane t finishes token t -----------------------------------------------
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            if (lane != t || t >= nt) continue;
            const float v0 = acc0[t], v1 = acc1[t];
            const int ptok = t0 + t;
            if (MODE == kModeResidual) {
                float* x = a.out + (size_t)ptok * a.R + r;
                x[0] = x[0] + v0;
                x[1] = x[1] + v1;
            } else if (MODE == kModeGateUp) {
                // silu as the reference writes it: g * (1/(1+exp(-g))), then * up
                const float sig = 1.0f / (1.0f + expf(-v0));
                a.out[(size_t)ptok * (a.R / 2) + g] = (v0 * sig) * v1;
            } else if (MODE == kModeHead) {
                float* o = a.out + (size_t)ptok * a.R + r;
                o[0] = v0;
                o[1] = v1;
            } else {   // QKV: rows [0,D) q, [D,2D) k, [2D,3D) v
                const int D = a.m.D, hd = a.m.hd;
                const int which = r / D, col = r - which * D;
                const int head = col / hd, d = col - head * hd;
                const int pos = a.pass.tok_pos[ptok];
                float o0 = v0, o1 = v1;
                if (which < 2) {     // interleaved-pair rotation, src/ops/rope.cpp:60-76
                    const float2 cs = a.rope[(size_t)pos * (hd / 2) + (d >> 1)];
                    o0 = v0 * cs.x - v1 * cs.y;
                    o1 = v0 * cs.y + v1 * cs.x;
                }
                if (which == 0) {
                    float* q = a.out + (size_t)ptok * D + col;
                    q[0] = o0;
                    q[1] = o1;
                } else {
                    const int slot = a.pass.tok_slot[ptok];
                    const int page = a.kv.block_table[(size_t)slot * a.kv.pages_per_seq + pos / kPage];
                    WT* dst = kv_ptr<WT>(a.kv, a.m, a.layer, page, which - 1, head, pos % kPage) + d;
                    dst[0] = from_float<WT>(o0);
                    dst[1] = from_float<WT>(o1);
                }
            }
        }
    }
}

}  // namespace sllm
