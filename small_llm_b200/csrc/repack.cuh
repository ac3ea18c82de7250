// Load-time conversion of the reference's fp32 parameters into the engine's layouts
// (the counterpart of Model::refresh_bf16_weights, src/model.cpp:151-158, which casts each
// matrix to bf16; here the cast is fused with the re-layout).
#pragma once
#include "common.cuh"

namespace sllm {

// src fp32 [K][N] (the reference's x@W layout) -> dst[(n*row_mul + row_add)][k], i.e. one
// contiguous row of K weights per output feature.  32x32 tiles through shared memory.
template <typename WT>
__global__ void k_repack_transpose(const float* __restrict__ src, WT* __restrict__ dst, int K, int N,
                                   int row_mul, int row_add) {
    __shared__ float tile[32][33];
    const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int k = k0 + i, n = n0 + threadIdx.x;
        tile[i][threadIdx.x] = (k < K && n < N) ? src[(size_t)k * N + n] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int n = n0 + i, k = k0 + threadIdx.x;
        if (n < N && k < K) dst[((size_t)n * row_mul + row_add) * K + k] = from_float<WT>(tile[threadIdx.x][i]);
    }
}

// plain cast, same layout (embedding [V][D], which already is one row per output of the tied head)
template <typename WT>
__global__ void k_cast(const float* __restrict__ src, WT* __restrict__ dst, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = from_float<WT>(src[i]);
}

}  // namespace sllm
