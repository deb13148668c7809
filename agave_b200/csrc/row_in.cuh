// The output of a stacked projection as a kernel reads it, row by row.
#pragma once
#include "common.cuh"

namespace {

// The input row of token t: 32-bit partial sums [n_splits, T, W] or the row itself.
template <typename T>
struct RowIn {
    const T* row;              // [T, ld] or null
    long long ld;
    const float* part;         // [n_splits, T, W] or null
    int n_splits;
    long long split_stride;
    int W;
    __device__ __forceinline__ float at(int t, int e) const {
        if (part) {
            float s = 0.f;
            const float* p = part + (size_t)t * W + e;
            for (int sp = 0; sp < n_splits; ++sp) s += p[(size_t)sp * split_stride];
            return s;
        }
        return to_f32(row[(size_t)t * ld + e]);
    }
    // The whole row of token t into shared memory, 32-bit: eight values per thread at a
    // time with all their loads issued before the first is used (a dependent trip to L2 or
    // HBM costs about a microsecond, and a decode step has few rows to hide it behind).
    __device__ __forceinline__ void load(int t, float* buf) const {
        for (int e0 = threadIdx.x; e0 < W; e0 += blockDim.x * 8) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
            if (part) {
                const float* p = part + (size_t)t * W;
#pragma unroll 4
                for (int sp = 0; sp < n_splits; ++sp) {
                    const float* ps = p + (size_t)sp * split_stride;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int e = e0 + i * blockDim.x;
                        if (e < W) v[i] += ps[e];
                    }
                }
            } else {
                const T* r = row + (size_t)t * ld;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int e = e0 + i * blockDim.x;
                    if (e < W) v[i] = to_f32(r[e]);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int e = e0 + i * blockDim.x;
                if (e < W) buf[e] = v[i];
            }
        }
        __syncthreads();
    }
};

}  // namespace
