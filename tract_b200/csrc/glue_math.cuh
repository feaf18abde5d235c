// Scalar arithmetic shared by the element-wise kernels and by the kernels that fuse them with the activation quantiser.
#pragma once
#include <cuda_runtime.h>

namespace b200kv {

__device__ inline float clamp_keep_nan(float x, float lo, float hi) {  // f32::clamp: a NaN stays a NaN
    return x != x ? x : fminf(fmaxf(x, lo), hi);
}

// linalg/src/generic/sigmoid.rs:11-45
__device__ inline float ssigmoid(float x) {
    x = clamp_keep_nan(x, -18.6f, 18.6f);
    const float x2 = __fmul_rn(x, x);
    float p = -4.433153405e-18f;
    p = __fadd_rn(__fmul_rn(x2, p), 1.169974371e-14f);
    p = __fadd_rn(__fmul_rn(x2, p), -1.875289645e-11f);
    p = __fadd_rn(__fmul_rn(x2, p), 4.257889523e-8f);
    p = __fadd_rn(__fmul_rn(x2, p), 0.00004811817576f);
    p = __fadd_rn(__fmul_rn(x2, p), 0.008163842030f);
    p = __fadd_rn(__fmul_rn(x2, p), 0.2499999971f);
    p = __fmul_rn(p, x);
    float q = 3.922935744e-6f;
    q = __fadd_rn(__fmul_rn(x2, q), 0.001524872358f);
    q = __fadd_rn(__fmul_rn(x2, q), 0.1159886749f);
    q = __fadd_rn(__fmul_rn(x2, q), 1.0f);
    return clamp_keep_nan(__fadd_rn(__fdiv_rn(p, q), 0.5f), 0.f, 1.f);
}

// Threads per row of the RmsNorm kernels.  The sum of squares is a tree over the threads: the fused and the stand-alone
// kernel use the same shape, so they give the same bits.
__host__ __device__ inline int rms_norm_threads(int d) { return d >= 2048 ? 512 : (d >= 512 ? 256 : 128); }

// 1 / sqrt(mean(x^2) + eps) of one row, every thread of the CTA holding its share `ss` of the sum of squares; `part` is
// 32 floats of shared memory.  Returns the value to every thread.
__device__ inline float rms_norm_inv(float ss, float* part, int d, float eps) {
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) part[0] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)d), eps)));
    }
    __syncthreads();
    return part[0];
}

}  // namespace b200kv
