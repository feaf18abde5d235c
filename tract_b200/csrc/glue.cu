// The element-wise and row-wise ops that sit between the linear layers and the attention of a decoder block:
// RmsNorm, SiLU(gate) * up, residual add, greedy argmax, embedding gather.  Small, HBM / launch bound.
//
//   RmsNorm   core/src/ops/nn/rms_norm.rs:28-66 -> tract-linalg rms_norm_f32 (generic: linalg/src/generic/rms_norm.rs:7-18):
//             out_i = x_i * (1 / sqrt(mean(x^2) + eps)), f32 arithmetic whatever the tensor type; replaces
//             cuda/src/kernels/cu/nn.cu `rms_norm_*`.  The sum of squares is a tree here and a left-to-right fold there:
//             equal to the reference's own tolerance (1e-5), not bit for bit.  The optional weight is the Mul that follows
//             RmsNorm in the graph, fused.
//   SiLU      x * sigmoid(x) with tract-linalg's generic rational sigmoid (linalg/src/generic/sigmoid.rs:11-45, silu.rs:26-30),
//             every operation rounded on its own, in the reference's order: bit for bit in f32.  The product with `up` is
//             the Mul that follows in the graph (cu/element_wise.cu, cu/binary.cu).
//   argmax    first index of the row maximum (core/src/ops/nn/reduce.rs ArgMax { last: false }).
#include "glue_math.cuh"
#include "internal.h"

namespace b200kv {

// One CTA per row.
__global__ void rms_norm_kernel(const void* __restrict__ x, int64_t x_stride, const void* __restrict__ w, void* __restrict__ out,
                                int64_t out_stride, int d, float eps, int dtype) {
    __shared__ float part[32];
    const int64_t row = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = ld_as_f32(x, dtype, row * x_stride + i);
        ss = fmaf(v, v, ss);
    }
    const float inv = rms_norm_inv(ss, part, d, eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = __fmul_rn(ld_as_f32(x, dtype, row * x_stride + i), inv);
        if (w) v = __fmul_rn(round_to_dtype(v, dtype), ld_as_f32(w, dtype, i));  // RmsNorm's result is a tensor of `dtype` before the Mul
        st_from_f32(out, dtype, row * out_stride + i, v);
    }
}

__global__ void silu_mul_kernel(const void* __restrict__ gate, const void* __restrict__ up, void* __restrict__ out, int64_t n, int dtype) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = ld_as_f32(gate, dtype, i);
    float s = round_to_dtype(__fmul_rn(g, ssigmoid(g)), dtype);  // Silu's output tensor
    if (up) s = __fmul_rn(s, ld_as_f32(up, dtype, i));
    st_from_f32(out, dtype, i, s);
}

__global__ void add_kernel(const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ out, int64_t n, int dtype) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) st_from_f32(out, dtype, i, __fadd_rn(ld_as_f32(a, dtype, i), ld_as_f32(b, dtype, i)));
}

// One CTA per row; ties go to the smallest index; a NaN never wins (f32 partial order: `>` is false for it).
__global__ void argmax_kernel(const float* __restrict__ x, int64_t stride, int n, int32_t* __restrict__ out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = x + (int64_t)blockIdx.x * stride;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    auto take = [&](float v, int i) {
        if (v > best || (v == best && i < idx)) best = v, idx = i;
    };
    if (((uintptr_t)row & 15) == 0) {  // 16-byte loads, four of them in flight per thread
        const float4* r4 = (const float4*)row;
        const int n4 = n / 4;
        for (int i = threadIdx.x; i < n4; i += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int k = i + u * blockDim.x;
                v[u] = k < n4 ? r4[k] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int k = i + u * blockDim.x;
                if (k < n4) take(v[u].x, 4 * k), take(v[u].y, 4 * k + 1), take(v[u].z, 4 * k + 2), take(v[u].w, 4 * k + 3);
            }
        }
        for (int i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) take(row[i], i);
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) take(row[i], i);
    }
    auto merge = [&](float ov, int oi) {
        if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
    };
#pragma unroll
    for (int o = 16; o; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if ((threadIdx.x & 31) == 0) bv[threadIdx.x >> 5] = best, bi[threadIdx.x >> 5] = idx;
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < (blockDim.x >> 5) ? bv[threadIdx.x] : -INFINITY;
        idx = threadIdx.x < (blockDim.x >> 5) ? bi[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
        if (threadIdx.x == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;  // a row of -inf / NaN only: index 0
    }
}

__global__ void gather_rows_kernel(const uint8_t* __restrict__ table, const int32_t* __restrict__ ids, uint8_t* __restrict__ out,
                                   int64_t row_bytes, int64_t n_rows_table) {
    const int64_t r = blockIdx.x;
    int64_t id = ids[r];
    if (id < 0 || id >= n_rows_table) id = 0;
    const uint4* src = (const uint4*)(table + id * row_bytes);
    uint4* dst = (uint4*)(out + r * row_bytes);
    for (int64_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) dst[i] = src[i];
}

__global__ void cast2d_kernel(const void* __restrict__ src, int64_t src_stride, int src_dtype, void* __restrict__ dst, int64_t dst_stride,
                              int dst_dtype, int64_t rows, int64_t cols) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * cols) return;
    const int64_t r = i / cols, c = i % cols;
    st_from_f32(dst, dst_dtype, r * dst_stride + c, ld_as_f32(src, src_dtype, r * src_stride + c));
}

}  // namespace b200kv

using namespace b200kv;

static int check_dtype(int dtype) { return (dtype < B200KV_F32 || dtype > B200KV_BF16) ? fail("unknown dtype %d", dtype) : B200KV_OK; }

extern "C" int b200kv_rms_norm(const void* x, int64_t x_stride, const void* weight, void* out, int64_t out_stride, int64_t rows, int32_t d,
                               float eps, int32_t dtype, void* stream) {
    if (!x || !out) return fail("null tensor");
    if (rows <= 0 || d <= 0) return fail("rows and d must be positive");
    if (check_dtype(dtype) != B200KV_OK) return B200KV_KO;
    const int threads = rms_norm_threads(d);
    rms_norm_kernel<<<(unsigned)rows, threads, 0, (cudaStream_t)stream>>>(x, x_stride, weight, out, out_stride, d, eps, dtype);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

extern "C" int b200kv_silu_mul(const void* gate, const void* up, void* out, int64_t n, int32_t dtype, void* stream) {
    if (!gate || !out) return fail("null tensor");
    if (n <= 0) return fail("n must be positive");
    if (check_dtype(dtype) != B200KV_OK) return B200KV_KO;
    silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gate, up, out, n, dtype);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

extern "C" int b200kv_add(const void* a, const void* b, void* out, int64_t n, int32_t dtype, void* stream) {
    if (!a || !b || !out) return fail("null tensor");
    if (n <= 0) return fail("n must be positive");
    if (check_dtype(dtype) != B200KV_OK) return B200KV_KO;
    add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, b, out, n, dtype);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

extern "C" int b200kv_argmax(const float* x, int64_t stride, int64_t rows, int32_t n, int32_t* out, void* stream) {
    if (!x || !out) return fail("null tensor");
    if (rows <= 0 || n <= 0) return fail("rows and n must be positive");
    argmax_kernel<<<(unsigned)rows, 1024, 0, (cudaStream_t)stream>>>(x, stride, n, out);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

extern "C" int b200kv_gather_rows(const void* table, int64_t n_rows_table, int64_t row_bytes, const int32_t* ids, int64_t n_ids, void* out,
                                  void* stream) {
    if (!table || !ids || !out) return fail("null tensor");
    if (row_bytes <= 0 || row_bytes % 16 || (uintptr_t)table % 16 || (uintptr_t)out % 16) return fail("rows must be 16-byte multiples, 16-byte aligned");
    if (n_ids <= 0) return fail("n_ids must be positive");
    gather_rows_kernel<<<(unsigned)n_ids, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)table, ids, (uint8_t*)out, row_bytes, n_rows_table);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

extern "C" int b200kv_cast(const void* src, int64_t src_stride, int32_t src_dtype, void* dst, int64_t dst_stride, int32_t dst_dtype,
                           int64_t rows, int64_t cols, void* stream) {
    if (!src || !dst) return fail("null tensor");
    if (rows <= 0 || cols <= 0) return fail("rows and cols must be positive");
    if (check_dtype(src_dtype) != B200KV_OK || check_dtype(dst_dtype) != B200KV_OK) return B200KV_KO;
    const int64_t n = rows * cols;
    cast2d_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(src, src_stride, src_dtype, dst, dst_stride, dst_dtype, rows, cols);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}
