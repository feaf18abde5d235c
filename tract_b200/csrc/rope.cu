// ApplyRope as a stand-alone kernel: out = x * cos + rotate_half(x) * sin (transformers/src/ops/apply_rope.rs:
// 143-176; replaces cuda/src/kernels/cu/nn.cu `apply_rope_nd*`).  The query side of an attention layer goes
// through this; the key side is fused into the cache append (b200kv_append_rope).  Results are bit-identical to
// the CPU op: three separate operations, each rounded to the tensor's type.
#include "internal.h"

namespace b200kv {

struct RopeParams {
    const void *x, *cos, *sin;
    void* out;
    int64_t xs[3], os[3], rb, rs;
    int32_t B, H, S, D, dtype;
};

__global__ void rope_kernel(RopeParams p) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t total = (int64_t)p.B * p.H * p.S * p.D;
    if (idx >= total) return;
    const int ch = (int)(idx % p.D);
    const int64_t row = idx / p.D;
    const int s = (int)(row % p.S), h = (int)((row / p.S) % p.H), b = (int)(row / ((int64_t)p.S * p.H));
    const int esz = dtype_size(p.dtype);
    const uint8_t* xr = (const uint8_t*)p.x + (b * p.xs[0] + h * p.xs[1] + s * p.xs[2]) * esz;
    const uint8_t* cr = (const uint8_t*)p.cos + (b * p.rb + s * p.rs) * esz;
    const uint8_t* sr = (const uint8_t*)p.sin + (b * p.rb + s * p.rs) * esz;
    st_from_f32(p.out, p.dtype, b * p.os[0] + h * p.os[1] + s * p.os[2] + ch, rope_row_elem(xr, cr, sr, p.dtype, p.D, ch));
}

}  // namespace b200kv

using namespace b200kv;

extern "C" int b200kv_rope(const void* x, const int64_t x_strides[3], const void* cos, const void* sin, const int64_t rope_strides[2],
                           void* out, const int64_t out_strides[3], int32_t batch, int32_t n_heads, int32_t n_tokens, int32_t head_dim,
                           int32_t dtype, void* stream) {
    if (!x || !cos || !sin || !out || !x_strides || !rope_strides || !out_strides) return fail("null tensor or strides");
    if (batch < 0 || n_heads <= 0 || n_tokens < 0 || head_dim <= 0) return fail("bad dimensions");
    if (head_dim % 2) return fail("RotateHalf possible only if the most inner dimension (%d) is divisible by 2", head_dim);
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if (x == out) return fail("ApplyRope cannot run in place: every output element reads two input elements");
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) return fail("no CUDA device: b200kv has no CPU fallback");
    RopeParams p{};
    p.x = x, p.cos = cos, p.sin = sin, p.out = out;
    for (int i = 0; i < 3; i++) p.xs[i] = x_strides[i], p.os[i] = out_strides[i];
    p.rb = rope_strides[0], p.rs = rope_strides[1];
    p.B = batch, p.H = n_heads, p.S = n_tokens, p.D = head_dim, p.dtype = dtype;
    const int64_t total = (int64_t)batch * n_heads * n_tokens * head_dim;
    if (total == 0) return B200KV_OK;
    rope_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(p);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}
