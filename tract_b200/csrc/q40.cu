// Q4_0 weights x int8-quantised activations: the decode-time linear layers either side of the KV-cache path.
//
// Arithmetic: Q4_0::w4a8_gemm / w4a8_gemv of tract-linalg (linalg/src/frame/block_quant/q4_0.rs:199-310), bit for bit:
// the activation row is quantised per block of 32 (scale = max|a| / 127, codes = round(a / scale) clamped to +-127),
// every (weight block, activation block) pair contributes (dot as f32) * w_scale * a_scale with an exact int32 dot
// product, and the contributions are added to the output in ascending block order.  Replaces the GGML-derived
// cuda/src/kernels/cu/mm_mv_q.cu (`mul_vec_q40_m_*`) and cu/quantize.cu (dispatch: cuda/src/kernels/matmul/mod.rs:481-520),
// whose Q8_1 activation format (f16 scales) gives different bits from the CPU.
//
// Kernel: HBM bound (18 bytes per 32 weights, read once).  The weights are repacked once into tiles of 16 output rows
// x all blocks, [block][16 rows x 16 nibble bytes | 16 f16 scales], so that a tile is one contiguous stream.  One warp
// owns a tile: it pulls the stream through a private ring of cp.async.bulk stages, turns each block into the A operand
// of one mma.sync.m16n8k32 (u8 nibbles x s8 activations -> s32: 16 rows x 8 activation rows of exact dot products;
// the -8 of the nibbles is removed with the block's activation sum), and keeps the 16 x 8 f32 accumulators in the
// C-fragment registers, where consecutive blocks arrive in order -- the order the reference adds them in.
#include "internal.h"

namespace b200kv {

constexpr int QK = 32;                    // block length
constexpr int Q_TILE_ROWS = 16;           // output rows per warp (the M of the MMA)
constexpr int Q_BLOCK_BYTES = 16 * 16 + 16 * 2;  // one block of a tile: 256 nibble bytes + 16 f16 scales
constexpr int Q_STAGE_BLOCKS = 8;
constexpr int Q_STAGE_BYTES = Q_STAGE_BLOCKS * Q_BLOCK_BYTES;  // 2304
constexpr int Q_STAGES = 6;
constexpr int Q_ACT_BLOCK = 2 * 8 * 16 + 8 * 4 + 8 * 4;  // per block and group of 8 activation rows: codes [2 halves][8][16], scales f32 [8], sums i32 [8]
constexpr int Q_HEADER = 256;             // scratch header: the status word

// ---- repack: GGML blocks [n][k/32][18 B] -> tiles ------------------------------------------------------
__global__ void q40_pack_kernel(const uint8_t* __restrict__ blocks, int64_t n, int64_t nb, uint8_t* __restrict__ packed) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // (tile row, block)
    const int64_t n_pad = (n + Q_TILE_ROWS - 1) / Q_TILE_ROWS * Q_TILE_ROWS;
    if (idx >= n_pad * nb) return;
    const int64_t row = idx / nb, b = idx % nb;
    uint8_t* dst = packed + ((row / Q_TILE_ROWS) * nb + b) * Q_BLOCK_BYTES;
    const int rr = (int)(row % Q_TILE_ROWS);
    uint16_t w[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};  // rows past n: scale 0, nibbles 0
    if (row < n) {
        const uint16_t* src = (const uint16_t*)(blocks + (row * nb + b) * 18);  // 18-byte blocks are 2-byte aligned
#pragma unroll
        for (int i = 0; i < 9; i++) w[i] = src[i];
    }
    *(uint16_t*)(dst + 256 + 2 * rr) = w[0];
    uint32_t* q = (uint32_t*)(dst + 16 * rr);
#pragma unroll
    for (int i = 0; i < 4; i++) q[i] = (uint32_t)w[1 + 2 * i] | ((uint32_t)w[2 + 2 * i] << 16);
}

// ---- activation quantiser: one warp per (block, activation row slot) ----------------------------------------------
__global__ void q40_quant_act_kernel(const void* __restrict__ a, int64_t a_stride, int32_t m, int32_t dtype, int64_t nb,
                                     uint8_t* __restrict__ act) {
    const int lane = threadIdx.x & 31;
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t groups = (m + 7) / 8;
    if (wid >= groups * nb * 8) return;
    const int slot = (int)(wid % 8);
    const int64_t b = (wid / 8) % nb, g = wid / (8 * nb);
    const int64_t mi = g * 8 + slot;
    uint8_t* dst = act + (g * nb + b) * Q_ACT_BLOCK;
    float x = 0.f;
    if (mi < m) x = ld_as_f32(a, dtype, mi * a_stride + b * QK + lane);
    float amax = fabsf(x);
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));  // fmaxf ignores a NaN operand, as f32::max does
    amax = fmaxf(0.f, amax);                                                                 // the fold starts from 0: an all-NaN block gives 0
    const float scale = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float r = __fdiv_rn(1.0f, scale);
    const float t = roundf(__fmul_rn(x, r));  // NaN for a NaN input and for inf * 0
    const int q = (t != t) ? 0 : (int)fminf(fmaxf(t, -127.f), 127.f);  // f32::clamp keeps a NaN, the cast to i8 makes it 0
    const int sum = __reduce_add_sync(0xffffffffu, q);
    dst[(lane >> 4) * 128 + slot * 16 + (lane & 15)] = (uint8_t)(int8_t)q;
    if (lane == 0) {
        ((float*)(dst + 256))[slot] = mi < m ? scale : 0.f;
        ((int32_t*)(dst + 288))[slot] = sum;
    }
}

struct Q40Gemm {
    const uint8_t* packed;
    const uint8_t* act;
    float* out;
    int* status;
    int64_t n, nb, out_stride;
    int32_t m;
};

__device__ inline void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid: (tiles, groups of 8 activation rows); one warp per CTA.
__global__ void __launch_bounds__(32) q40_gemm_kernel(Q40Gemm p) {
    __shared__ __align__(128) uint8_t ring[Q_STAGES * Q_STAGE_BYTES];
    __shared__ uint64_t bars[Q_STAGES];
    const int lane = threadIdx.x, r = lane >> 2, c = lane & 3;
    const int64_t tile = blockIdx.x, g = blockIdx.y;
    const uint8_t* wsrc = p.packed + tile * p.nb * Q_BLOCK_BYTES;
    const uint8_t* asrc = p.act + g * p.nb * Q_ACT_BLOCK;
    const int n_stages = (int)((p.nb + Q_STAGE_BLOCKS - 1) / Q_STAGE_BLOCKS);
    auto issue = [&](int s) {  // lane 0 only
        const int64_t b0 = (int64_t)s * Q_STAGE_BLOCKS;
        const uint32_t bytes = (uint32_t)(min((int64_t)Q_STAGE_BLOCKS, p.nb - b0) * Q_BLOCK_BYTES);
        mbar_expect_tx(&bars[s % Q_STAGES], bytes);
        bulk_g2s(ring + (s % Q_STAGES) * Q_STAGE_BYTES, wsrc + b0 * Q_BLOCK_BYTES, bytes, &bars[s % Q_STAGES]);
    };
    if (lane == 0) {
        for (int s = 0; s < Q_STAGES; s++) mbar_init(&bars[s], 1);
        mbar_fence_init();
        for (int s = 0; s < Q_STAGES && s < n_stages; s++) issue(s);
    }
    __syncwarp();
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // (row r, act 2c), (r, 2c + 1), (r + 8, 2c), (r + 8, 2c + 1)
    bool failed = false;
    for (int s = 0; s < n_stages && !failed; s++) {
        const int64_t b0 = (int64_t)s * Q_STAGE_BLOCKS;
        const int nblk = (int)min((int64_t)Q_STAGE_BLOCKS, p.nb - b0);
        // this stage's activation fragments come straight from L2 and do not depend on the accumulators: fetch them all first
        uint32_t bq[Q_STAGE_BLOCKS][2];
        float2 asc[Q_STAGE_BLOCKS];
        int2 asum[Q_STAGE_BLOCKS];
#pragma unroll
        for (int j = 0; j < Q_STAGE_BLOCKS; j++) {
            if (j < nblk) {
                const uint8_t* ab = asrc + (b0 + j) * Q_ACT_BLOCK;
                bq[j][0] = __ldg((const uint32_t*)(ab + r * 16 + 4 * c));        // activation row r, elements 4c .. 4c+3
                bq[j][1] = __ldg((const uint32_t*)(ab + 128 + r * 16 + 4 * c));  // elements 16 + 4c ..
                asc[j] = __ldg((const float2*)(ab + 256) + c);
                asum[j] = __ldg((const int2*)(ab + 288) + c);
            }
        }
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bars[s % Q_STAGES], (uint32_t)((s / Q_STAGES) & 1)))) {
            failed = true;
            break;
        }
        const uint8_t* st = ring + (s % Q_STAGES) * Q_STAGE_BYTES;
#pragma unroll
        for (int j = 0; j < Q_STAGE_BLOCKS; j++) {
            if (j < nblk) {
                const uint8_t* wb = st + j * Q_BLOCK_BYTES;
                // bytes 4c .. 4c+3 of a row's 16: low nibbles = elements 4c .. 4c+3, high nibbles = elements 16 + 4c ..
                const uint32_t wa = *(const uint32_t*)(wb + r * 16 + 4 * c), wc = *(const uint32_t*)(wb + (r + 8) * 16 + 4 * c);
                const uint32_t a[4] = {wa & 0x0f0f0f0fu, wc & 0x0f0f0f0fu, (wa >> 4) & 0x0f0f0f0fu, (wc >> 4) & 0x0f0f0f0fu};
                int d[4] = {0, 0, 0, 0};
                mma_u8s8(d, a, bq[j][0], bq[j][1]);
                const float wsA = __half2float(*(const __half*)(wb + 256 + 2 * r)), wsB = __half2float(*(const __half*)(wb + 256 + 2 * (r + 8)));
                // (dot as f32) * w_scale * a_scale, then +=, each operation rounded on its own
                acc[0] = __fadd_rn(acc[0], __fmul_rn(__fmul_rn((float)(d[0] - 8 * asum[j].x), wsA), asc[j].x));
                acc[1] = __fadd_rn(acc[1], __fmul_rn(__fmul_rn((float)(d[1] - 8 * asum[j].y), wsA), asc[j].y));
                acc[2] = __fadd_rn(acc[2], __fmul_rn(__fmul_rn((float)(d[2] - 8 * asum[j].x), wsB), asc[j].x));
                acc[3] = __fadd_rn(acc[3], __fmul_rn(__fmul_rn((float)(d[3] - 8 * asum[j].y), wsB), asc[j].y));
            }
        }
        __syncwarp();  // every lane is done with the stage
        if (lane == 0 && s + Q_STAGES < n_stages) issue(s + Q_STAGES);
    }
    if (failed) {
        if (lane == 0) atomicOr(p.status, STATUS_WAIT_EXPIRED);
        __nanosleep(200000);  // copies that may still be in flight land before the CTA's memory is released
        acc[0] = acc[1] = acc[2] = acc[3] = __int_as_float(0x7fc00000);
    }
    const int64_t row = tile * Q_TILE_ROWS + r, m0 = g * 8 + 2 * c;
    if (row < p.n) {
        if (m0 < p.m) p.out[m0 * p.out_stride + row] = acc[0];
        if (m0 + 1 < p.m) p.out[(m0 + 1) * p.out_stride + row] = acc[1];
    }
    if (row + 8 < p.n) {
        if (m0 < p.m) p.out[m0 * p.out_stride + row + 8] = acc[2];
        if (m0 + 1 < p.m) p.out[(m0 + 1) * p.out_stride + row + 8] = acc[3];
    }
}

}  // namespace b200kv

using namespace b200kv;

extern "C" int64_t b200kv_q40_packed_bytes(int64_t n, int64_t k) {
    if (n <= 0 || k <= 0 || k % QK) return -1;
    return (n + Q_TILE_ROWS - 1) / Q_TILE_ROWS * (k / QK) * Q_BLOCK_BYTES;
}

extern "C" int64_t b200kv_q40_scratch_bytes(int64_t k, int32_t m) {
    if (m <= 0 || k <= 0 || k % QK) return -1;
    return Q_HEADER + (int64_t)((m + 7) / 8) * (k / QK) * Q_ACT_BLOCK;
}

extern "C" int b200kv_q40_pack(const void* blocks, int64_t n, int64_t k, void* packed, void* stream) {
    if (!blocks || !packed) return fail("null pointer");
    if (n <= 0 || k <= 0 || k % QK) return fail("Q4_0 weights need K a multiple of %d, got %lld", QK, (long long)k);
    if ((uintptr_t)blocks % 2 || (uintptr_t)packed % 16) return fail("blocks must be 2-byte aligned and the packed buffer 16-byte aligned");
    const int64_t nb = k / QK, total = (n + Q_TILE_ROWS - 1) / Q_TILE_ROWS * Q_TILE_ROWS * nb;
    q40_pack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)blocks, n, nb, (uint8_t*)packed);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

extern "C" int b200kv_q40_gemm(const void* packed, int64_t n, int64_t k, const void* a, int64_t a_stride, int32_t m, int32_t dtype,
                               void* scratch, float* out, int64_t out_stride, void* stream_) {
    if (!packed || !a || !scratch || !out) return fail("null pointer");
    if (n <= 0 || k <= 0 || k % QK) return fail("W4A8 GEMM needs K a multiple of %d, got %lld", QK, (long long)k);
    if (m <= 0) return fail("m must be positive");
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if ((uintptr_t)packed % 16 || (uintptr_t)scratch % 16) return fail("packed weights and scratch must be 16-byte aligned");
    if (a_stride < k || out_stride < n) return fail("strides shorter than the rows");
    cudaStream_t stream = (cudaStream_t)stream_;
    const int64_t nb = k / QK, groups = (m + 7) / 8;
    uint8_t* act = (uint8_t*)scratch + Q_HEADER;
    B200KV_CUDA(cudaMemsetAsync(scratch, 0, 4, stream));
    const int64_t warps = groups * nb * 8;
    q40_quant_act_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(a, a_stride, m, dtype, nb, act);
    B200KV_CUDA(cudaGetLastError());
    Q40Gemm p{};
    p.packed = (const uint8_t*)packed, p.act = act, p.out = out, p.status = (int*)scratch;
    p.n = n, p.nb = nb, p.out_stride = out_stride, p.m = m;
    dim3 grid((unsigned)((n + Q_TILE_ROWS - 1) / Q_TILE_ROWS), (unsigned)groups);
    q40_gemm_kernel<<<grid, 32, 0, stream>>>(p);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

extern "C" int b200kv_q40_check(const void* scratch, void* stream) {
    if (!scratch) return fail("null pointer");
    int st = 0;
    B200KV_CUDA(cudaMemcpyAsync(&st, scratch, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    B200KV_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (st & STATUS_WAIT_EXPIRED) return fail("a bounded wait in the Q4_0 GEMM kernel expired (a bulk copy never landed)");
    return B200KV_OK;
}
