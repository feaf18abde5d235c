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
// x all blocks, [block][16 rows x 16 nibble bytes | 16 f16 scales], so that a tile is one contiguous stream.  A CTA
// owns a tile and its warps take turns at the stages of 8 blocks: a warp pulls its stage, and the quantised activations
// beside it (L2 resident, shared by every tile), through cp.async.bulk, turns each block into the A operand
// of one mma.sync.m16n8k32 (u8 nibbles x s8 activations -> s32: 16 rows x 8 activation rows of exact dot products;
// the -8 of the nibbles and the int -> f32 conversion are one exact float addition, see q40_common.cuh; the two
// multiplications and the addition of a contribution are the packed f32x2 instructions, each lane rounded as the scalar
// ones are), and adds the 8 contributions to the 16 x 8 f32 accumulators, which travel from warp to warp in stage order -- the order the reference adds the blocks in.
#include <type_traits>

#include "glue_math.cuh"
#include "internal.h"
#include "f32x2.cuh"
#include "q40_common.cuh"

namespace b200kv {

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

// ---- activation quantisers --------------------------------------------------------------------------------------
// One warp per (block, activation row slot).  With `up`, the value quantised is Silu(a) * up (the gate of a gated FFN), each
// of the two ops rounded to `dtype` as the stand-alone kernels round them.
__global__ void q40_quant_act_kernel(const void* __restrict__ a, int64_t a_stride, const void* __restrict__ up, int64_t up_stride, int32_t m,
                                     int32_t dtype, int64_t nb, uint8_t* __restrict__ act, int* __restrict__ status) {
    grid_launch_dependents();  // the GEMM may be scheduled: it starts pulling weights and waits for this grid before it reads `act`
    grid_dependency_wait();    // the kernel before has written the activation (and has finished with `act`, if it was a GEMM)
    if (blockIdx.x == 0 && threadIdx.x == 0) q40_status_begin(status);
    const int lane = threadIdx.x & 31;
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t groups = (m + 7) / 8;
    if (wid >= groups * nb * 8) return;
    const int slot = (int)(wid % 8);
    const int64_t b = (wid / 8) % nb, g = wid / (8 * nb);
    const int64_t mi = g * 8 + slot;
    float x = 0.f;
    if (mi < m) {
        x = ld_as_f32(a, dtype, mi * a_stride + b * QK + lane);
        if (up) {
            const float s = round_to_dtype(__fmul_rn(x, ssigmoid(x)), dtype);
            x = round_to_dtype(__fmul_rn(s, ld_as_f32(up, dtype, mi * up_stride + b * QK + lane)), dtype);
        }
    }
    q40_quantize_block(x, mi < m, act, m, nb, mi, b, lane);
}

// One CTA per activation row slot: v = x (+ residual), stored to x_out when given; then RmsNorm(v) * weight, quantised.
// The same arithmetic, in the same order, as the add, RmsNorm and quantiser kernels run one after the other.  A thread
// keeps its EPT values of the row (elements tid, tid + threads, ...) in registers: every load of the row is in flight at
// once, and the second pass reads nothing but the weight (from L2).
template <int EPT>
__global__ void __launch_bounds__(512) q40_norm_quant_kernel(const float* x, int64_t x_stride, const float* residual, int64_t res_stride,
                                      const float* __restrict__ weight, float eps, float* x_out, int64_t xo_stride, int32_t m, int d,
                                      uint8_t* __restrict__ act, int* __restrict__ status) {
    __shared__ float part[32];
    grid_launch_dependents();
    constexpr int WPT = EPT <= 8 ? EPT : 1;  // short rows: the weights wait in registers, fetched while the kernel before drains
    float w[WPT];
    if (EPT <= 8) {
#pragma unroll
        for (int j = 0; j < WPT; j++) {
            const int i = threadIdx.x + j * blockDim.x;
            w[j] = (weight && i < d) ? weight[i] : 1.f;
        }
    }
    grid_dependency_wait();  // the kernel before (the GEMM that wrote `residual`, and read `act`) is done
    if (blockIdx.x == 0 && threadIdx.x == 0) q40_status_begin(status);
    const int64_t mi = blockIdx.x, nb = d / QK;
    const int lane = threadIdx.x & 31;
    const bool valid = mi < m;
    float v[EPT];
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        v[j] = (valid && i < d) ? x[mi * x_stride + i] : 0.f;
    }
    if (residual) {
        float r[EPT];
#pragma unroll
        for (int j = 0; j < EPT; j++) {
            const int i = threadIdx.x + j * blockDim.x;
            r[j] = (valid && i < d) ? residual[mi * res_stride + i] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < EPT; j++) v[j] = __fadd_rn(v[j], r[j]);
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        if (valid && i < d) {
            if (x_out) x_out[mi * xo_stride + i] = v[j];
            ss = fmaf(v[j], v[j], ss);  // ascending j: the order of the stand-alone kernel's loop
        }
    }
    const float inv = rms_norm_inv(ss, part, d, eps);
#pragma unroll
    for (int j = 0; j < EPT; j++) {  // d and the CTA are multiples of 32: a warp covers one block per turn
        const int i = threadIdx.x + j * blockDim.x;
        if (i < d) {
            float t = __fmul_rn(v[j], inv);
            if (weight) t = __fmul_rn(t, EPT <= 8 ? w[j < WPT ? j : 0] : weight[i]);
            q40_quantize_block(t, valid, act, m, nb, mi, i / QK, lane);
        }
    }
}

struct Q40Gemm {
    const uint8_t* packed;
    const uint8_t* act;
    void* out;  // [m][n] of out_dtype: the f32 result, rounded once on the way out when the type is narrower
    int* status;
    int64_t n, nb, out_stride;
    int32_t m, out_dtype;
    float one;  // 1.0f, see f2_accumulate
};

// D = A . B + c in every accumulator: 16 rows x 8 activation rows of exact dot products on top of the start value.
__device__ inline void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, int c) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c));
}

// acc + t as fma(t, 1, acc) with a 1 the compiler cannot see through (a kernel parameter): the assembler was seen to
// contract mul.rn.f32x2 followed by add.rn.f32x2 into one fused multiply-add, which rounds once where the reference
// rounds twice; a product that feeds the multiplicand of an fma cannot be contracted into it.
__device__ inline uint64_t f2_accumulate(uint64_t acc, uint64_t t, uint64_t one2) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(t), "l"(one2), "l"(acc));
    return r;
}
// The contributions of one block to two accumulators (one weight row, activation rows 2c and 2c + 1):
// (dot as f32) * w_scale * a_scale, each operation rounded on its own.  d0, d1: finished MMA accumulators (started at
// Q_F32_INT_BASE); par = {a_scale of the two rows, their offset terms}.
__device__ inline uint64_t q40_contribution(int d0, int d1, uint64_t w_scale2, const float4& par) {
    const uint64_t dot = f2_add(f2_pack_bits((uint32_t)d0, (uint32_t)d1), f2_pack(par.z, par.w));
    return f2_mul(f2_mul(dot, w_scale2), f2_pack(par.x, par.y));
}

// Waits for a barrier phase unless the CTA has already failed; gives up after ~1 s and marks the CTA failed.
__device__ inline void q40_wait(uint64_t* bar, uint32_t parity, volatile int* fail) {
    if (mbar_try_wait(bar, parity)) return;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        if (*fail) return;
#pragma unroll 1
        for (int i = 0; i < 32; i++)
            if (mbar_try_wait(bar, parity)) return;
        if (globaltimer_ns() - t0 > 1000000000ull) {
            *fail = 1;
            return;
        }
    }
}
__device__ inline void q40_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// grid: (tiles, groups of 8 activation rows); Q_WARPS warps per tile.  Warp w takes the stages s = w, w + Q_WARPS, ...:
// it computes the 8 x (16 x 8) contributions of its stage on its own, then receives the running accumulators from the
// warp that had stage s - 1, adds its contributions in block order and hands the accumulators on.  Only that short
// hand-off is serial; it keeps the additions in the order of the reference.
// MG > 1 (more than 8 activation rows): a CTA keeps each weight stage for MG groups of 8 rows; every group has its own
// chain of hand-offs, so the warps work as a wavefront over (stage, group).
template <int Q_WARPS, int MG>
__global__ void __launch_bounds__(Q_WARPS * 32, MG == 1 ? 2 : 1) q40_gemm_kernel(Q40Gemm p) {
    constexpr int STAGE = Q_STAGE_BYTES + MG * Q_STAGE_BLOCKS * Q_ACT_BLOCK;  // weights, then the activations of each group
    extern __shared__ __align__(128) uint8_t ring[];                      // Q_WARPS * Q_DEPTH stages; warp w owns slots w * Q_DEPTH ..
    float4* hand = (float4*)(ring + Q_WARPS * Q_DEPTH * STAGE);           // [Q_WARPS][MG][32 lanes]: accumulators on their way to warp w
    uint64_t* full = (uint64_t*)(hand + Q_WARPS * MG * 32);               // [Q_WARPS * Q_DEPTH] bytes landed
    uint64_t* token = full + Q_WARPS * Q_DEPTH;                           // [Q_WARPS][MG] accumulators handed to warp w
    volatile int* fail_s = (volatile int*)(token + Q_WARPS * MG);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, c = lane & 3;
    const int64_t tile = blockIdx.x, g0 = (int64_t)blockIdx.y * MG;
    const int ng = (int)min((int64_t)MG, (p.m + 7) / 8 - g0);             // groups of 8 activation rows this CTA has
    const uint8_t* wsrc = p.packed + tile * p.nb * Q_BLOCK_BYTES;
    const uint8_t* asrc = p.act + g0 * p.nb * Q_ACT_BLOCK;
    const int n_stages = (int)((p.nb + Q_STAGE_BLOCKS - 1) / Q_STAGE_BLOCKS);
    // stage s lives in slot (s % Q_WARPS) * Q_DEPTH + (s / Q_WARPS) % Q_DEPTH
    auto slot_of = [&](int s) { return (s % Q_WARPS) * Q_DEPTH + (s / Q_WARPS) % Q_DEPTH; };
    auto issue = [&](int s, bool weights, bool acts) {  // one lane of the owning warp
        const int64_t b0 = (int64_t)s * Q_STAGE_BLOCKS;
        const uint32_t nblk = (uint32_t)min((int64_t)Q_STAGE_BLOCKS, p.nb - b0);
        const int sl = slot_of(s);
        uint8_t* dst = ring + sl * STAGE;
        if (weights) {
            mbar_expect_tx(&full[sl], nblk * (Q_BLOCK_BYTES + ng * Q_ACT_BLOCK));
            bulk_g2s(dst, wsrc + b0 * Q_BLOCK_BYTES, nblk * Q_BLOCK_BYTES, &full[sl]);
        }
        if (acts)
            for (int gi = 0; gi < ng; gi++)
                bulk_g2s(dst + Q_STAGE_BYTES + gi * Q_STAGE_BLOCKS * Q_ACT_BLOCK, asrc + (gi * p.nb + b0) * Q_ACT_BLOCK, nblk * Q_ACT_BLOCK,
                         &full[sl]);
    };
    if (tid == 0) {
        for (int i = 0; i < Q_WARPS * Q_DEPTH; i++) mbar_init(&full[i], 1);
        for (int i = 0; i < Q_WARPS * MG; i++) mbar_init(&token[i], 1);
        *fail_s = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (lane == 0)  // the weights do not depend on the launch before: start pulling them
        for (int d = 0; d < Q_DEPTH; d++)
            if (warp + d * Q_WARPS < n_stages) issue(warp + d * Q_WARPS, true, false);
    grid_launch_dependents();  // whatever consumes the result may be scheduled and do its own set-up; it waits for this grid before it reads
    grid_dependency_wait();    // the activation quantiser has finished
    if (lane == 0)
        for (int d = 0; d < Q_DEPTH; d++)
            if (warp + d * Q_WARPS < n_stages) issue(warp + d * Q_WARPS, false, true);
    __syncwarp();

    for (int s = warp; s < n_stages; s += Q_WARPS) {
        const int turn = s / Q_WARPS;  // how many stages this warp has had before
        const int64_t b0 = (int64_t)s * Q_STAGE_BLOCKS;
        const int nblk = (int)min((int64_t)Q_STAGE_BLOCKS, p.nb - b0);
        const int sl = slot_of(s);
        q40_wait(&full[sl], (uint32_t)((turn / Q_DEPTH) & 1), fail_s);
        const uint8_t* st = ring + sl * STAGE;
        // Passes over the blocks of the stage, so that the loads, the MMAs and the conversions of different blocks overlap.
        uint32_t af[Q_STAGE_BLOCKS][4];
        uint64_t wsA[Q_STAGE_BLOCKS], wsB[Q_STAGE_BLOCKS];  // the block's scale of weight rows r and r + 8, in both lanes of a pair
#pragma unroll
        for (int j = 0; j < Q_STAGE_BLOCKS; j++) {
            const uint8_t* wb = st + j * Q_BLOCK_BYTES;
            // bytes 4c .. 4c+3 of a row's 16: low nibbles = elements 4c .. 4c+3, high nibbles = elements 16 + 4c ..
            const uint32_t wa = *(const uint32_t*)(wb + r * 16 + 4 * c), wc = *(const uint32_t*)(wb + (r + 8) * 16 + 4 * c);
            af[j][0] = wa & 0x0f0f0f0fu, af[j][1] = wc & 0x0f0f0f0fu, af[j][2] = (wa >> 4) & 0x0f0f0f0fu, af[j][3] = (wc >> 4) & 0x0f0f0f0fu;
            const float sa = __half2float(*(const __half*)(wb + 256 + 2 * r)), sb = __half2float(*(const __half*)(wb + 256 + 2 * (r + 8)));
            wsA[j] = f2_pack(sa, sa), wsB[j] = f2_pack(sb, sb);
        }
#pragma unroll 1
        for (int gi = 0; gi < ng; gi++) {
            uint2 bf[Q_STAGE_BLOCKS];
            float4 par[Q_STAGE_BLOCKS];
#pragma unroll
            for (int j = 0; j < Q_STAGE_BLOCKS; j++) {
                const uint8_t* ab = st + Q_STAGE_BYTES + (gi * Q_STAGE_BLOCKS + j) * Q_ACT_BLOCK;
                bf[j] = *(const uint2*)(ab + lane * 8);                          // activation row r: elements 4c .. 4c+3 | 16 + 4c ..
                par[j] = *(const float4*)(ab + Q_ACT_PARAMS + c * 16);           // activation rows 2c, 2c + 1: scales, offset terms
            }
            int d[Q_STAGE_BLOCKS][4];
#pragma unroll
            for (int j = 0; j < Q_STAGE_BLOCKS; j++) mma_u8s8(d[j], af[j], bf[j].x, bf[j].y, Q_F32_INT_BASE);
            uint64_t t01[Q_STAGE_BLOCKS], t23[Q_STAGE_BLOCKS];  // contributions to (row r; 2c, 2c + 1) and (row r + 8; 2c, 2c + 1)
#pragma unroll
            for (int j = 0; j < Q_STAGE_BLOCKS; j++) {
                t01[j] = q40_contribution(d[j][0], d[j][1], wsA[j], par[j]);
                t23[j] = q40_contribution(d[j][2], d[j][3], wsB[j], par[j]);
            }
            if (gi == ng - 1) {  // the stage's bytes are in registers: refill the slot for this warp's stage after next
                __syncwarp();
                if (lane == 0 && s + Q_DEPTH * Q_WARPS < n_stages) issue(s + Q_DEPTH * Q_WARPS, true, true);
            }
            // ---- the ordered part: take the group's accumulators over, add this stage's blocks in order, hand them on ----
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);  // (row r, act 2c), (r, 2c + 1), (r + 8, 2c), (r + 8, 2c + 1)
            if (s > 0) {
                const int received = warp == 0 ? turn - 1 : turn;  // hand-offs this warp has taken before (per group)
                q40_wait(&token[warp * MG + gi], (uint32_t)(received & 1), fail_s);
                acc = hand[(warp * MG + gi) * 32 + lane];
            }
#pragma unroll
            for (int j = 0; j < Q_STAGE_BLOCKS; j++) {
                if (j < nblk) {  // the blocks of a short last stage hold stale bytes: leave them out
                    // scalar additions: this chain is the serial part of the tile, where latency counts and instruction slots do not
                    const float2 lo = f2_unpack(t01[j]), hi = f2_unpack(t23[j]);
                    acc.x = __fadd_rn(acc.x, lo.x), acc.y = __fadd_rn(acc.y, lo.y);
                    acc.z = __fadd_rn(acc.z, hi.x), acc.w = __fadd_rn(acc.w, hi.y);
                }
            }
            if (s + 1 < n_stages) {
                const int nw = (warp + 1) % Q_WARPS;
                hand[(nw * MG + gi) * 32 + lane] = acc;
                __syncwarp();
                if (lane == 0) q40_arrive(&token[nw * MG + gi]);
            } else {  // the last stage: this warp holds the result
                if (*fail_s) acc = make_float4(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000), __int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
                const int64_t row = tile * Q_TILE_ROWS + r, m0 = (g0 + gi) * 8 + 2 * c;
                if (row < p.n) {
                    if (m0 < p.m) st_from_f32(p.out, p.out_dtype, m0 * p.out_stride + row, acc.x);
                    if (m0 + 1 < p.m) st_from_f32(p.out, p.out_dtype, (m0 + 1) * p.out_stride + row, acc.y);
                }
                if (row + 8 < p.n) {
                    if (m0 < p.m) st_from_f32(p.out, p.out_dtype, m0 * p.out_stride + row + 8, acc.z);
                    if (m0 + 1 < p.m) st_from_f32(p.out, p.out_dtype, (m0 + 1) * p.out_stride + row + 8, acc.w);
                }
            }
        }
    }
    __syncthreads();
    if (*fail_s) {
        if (tid == 0) q40_status_fail(p.status, STATUS_WAIT_EXPIRED);
        __nanosleep(200000);  // copies that may still be in flight land before the CTA's memory is released
    }
}

// ---- many activation rows (a prompt pass) ------------------------------------------------------------------------
// grid: (tiles of 16 output rows, blocks of R_WARPS * R_GPW groups of 8 activation rows).  Every warp owns R_GPW groups and
// walks ALL stages of the tile in order, so its accumulators never leave its registers and the additions are in the
// reference's order by construction.  The weight stages are shared: a producer warp pulls them into a ring that the
// R_WARPS consumer warps read (full / empty barriers); every consumer pulls the quantised activations of its own rows.
constexpr int R_WARPS = 8;     // consumer warps per CTA
constexpr int R_GPW = 2;       // groups of 8 activation rows per warp: the unpacked weights of a block serve both
constexpr int R_WDEPTH = 4;    // weight stages in flight per CTA
constexpr int R_ADEPTH = 2;    // activation stages in flight per warp
constexpr int R_ASTAGE = Q_STAGE_BLOCKS * Q_ACT_BLOCK;  // one group's blocks of a stage: 2560 bytes
constexpr size_t R_SMEM = (size_t)R_WDEPTH * Q_STAGE_BYTES + (size_t)R_WARPS * R_ADEPTH * R_GPW * R_ASTAGE + (2 * R_WDEPTH + R_WARPS * R_ADEPTH) * 8 + 16;

__global__ void __launch_bounds__((R_WARPS + 1) * 32, 2) q40_gemm_rows_kernel(Q40Gemm p) {
    extern __shared__ __align__(128) uint8_t ring[];
    uint8_t* aring = ring + R_WDEPTH * Q_STAGE_BYTES;                           // [R_WARPS][R_ADEPTH][R_GPW] activation stages
    uint64_t* wfull = (uint64_t*)(aring + R_WARPS * R_ADEPTH * R_GPW * R_ASTAGE);  // [R_WDEPTH] weight bytes landed
    uint64_t* wempty = wfull + R_WDEPTH;                                        // [R_WDEPTH] consumer warps done with the slot
    uint64_t* afull = wempty + R_WDEPTH;                                        // [R_WARPS][R_ADEPTH]
    volatile int* fail_s = (volatile int*)(afull + R_WARPS * R_ADEPTH);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, c = lane & 3;
    const int64_t tile = blockIdx.x, groups = (p.m + 7) / 8, g0 = (int64_t)blockIdx.y * (R_WARPS * R_GPW);
    const int nw = (int)min((int64_t)R_WARPS, (groups - g0 + R_GPW - 1) / R_GPW);  // consumer warps with rows
    const uint8_t* wsrc = p.packed + tile * p.nb * Q_BLOCK_BYTES;
    const int n_stages = (int)((p.nb + Q_STAGE_BLOCKS - 1) / Q_STAGE_BLOCKS);
    const uint64_t one2 = f2_pack(p.one, p.one);
    auto blocks_of = [&](int s) { return (uint32_t)min((int64_t)Q_STAGE_BLOCKS, p.nb - (int64_t)s * Q_STAGE_BLOCKS); };
    if (tid == 0) {
        for (int i = 0; i < R_WDEPTH; i++) mbar_init(&wfull[i], 1), mbar_init(&wempty[i], nw);
        for (int i = 0; i < R_WARPS * R_ADEPTH; i++) mbar_init(&afull[i], 1);
        *fail_s = 0;
        mbar_fence_init();
    }
    __syncthreads();
    grid_launch_dependents();
    if (warp == R_WARPS) {  // ---- producer of the weight stages (one lane) ----
        if (lane == 0)
            for (int s = 0; s < n_stages; s++) {
                const int sl = s % R_WDEPTH;
                if (s >= R_WDEPTH) q40_wait(&wempty[sl], (uint32_t)((s / R_WDEPTH - 1) & 1), fail_s);
                if (*fail_s) break;
                mbar_expect_tx(&wfull[sl], blocks_of(s) * Q_BLOCK_BYTES);
                bulk_g2s(ring + sl * Q_STAGE_BYTES, wsrc + (int64_t)s * Q_STAGE_BYTES, blocks_of(s) * Q_BLOCK_BYTES, &wfull[sl]);
            }
    } else if (warp < nw) {  // ---- consumers ----
        const int64_t gw = g0 + (int64_t)warp * R_GPW;                 // first group of this warp
        const int ngw = (int)min((int64_t)R_GPW, groups - gw);        // its live groups
        const uint8_t* asrc = p.act + gw * p.nb * Q_ACT_BLOCK;
        uint8_t* mine = aring + warp * R_ADEPTH * R_GPW * R_ASTAGE;
        auto pull = [&](int s) {  // lane 0
            const int sl = s % R_ADEPTH;
            mbar_expect_tx(&afull[warp * R_ADEPTH + sl], ngw * blocks_of(s) * Q_ACT_BLOCK);
            for (int gi = 0; gi < ngw; gi++)
                bulk_g2s(mine + (sl * R_GPW + gi) * R_ASTAGE, asrc + ((int64_t)gi * p.nb + (int64_t)s * Q_STAGE_BLOCKS) * Q_ACT_BLOCK,
                         blocks_of(s) * Q_ACT_BLOCK, &afull[warp * R_ADEPTH + sl]);
        };
        grid_dependency_wait();  // the activation quantiser has finished
        if (lane == 0)
            for (int d = 0; d < R_ADEPTH && d < n_stages; d++) pull(d);
        uint64_t acc01[R_GPW], acc23[R_GPW];  // per group, as packed pairs: (row r; act 2c, 2c + 1) and (row r + 8; 2c, 2c + 1)
#pragma unroll
        for (int gi = 0; gi < R_GPW; gi++) acc01[gi] = acc23[gi] = f2_pack(0.f, 0.f);
        for (int s = 0; s < n_stages; s++) {
            const int nblk = (int)blocks_of(s), wsl = s % R_WDEPTH, asl = s % R_ADEPTH;
            q40_wait(&wfull[wsl], (uint32_t)((s / R_WDEPTH) & 1), fail_s);
            const uint8_t* st = ring + wsl * Q_STAGE_BYTES;
            uint32_t af[Q_STAGE_BLOCKS][4];
            uint64_t wsA[Q_STAGE_BLOCKS], wsB[Q_STAGE_BLOCKS];
#pragma unroll
            for (int j = 0; j < Q_STAGE_BLOCKS; j++) {
                const uint8_t* wb = st + j * Q_BLOCK_BYTES;
                const uint32_t wa = *(const uint32_t*)(wb + r * 16 + 4 * c), wc = *(const uint32_t*)(wb + (r + 8) * 16 + 4 * c);
                af[j][0] = wa & 0x0f0f0f0fu, af[j][1] = wc & 0x0f0f0f0fu, af[j][2] = (wa >> 4) & 0x0f0f0f0fu, af[j][3] = (wc >> 4) & 0x0f0f0f0fu;
                const float sa = __half2float(*(const __half*)(wb + 256 + 2 * r)), sb = __half2float(*(const __half*)(wb + 256 + 2 * (r + 8)));
                wsA[j] = f2_pack(sa, sa), wsB[j] = f2_pack(sb, sb);
            }
            __syncwarp();
            if (lane == 0) q40_arrive(&wempty[wsl]);  // the weights of the stage are in registers
            q40_wait(&afull[warp * R_ADEPTH + asl], (uint32_t)((s / R_ADEPTH) & 1), fail_s);
            // a full stage (all but, at most, the last) runs without the per-block test; a short one leaves its stale blocks out
            auto contract = [&](auto full_stage) {
                constexpr bool FULL = decltype(full_stage)::value;
#pragma unroll
                for (int gi = 0; gi < R_GPW; gi++) {
                    if (gi < ngw) {  // warp-uniform
                        const uint8_t* as = mine + (asl * R_GPW + gi) * R_ASTAGE;
#pragma unroll
                        for (int j = 0; j < Q_STAGE_BLOCKS; j++) {
                            const uint8_t* ab = as + j * Q_ACT_BLOCK;
                            const uint2 bq = *(const uint2*)(ab + lane * 8);
                            const float4 par = *(const float4*)(ab + Q_ACT_PARAMS + c * 16);
                            int d[4];
                            mma_u8s8(d, af[j], bq.x, bq.y, Q_F32_INT_BASE);
                            if (FULL || j < nblk) {
                                acc01[gi] = f2_accumulate(acc01[gi], q40_contribution(d[0], d[1], wsA[j], par), one2);
                                acc23[gi] = f2_accumulate(acc23[gi], q40_contribution(d[2], d[3], wsB[j], par), one2);
                            }
                        }
                    }
                }
            };
            if (nblk == Q_STAGE_BLOCKS) contract(std::true_type{});
            else contract(std::false_type{});
            __syncwarp();
            if (lane == 0 && s + R_ADEPTH < n_stages) pull(s + R_ADEPTH);  // every lane has read the stage: refill its slot
        }
#pragma unroll
        for (int gi = 0; gi < R_GPW; gi++) {
            if (gi >= ngw) break;
            const float2 lo = f2_unpack(acc01[gi]), hi = f2_unpack(acc23[gi]);
            float4 a = make_float4(lo.x, lo.y, hi.x, hi.y);
            if (*fail_s) a = make_float4(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000), __int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
            const int64_t row = tile * Q_TILE_ROWS + r, m0 = (gw + gi) * 8 + 2 * c;
            if (row < p.n) {
                if (m0 < p.m) st_from_f32(p.out, p.out_dtype, m0 * p.out_stride + row, a.x);
                if (m0 + 1 < p.m) st_from_f32(p.out, p.out_dtype, (m0 + 1) * p.out_stride + row, a.y);
            }
            if (row + 8 < p.n) {
                if (m0 < p.m) st_from_f32(p.out, p.out_dtype, m0 * p.out_stride + row + 8, a.z);
                if (m0 + 1 < p.m) st_from_f32(p.out, p.out_dtype, (m0 + 1) * p.out_stride + row + 8, a.w);
            }
        }
    }
    __syncthreads();
    if (*fail_s) {
        if (tid == 0) q40_status_fail(p.status, STATUS_WAIT_EXPIRED);
        __nanosleep(200000);  // copies that may still be in flight land before the CTA's memory is released
    }
}

}  // namespace b200kv

using namespace b200kv;

// The GEMM requests weight stages before it waits for the kernel before it.  This empty kernel, launched the ordinary way
// behind the repacking, separates the two: whatever is scheduled early behind it starts after the packed weights are complete.
__global__ void q40_pack_done_kernel() {}

extern "C" int64_t b200kv_q40_packed_bytes(int64_t n, int64_t k) {
    if (n <= 0 || k <= 0 || k % QK) return -1;
    return (n + Q_TILE_ROWS - 1) / Q_TILE_ROWS * (k / QK) * Q_BLOCK_BYTES;
}

extern "C" int64_t b200kv_q40_scratch_bytes(int64_t k, int32_t m) {
    if (m <= 0 || k <= 0 || k % QK) return -1;
    return Q_HEADER + q40_act_bytes(m, k / QK);  // the larger of the two activation layouts a call with up to m rows may use
}

extern "C" int b200kv_q40_pack(const void* blocks, int64_t n, int64_t k, void* packed, void* stream) {
    if (!blocks || !packed) return fail("null pointer");
    if (n <= 0 || k <= 0 || k % QK) return fail("Q4_0 weights need K a multiple of %d, got %lld", QK, (long long)k);
    if ((uintptr_t)blocks % 2 || (uintptr_t)packed % 16) return fail("blocks must be 2-byte aligned and the packed buffer 16-byte aligned");
    const int64_t nb = k / QK, total = (n + Q_TILE_ROWS - 1) / Q_TILE_ROWS * Q_TILE_ROWS * nb;
    q40_pack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)blocks, n, nb, (uint8_t*)packed);
    q40_pack_done_kernel<<<1, 32, 0, (cudaStream_t)stream>>>();
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

static int q40_check_shape(const void* scratch, int64_t k, int32_t m) {
    if (!scratch) return fail("null pointer");
    if (k <= 0 || k % QK) return fail("W4A8 GEMM needs K a multiple of %d, got %lld", QK, (long long)k);
    if (m <= 0) return fail("m must be positive");
    if ((uintptr_t)scratch % 16) return fail("scratch must be 16-byte aligned");
    return B200KV_OK;
}

extern "C" int b200kv_q40_quantize(const void* a, int64_t a_stride, int32_t m, int32_t dtype, int64_t k, void* scratch, void* stream) {
    if (q40_check_shape(scratch, k, m) != B200KV_OK) return B200KV_KO;
    if (!a) return fail("null pointer");
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if (a_stride < k) return fail("strides shorter than the rows");
    const int64_t nb = k / QK, warps = (int64_t)((m + 7) / 8) * nb * 8;
    B200KV_CUDA(launch_after_predecessor(q40_quant_act_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, a,
                                         a_stride, (const void*)nullptr, (int64_t)0, m, dtype, nb, (uint8_t*)scratch + Q_HEADER, (int*)scratch));
    return B200KV_OK;
}

extern "C" int b200kv_q40_silu_mul_quantize(const void* gate, int64_t gate_stride, const void* up, int64_t up_stride, int32_t m, int32_t dtype,
                                            int64_t k, void* scratch, void* stream) {
    if (q40_check_shape(scratch, k, m) != B200KV_OK) return B200KV_KO;
    if (!gate || !up) return fail("null pointer");
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if (gate_stride < k || up_stride < k) return fail("strides shorter than the rows");
    const int64_t nb = k / QK, warps = (int64_t)((m + 7) / 8) * nb * 8;
    B200KV_CUDA(launch_after_predecessor(q40_quant_act_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, gate,
                                         gate_stride, up, up_stride, m, dtype, nb, (uint8_t*)scratch + Q_HEADER, (int*)scratch));
    return B200KV_OK;
}

extern "C" int b200kv_q40_add_rms_norm_quantize(const float* x, int64_t x_stride, const float* residual, int64_t residual_stride,
                                                const float* weight, float eps, float* x_out, int64_t x_out_stride, int32_t m, int64_t k,
                                                void* scratch, void* stream) {
    if (q40_check_shape(scratch, k, m) != B200KV_OK) return B200KV_KO;
    if (!x) return fail("null pointer");
    if (k > 32 * 512) return fail("rows of at most %d values", 32 * 512);
    if (x_stride < k || (residual && residual_stride < k) || (x_out && x_out_stride < k)) return fail("strides shorter than the rows");
    const int threads = rms_norm_threads((int)k);
    const dim3 grid((unsigned)((m + 7) / 8 * 8));
    uint8_t* act = (uint8_t*)scratch + Q_HEADER;
    int* status = (int*)scratch;
    const int d = (int)k;
    if (k <= 8 * threads)
        B200KV_CUDA(launch_after_predecessor(q40_norm_quant_kernel<8>, grid, dim3(threads), 0, (cudaStream_t)stream, x, x_stride, residual,
                                             residual_stride, weight, eps, x_out, x_out_stride, m, d, act, status));
    else
        B200KV_CUDA(launch_after_predecessor(q40_norm_quant_kernel<32>, grid, dim3(threads), 0, (cudaStream_t)stream, x, x_stride, residual,
                                             residual_stride, weight, eps, x_out, x_out_stride, m, d, act, status));
    return B200KV_OK;
}

extern "C" int b200kv_q40_gemm_quantized_as(const void* packed, int64_t n, int64_t k, int32_t m, void* scratch, void* out, int64_t out_stride,
                                            int32_t out_dtype, void* stream_) {
    if (q40_check_shape(scratch, k, m) != B200KV_OK) return B200KV_KO;
    if (out_dtype < B200KV_F32 || out_dtype > B200KV_BF16) return fail("unknown dtype %d", out_dtype);
    if (!packed || !out) return fail("null pointer");
    if (n <= 0) return fail("n must be positive");
    if ((uintptr_t)packed % 16) return fail("packed weights must be 16-byte aligned");
    if (out_stride < n) return fail("strides shorter than the rows");
    cudaStream_t stream = (cudaStream_t)stream_;
    const int64_t nb = k / QK, groups = (m + 7) / 8;
    uint8_t* act = (uint8_t*)scratch + Q_HEADER;
    Q40Gemm p{};
    p.packed = (const uint8_t*)packed, p.act = act, p.out = out, p.status = (int*)scratch;
    p.n = n, p.nb = nb, p.out_stride = out_stride, p.m = m, p.out_dtype = out_dtype, p.one = 1.0f;
    if (q40_tiled(m))  // a prompt pass: the tcgen05 kernel over the tiled activation layout its producers wrote
        return launch_q40_gemm_tc(packed, act, out, (int*)scratch, n, nb, out_stride, m, out_dtype, stream);
    if (groups >= 4) {  // a few dozen rows: every warp keeps the accumulators of its own 8 rows, the weight stages are shared by 8 warps
        static thread_local int rows_attr_device = -1;
        int dev = 0;
        B200KV_CUDA(cudaGetDevice(&dev));
        if (rows_attr_device != dev) {
            B200KV_CUDA(cudaFuncSetAttribute(q40_gemm_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)R_SMEM));
            rows_attr_device = dev;
        }
        dim3 rgrid((unsigned)((n + Q_TILE_ROWS - 1) / Q_TILE_ROWS), (unsigned)((groups + R_WARPS * R_GPW - 1) / (R_WARPS * R_GPW)));
        B200KV_CUDA(launch_after_predecessor(q40_gemm_rows_kernel, rgrid, dim3((R_WARPS + 1) * 32), R_SMEM, stream, p));
        return B200KV_OK;
    }
    // warps per tile: enough stages per warp (>= 4) that the start-up of a CTA is amortised
    const int64_t n_stages = (nb + Q_STAGE_BLOCKS - 1) / Q_STAGE_BLOCKS;
    // A matrix of few tiles (at most two CTAs of 8 warps per SM, all resident at once) leaves the GPU short of warps: 8 warps
    // per tile put every stage of a K = 4096 tile in flight at once (+10 % on [4096 x 4096]); with more tiles, 4 are faster.
    // more than 8 activation rows: 4 groups share each weight stage (a prompt pass re-reads the weights M / 32 times, from L2)
    const int mg = groups > 1 ? 4 : 1;
    const int64_t n_tiles = (n + Q_TILE_ROWS - 1) / Q_TILE_ROWS;
    const int tile_warps = n_stages >= 32 ? 8 : (n_stages >= 16 ? (mg == 1 && n_tiles <= 2 * 148 ? 8 : 4) : 2);
    auto smem_of = [](int w, int g) {
        return (size_t)w * Q_DEPTH * (Q_STAGE_BYTES + g * Q_STAGE_BLOCKS * Q_ACT_BLOCK) + (size_t)w * g * 32 * 16 + (w * Q_DEPTH + w * g) * 8 + 16;
    };
    const size_t smem = smem_of(tile_warps, mg);
    static thread_local int attr_device = -1;  // the attribute is per device and sticks: set it once per (thread, device)
    int cur = 0;
    B200KV_CUDA(cudaGetDevice(&cur));
    if (attr_device != cur) {
        const int most = (int)smem_of(8, 4);
        B200KV_CUDA(cudaFuncSetAttribute(q40_gemm_kernel<8, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
        B200KV_CUDA(cudaFuncSetAttribute(q40_gemm_kernel<4, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
        B200KV_CUDA(cudaFuncSetAttribute(q40_gemm_kernel<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
        B200KV_CUDA(cudaFuncSetAttribute(q40_gemm_kernel<8, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
        B200KV_CUDA(cudaFuncSetAttribute(q40_gemm_kernel<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
        B200KV_CUDA(cudaFuncSetAttribute(q40_gemm_kernel<2, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
        attr_device = cur;
    }
    dim3 grid((unsigned)((n + Q_TILE_ROWS - 1) / Q_TILE_ROWS), (unsigned)((groups + mg - 1) / mg));
    dim3 block(tile_warps * 32);
    if (mg == 1) {
        if (tile_warps == 8) B200KV_CUDA(launch_after_predecessor(q40_gemm_kernel<8, 1>, grid, block, smem, stream, p));
        else if (tile_warps == 4) B200KV_CUDA(launch_after_predecessor(q40_gemm_kernel<4, 1>, grid, block, smem, stream, p));
        else B200KV_CUDA(launch_after_predecessor(q40_gemm_kernel<2, 1>, grid, block, smem, stream, p));
    } else {
        if (tile_warps == 8) B200KV_CUDA(launch_after_predecessor(q40_gemm_kernel<8, 4>, grid, block, smem, stream, p));
        else if (tile_warps == 4) B200KV_CUDA(launch_after_predecessor(q40_gemm_kernel<4, 4>, grid, block, smem, stream, p));
        else B200KV_CUDA(launch_after_predecessor(q40_gemm_kernel<2, 4>, grid, block, smem, stream, p));
    }
    return B200KV_OK;
}

extern "C" int b200kv_q40_gemm_quantized(const void* packed, int64_t n, int64_t k, int32_t m, void* scratch, float* out, int64_t out_stride,
                                         void* stream) {
    return b200kv_q40_gemm_quantized_as(packed, n, k, m, scratch, out, out_stride, B200KV_F32, stream);
}

extern "C" int b200kv_q40_gemm(const void* packed, int64_t n, int64_t k, const void* a, int64_t a_stride, int32_t m, int32_t dtype,
                               void* scratch, float* out, int64_t out_stride, void* stream) {
    if (!packed || !out || n <= 0 || (uintptr_t)packed % 16 || out_stride < n)  // nothing is enqueued for a call that cannot finish
        return fail("W4A8 GEMM: null pointer, packed weights not 16-byte aligned, or out_stride shorter than n");
    if (b200kv_q40_quantize(a, a_stride, m, dtype, k, scratch, stream) != B200KV_OK) return B200KV_KO;
    return b200kv_q40_gemm_quantized(packed, n, k, m, scratch, out, out_stride, stream);
}

extern "C" int b200kv_q40_check(const void* scratch, void* stream) {
    if (!scratch) return fail("null pointer");
    int st[3] = {0, 0, 0};
    B200KV_CUDA(cudaMemcpyAsync(st, scratch, sizeof st, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    B200KV_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    const bool sticky = (uint32_t)st[2] == Q_MAGIC && (st[1] & STATUS_WAIT_EXPIRED);
    if (sticky) B200KV_CUDA(cudaMemsetAsync((uint8_t*)const_cast<void*>(scratch) + 4, 0, 4, (cudaStream_t)stream));  // reported once
    if (sticky || (st[0] & STATUS_WAIT_EXPIRED))
        return fail("a bounded wait in a Q4_0 GEMM that used this scratch expired (a bulk copy never landed)");
    return B200KV_OK;
}
