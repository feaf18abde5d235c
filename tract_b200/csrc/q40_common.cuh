// Layout of the quantised activations of the W4A8 GEMM, and the quantiser of one block: shared by the GEMM's own producers
// and by the attention kernels that leave their result in that form.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace b200kv {

constexpr int QK = 32;                    // block length
constexpr int Q_TILE_ROWS = 16;           // output rows per warp (the M of the MMA)
constexpr int Q_BLOCK_BYTES = 16 * 16 + 16 * 2;  // one block of a tile: 256 nibble bytes + 16 f16 scales
constexpr int Q_STAGE_BLOCKS = 8;
constexpr int Q_STAGE_BYTES = Q_STAGE_BLOCKS * Q_BLOCK_BYTES;  // 2304
constexpr int Q_DEPTH = 2;                // stages in flight per warp
// Per block and group of 8 activation rows (320 bytes), laid out as the lanes of the GEMM's MMA read it: codes
// [row 8][quad 4][elements 4q .. 4q+3 | 16+4q .. 16+4q+3] (lane 4 row + quad takes its 8 bytes in one load), then per
// quad four floats {scale of row 2q, scale of row 2q+1, -(Q_F32_BASE + 8 * code sum of row 2q), the same of row 2q+1}.
// The MMA's int32 accumulators start at Q_F32_INT_BASE, the bits of the float Q_F32_BASE = 1.5 * 2^23: the finished
// accumulator, read as a float, is Q_F32_BASE + (dot product with the unsigned nibbles) exactly, and one float addition
// of the row's third parameter leaves (dot product with nibble - 8) as f32 -- the int -> float conversion and the offset
// correction of the reference in one exact operation (every value involved is an integer below 2^24).
constexpr int Q_ACT_BLOCK = 8 * 32 + 4 * 16;
constexpr int Q_ACT_PARAMS = 256;         // byte offset of the per-quad parameters
constexpr int32_t Q_F32_INT_BASE = 0x4B400000;
constexpr float Q_F32_BASE = 12582912.f;
constexpr int Q_HEADER = 256;             // scratch header: word 0 = status of the GEMMs since the last producer, word 1 = status of every
                                          // GEMM since the last b200kv_q40_check (no producer clears it), word 2 = Q_MAGIC once word 1 is valid
constexpr uint32_t Q_MAGIC = 0x51343041u;

// Run by one thread of every kernel that produces the activation: word 0 starts a new epoch; the sticky word is zeroed
// only the first time this scratch is seen (caller memory arrives uninitialised), so that a wait that expired in any
// GEMM of a step stays visible until the host asks.
__device__ inline void q40_status_begin(int* status) {
    if ((uint32_t)status[2] != Q_MAGIC) status[1] = 0, status[2] = (int)Q_MAGIC;
    status[0] = 0;
}
__device__ inline void q40_status_fail(int* status, int bits) {
    atomicOr(status, bits);
    atomicOr(status + 1, bits);
}
constexpr int Q_RING_STAGE = Q_STAGE_BYTES + Q_STAGE_BLOCKS * Q_ACT_BLOCK;  // weights then activations of 8 blocks: 4864 bytes

// ---- the second layout of the quantised activations: from Q_TC_MIN_ROWS rows on (a prompt pass) the GEMM runs on
// tcgen05 (q40_tc.cu) and wants the codes as operand tiles.  Rows are cut into tiles of 128, K into stages of 4 blocks
// (128 bytes of codes per row): a (row tile, stage) pair is 128 rows x 128 bytes with the 128-byte swizzle of a K-major
// tensor-core operand (16-byte unit u of row r at u ^ (r & 7)), 16 KB contiguous, so that one untiled bulk copy lands a
// stage in shared memory ready for the MMA.  The parameters follow the codes: per (row tile, block) 128 x {scale, offset
// term} f32, read by the thread that owns the row.  Same 40 bytes per row and block as the record layout above.
constexpr int Q_TC_MIN_ROWS = 128;
constexpr int Q_TC_ROWS = 128;                      // activation rows per tile (the M of the MMA)
constexpr int Q_TC_KBLOCKS = 4;                     // blocks per stage
constexpr int Q_TC_TILE = Q_TC_ROWS * Q_TC_KBLOCKS * QK;  // 16384 bytes of codes
__host__ __device__ inline bool q40_tiled(int64_t m) { return m >= Q_TC_MIN_ROWS; }
__host__ __device__ inline int64_t q40_tc_stages(int64_t nb) { return (nb + Q_TC_KBLOCKS - 1) / Q_TC_KBLOCKS; }
__host__ __device__ inline int64_t q40_tc_row_tiles(int64_t m) { return (m + Q_TC_ROWS - 1) / Q_TC_ROWS; }
__host__ __device__ inline int64_t q40_tc_codes_bytes(int64_t m, int64_t nb) { return q40_tc_row_tiles(m) * q40_tc_stages(nb) * Q_TC_TILE; }
__host__ __device__ inline int64_t q40_act_bytes(int64_t m, int64_t nb) {  // either layout, for up to m rows
    const int64_t records = (m + 7) / 8 * nb * Q_ACT_BLOCK;
    const int64_t tiled = q40_tiled(m) ? q40_tc_codes_bytes(m, nb) + q40_tc_row_tiles(m) * nb * Q_TC_ROWS * 8 : 0;
    return records > tiled ? records : tiled;
}

// Q4_0::quantize_row_q8 (q4_0.rs:199-222) for one block: the 32 lanes of a warp hold its 32 values.  Writes the codes,
// the scale and the offset term of activation row `mi`, block `b`, into the activation buffer `act` of a call with `m`
// rows and `nb` blocks per row, in the layout that call's GEMM reads.  `valid` false (a row past the last): zero codes,
// scale 0.
__device__ inline void q40_quantize_block(float x, bool valid, uint8_t* act, int64_t m, int64_t nb, int64_t mi, int64_t b, int lane) {
    if (!valid) x = 0.f;
    float amax = fabsf(x);
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));  // fmaxf ignores a NaN operand, as f32::max does
    amax = fmaxf(0.f, amax);                                                                 // the fold starts from 0: an all-NaN block gives 0
    const float scale = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float r = __fdiv_rn(1.0f, scale);
    const float t = roundf(__fmul_rn(x, r));  // NaN for a NaN input and for inf * 0
    const int q = (t != t) ? 0 : (int)fminf(fmaxf(t, -127.f), 127.f);  // f32::clamp keeps a NaN, the cast to i8 makes it 0
    const int sum = __reduce_add_sync(0xffffffffu, q);
    const float scale_out = valid ? scale : 0.f;
    const float offset_out = -(Q_F32_BASE + (float)(8 * sum));  // exact: |8 sum| <= 8 * 32 * 127
    if (q40_tiled(m)) {
        const int64_t tile = mi / Q_TC_ROWS, st = b / Q_TC_KBLOCKS;
        const int row = (int)(mi % Q_TC_ROWS), unit = 2 * (int)(b % Q_TC_KBLOCKS) + (lane >> 4);
        act[(tile * q40_tc_stages(nb) + st) * Q_TC_TILE + row * 128 + ((unit ^ (row & 7)) << 4) + (lane & 15)] = (uint8_t)(int8_t)q;
        if (lane == 0) {
            float2* par = (float2*)(act + q40_tc_codes_bytes(m, nb)) + (tile * nb + b) * Q_TC_ROWS + row;
            *par = make_float2(scale_out, offset_out);
        }
    } else {
        const int slot = (int)(mi & 7);
        uint8_t* dst = act + ((mi >> 3) * nb + b) * Q_ACT_BLOCK;
        dst[slot * 32 + ((lane & 15) >> 2) * 8 + (lane >> 4) * 4 + (lane & 3)] = (uint8_t)(int8_t)q;
        if (lane == 0) {
            uint8_t* par = dst + Q_ACT_PARAMS + (slot >> 1) * 16 + (slot & 1) * 4;
            *(float*)par = scale_out;
            *(float*)(par + 8) = offset_out;
        }
    }
}

}  // namespace b200kv
