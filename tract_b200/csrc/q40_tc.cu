// Q4_0 weights x int8-quantised activations for many activation rows (a prompt pass) on the 5th-generation tensor cores.
//
// Arithmetic: Q4_0::w4a8_gemm of tract-linalg (linalg/src/frame/block_quant/q4_0.rs:260-310), bit for bit, as in q40.cu:
// every (weight block, activation block) pair contributes (exact int32 dot as f32) * w_scale * a_scale, each operation
// rounded on its own, added to the output in ascending block order.  Replaces the prompt-pass use of
// cuda/src/kernels/cu/mm_mv_q.cu behind cuda/src/kernels/matmul/mod.rs:481-520.
//
// The cost of this GEMM is not the integer dot products but the three float operations every output owes every block.
// With mma.sync a thread owns 4 outputs of a 16 x 8 fragment and pays about 8 instructions per output and block for them
// (fragment loads, weight unpacking, scale loads).  Here ONE tcgen05.mma.kind::i8 (M = 128 activation rows, N = 128
// weight rows, K = 32: exactly one block) leaves the 128 x 128 dot products of a block in TMEM, and the threads that own
// the rows do nothing but the float part, as packed f32x2 instructions: 2.5 instructions per output and block.
//   - activations arrive as operand tiles (q40_common.cuh: 128 rows x 4 blocks, swizzled, one bulk copy per stage);
//   - weights arrive as they are packed for the other kernels (tiles of 16 rows, 8 bulk copies per stage); two converter
//     warps split the nibbles into unsigned bytes in the swizzled B tile and widen the block scales to f32;
//   - the accumulator buffers start at the bit pattern of 1.5 * 2^23 (written back by the thread that read them), so that a
//     finished int32 accumulator read as a float is 1.5 * 2^23 + dot, and one float addition of the row's offset term
//     gives (dot with nibble - 8) as f32 exactly: no integer subtraction, no conversion instruction;
//   - four accumulator buffers of 128 columns fill the 512 TMEM columns: the MMA of block b + 4 waits for the rows of
//     block b to be read, nothing else.
// Roles: 16 warps own the outputs (rows by TMEM lane quarter, four groups of 32 columns; with 8 warps of 64 columns the
// kernel issued 1.9 instructions per cycle and SM), 2 converter warps, 1 MMA warp, 1 loader warp.  Every wait is bounded; on expiry the CTA flags the status word and stores NaNs.
#include "f32x2.cuh"
#include "glue_math.cuh"
#include "q40_common.cuh"
#include "tc_common.cuh"

namespace b200kv {

constexpr int T_ROWS = Q_TC_ROWS;          // activation rows per CTA: the M of the MMA, one TMEM lane each
constexpr int T_COLS = 128;                // weight rows (output columns) per CTA: the N of the MMA
constexpr int T_KB = Q_TC_KBLOCKS;         // blocks per stage
constexpr int T_TILE = Q_TC_TILE;          // bytes of an operand tile: 128 rows x 128 bytes
constexpr int T_RAW16 = T_KB * Q_BLOCK_BYTES;                 // one 16-row weight tile's blocks of a stage: 1152 bytes
constexpr int T_RAW = (T_COLS / Q_TILE_ROWS) * T_RAW16;       // 9216 bytes of packed weights per stage
constexpr int T_NR = 3;                    // raw weight stages
constexpr int T_NS = 3;                    // operand stages (activation tile + converted weight tile)
constexpr int T_NWS = 8;                   // stages of f32 weight scales: the owners of the outputs read them up to two stages
                                           // behind the MMA, the converters write them up to three stages ahead
constexpr int T_ND = 4;                    // accumulator buffers
constexpr int T_EPI_WARPS = 16, T_CONV_WARPS = 2;
constexpr int T_EPI_COLS = T_COLS / (T_EPI_WARPS / 4);  // columns per output-owning thread: 32
constexpr int T_THREADS = (T_EPI_WARPS + T_CONV_WARPS + 2) * 32;
constexpr int T_N_BARS = 2 * T_NR + 3 * T_NS + 2 * T_ND;
constexpr size_t T_SMEM = (size_t)2 * T_NS * T_TILE + (size_t)T_NR * T_RAW + (size_t)T_NWS * T_KB * T_COLS * 4 + T_N_BARS * 8 + 64;

struct Q40TcGemm {
    const uint8_t* packed;
    const uint8_t* act;  // the tiled layout of q40_common.cuh
    void* out;
    int* status;
    int64_t n, nb, out_stride;
    int32_t m, out_dtype;
    float one;  // 1.0f the compiler cannot see through, see f2_accumulate in q40.cu
};

// D[tmem] (+)= A[smem] . B[smem], 8-bit integers, int32 accumulation
__device__ inline void tc_mma_i8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// instruction descriptor of kind::i8: int32 accumulators, A signed bytes, B unsigned bytes, both K-major
__host__ __device__ constexpr uint32_t instr_desc_i8(int M, int N) {
    return (2u << 4) | (1u << 7) | (0u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__global__ void __launch_bounds__(T_THREADS, 1) q40_gemm_tc_kernel(const __grid_constant__ Q40TcGemm p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* act_s = smem;                                  // [T_NS] activation tiles (A operand)
    uint8_t* wt_s = act_s + T_NS * T_TILE;                  // [T_NS] weight tiles (B operand): unsigned nibble values
    uint8_t* raw_s = wt_s + T_NS * T_TILE;                  // [T_NR] packed weights as they lie in memory
    float* ws_s = (float*)(raw_s + T_NR * T_RAW);           // [T_NWS][T_KB][T_COLS] block scales of the weight rows
    uint64_t* raw_full = (uint64_t*)(ws_s + T_NWS * T_KB * T_COLS);  // [T_NR] bytes landed
    uint64_t* raw_free = raw_full + T_NR;                   // [T_NR] the converters are done with the raw stage
    uint64_t* act_full = raw_free + T_NR;                   // [T_NS] bytes landed
    uint64_t* wt_full = act_full + T_NS;                    // [T_NS] the converters have written the tile
    uint64_t* stage_done = wt_full + T_NS;                  // [T_NS] every product on the stage has completed
    uint64_t* d_full = stage_done + T_NS;                   // [T_ND] the product of a block has completed
    uint64_t* d_free = d_full + T_ND;                       // [T_ND] every row of the buffer has been read and reset
    uint32_t* tmem_slot = (uint32_t*)(d_free + T_ND);
    volatile int* fail_s = (volatile int*)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t n0 = (int64_t)blockIdx.x * T_COLS, mt = blockIdx.y;
    const int64_t nb = p.nb, n_stages = q40_tc_stages(nb), n_tile16 = (p.n + Q_TILE_ROWS - 1) / Q_TILE_ROWS;
    auto blocks_of = [&](int64_t s) { return (int)min((int64_t)T_KB, nb - s * T_KB); };

    if (tid == 0) {
        for (int i = 0; i < T_NR; i++) mbar_init(&raw_full[i], 1), mbar_init(&raw_free[i], T_CONV_WARPS);
        for (int i = 0; i < T_NS; i++) mbar_init(&act_full[i], 1), mbar_init(&wt_full[i], T_CONV_WARPS), mbar_init(&stage_done[i], 1);
        for (int i = 0; i < T_ND; i++) mbar_init(&d_full[i], 1), mbar_init(&d_free[i], T_EPI_WARPS);
        *fail_s = (smem_u32(smem) & 1023u) ? 1 : 0;  // the swizzled operand tiles need a 1024-byte aligned base
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 512);
    grid_launch_dependents();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == T_EPI_WARPS + T_CONV_WARPS + 1) {
        // ================= loader: packed weights (8 tiles of 16 rows per stage) and activation tiles =================
        auto load_raw = [&](int64_t s) {
            if (s >= T_NR) wait_or_fail(&raw_free[s % T_NR], (uint32_t)((s / T_NR - 1) & 1), fail_s);
            if (elect_one()) {
                const uint32_t bytes = (uint32_t)blocks_of(s) * Q_BLOCK_BYTES;
                mbar_expect_tx(&raw_full[s % T_NR], (T_COLS / Q_TILE_ROWS) * bytes);
                for (int j = 0; j < T_COLS / Q_TILE_ROWS; j++) {
                    const int64_t t16 = min(n0 / Q_TILE_ROWS + j, n_tile16 - 1);  // past the last tile: any tile, its outputs are not stored
                    bulk_g2s(raw_s + (s % T_NR) * T_RAW + j * T_RAW16, p.packed + (t16 * nb + s * T_KB) * Q_BLOCK_BYTES, bytes, &raw_full[s % T_NR]);
                }
            }
            __syncwarp();
        };
        for (int64_t s = 0; s < T_NR && s < n_stages; s++) load_raw(s);  // the weights do not depend on the launch before
        grid_dependency_wait();                                           // the activation quantiser has finished
        for (int64_t s = 0; s < n_stages; s++) {
            if (s >= T_NS) wait_or_fail(&stage_done[s % T_NS], (uint32_t)((s / T_NS - 1) & 1), fail_s);
            if (elect_one()) {
                mbar_expect_tx(&act_full[s % T_NS], T_TILE);
                bulk_g2s(act_s + (s % T_NS) * T_TILE, p.act + (mt * n_stages + s) * T_TILE, T_TILE, &act_full[s % T_NS]);
            }
            __syncwarp();
            if (s + T_NR < n_stages) load_raw(s + T_NR);
        }
    } else if (warp == T_EPI_WARPS + T_CONV_WARPS) {
        // ================= one product per block: D[128 rows x 128 columns] += A_block . B_block^T =================
        const uint32_t idesc = instr_desc_i8(T_ROWS, T_COLS);
        const uint64_t a_desc = smem_desc(smem_u32(act_s), 0, 1024), b_desc = smem_desc(smem_u32(wt_s), 0, 1024);
        for (int64_t s = 0; s < n_stages; s++) {
            const uint32_t par = (uint32_t)((s / T_NS) & 1);
            wait_or_fail(&act_full[s % T_NS], par, fail_s);
            wait_or_fail(&wt_full[s % T_NS], par, fail_s);
            tc_fence_after();
            const int nblk = blocks_of(s);
            for (int q = 0; q < nblk; q++) {
                const int64_t b = s * T_KB + q;
                const int buf = (int)(b % T_ND);
                wait_or_fail(&d_free[buf], (uint32_t)((b / T_ND) & 1), fail_s);  // phase 0: the initial fill; phase k: block b - 4 has been read
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t off = (uint64_t)(((s % T_NS) * T_TILE + q * QK) >> 4);  // 32 bytes of K per block inside the 128-byte rows
                    tc_mma_i8_ss(tmem + buf * T_COLS, a_desc + off, b_desc + off, idesc, 1u);
                    tc_commit(&d_full[buf]);
                }
                __syncwarp();
            }
            if (elect_one()) tc_commit(&stage_done[s % T_NS]);
            __syncwarp();
        }
    } else if (warp >= T_EPI_WARPS) {
        // ================= converters: packed nibbles -> unsigned bytes in the swizzled B tile, f16 scales -> f32 =================
        const int ct = tid - T_EPI_WARPS * 32;  // 0 .. 63: weight rows ct and ct + 64 of the tile
        for (int64_t s = 0; s < n_stages; s++) {
            wait_or_fail(&raw_full[s % T_NR], (uint32_t)((s / T_NR) & 1), fail_s);
            if (s >= T_NS) wait_or_fail(&stage_done[s % T_NS], (uint32_t)((s / T_NS - 1) & 1), fail_s);
            const int nblk = blocks_of(s);
            const uint8_t* raw = raw_s + (s % T_NR) * T_RAW;
            uint8_t* wt = wt_s + (s % T_NS) * T_TILE;
            float* ws = ws_s + (s % T_NWS) * T_KB * T_COLS;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int nrow = ct + 64 * h;
                const uint8_t* src = raw + (nrow / Q_TILE_ROWS) * T_RAW16 + (nrow % Q_TILE_ROWS) * 16;
                for (int q = 0; q < nblk; q++) {
                    // bytes j of a row's 16: element j in the low nibble, element j + 16 in the high one (GGML order)
                    const uint4 x = *(const uint4*)(src + q * Q_BLOCK_BYTES);
                    const uint4 lo = make_uint4(x.x & 0x0f0f0f0fu, x.y & 0x0f0f0f0fu, x.z & 0x0f0f0f0fu, x.w & 0x0f0f0f0fu);
                    const uint4 hi = make_uint4((x.x >> 4) & 0x0f0f0f0fu, (x.y >> 4) & 0x0f0f0f0fu, (x.z >> 4) & 0x0f0f0f0fu, (x.w >> 4) & 0x0f0f0f0fu);
                    *(uint4*)(wt + nrow * 128 + (((2 * q) ^ (nrow & 7)) << 4)) = lo;
                    *(uint4*)(wt + nrow * 128 + (((2 * q + 1) ^ (nrow & 7)) << 4)) = hi;
                    ws[q * T_COLS + nrow] = __half2float(*(const __half*)(raw + (nrow / Q_TILE_ROWS) * T_RAW16 + q * Q_BLOCK_BYTES + 256 + 2 * (nrow % Q_TILE_ROWS)));
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&wt_full[s % T_NS]), mbar_arrive(&raw_free[s % T_NR]);
        }
    } else {
        // ================= owners of the outputs: row = TMEM lane, 32 of the 128 columns =================
        constexpr int EC = T_EPI_COLS, NCH = EC / 16;  // columns per thread, in chunks of 16
        const int quarter = warp & 3, group = warp >> 2, row = quarter * 32 + lane, c0 = group * EC;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16) + c0;
        uint32_t start[8];
#pragma unroll
        for (int i = 0; i < 8; i++) start[i] = (uint32_t)Q_F32_INT_BASE;
        for (int buf = 0; buf < T_ND; buf++) {
#pragma unroll
            for (int c = 0; c < EC / 8; c++) tmem_st8(lane_base + buf * T_COLS + 8 * c, start);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&d_free[buf]);
        }
        grid_dependency_wait();  // the activation parameters are read from memory below
        const float2* par = (const float2*)(p.act + q40_tc_codes_bytes(p.m, nb)) + mt * nb * T_ROWS + row;  // {scale, offset term} of (block, row)
        const uint64_t one2 = f2_pack(p.one, p.one);
        uint64_t acc[EC / 2];
#pragma unroll
        for (int j = 0; j < EC / 2; j++) acc[j] = f2_pack(0.f, 0.f);
        float2 pnext = par[0];
        for (int64_t b = 0; b < nb; b++) {
            const int buf = (int)(b % T_ND);
            const float2 pr = pnext;
            if (b + 1 < nb) pnext = par[(b + 1) * T_ROWS];
            wait_or_fail(&d_full[buf], (uint32_t)((b / T_ND) & 1), fail_s);
            tc_fence_after();
            const float* ws = ws_s + ((b / T_KB) % T_NWS) * T_KB * T_COLS + (b % T_KB) * T_COLS + c0;
            const uint64_t asc2 = f2_pack(pr.x, pr.x), off2 = f2_pack(pr.y, pr.y);
            // 16 columns at a time, the load of the next 16 in flight under the arithmetic of these; once the last load has
            // landed the buffer goes back to its start value and may take block b + 4
            uint32_t d[2][16];
            tmem_ld16(lane_base + buf * T_COLS, d[0]);
            tmem_ld_wait();
#pragma unroll
            for (int hh = 0; hh < NCH; hh++) {
                if (hh + 1 < NCH) tmem_ld16(lane_base + buf * T_COLS + 16 * (hh + 1), d[(hh + 1) & 1]);
                if (NCH == 1 || hh == NCH - 2) {
                    if (hh + 1 < NCH) tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < EC / 8; c++) tmem_st8(lane_base + buf * T_COLS + 8 * c, start);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&d_free[buf]);
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float2 w2 = *(const float2*)(ws + 16 * hh + 2 * j);
                    // (dot as f32) * w_scale * a_scale, each operation rounded on its own, then added in block order
                    const uint64_t dot = f2_add(f2_pack_bits(d[hh & 1][2 * j], d[hh & 1][2 * j + 1]), off2);
                    const uint64_t t = f2_mul(f2_mul(dot, f2_pack(w2.x, w2.y)), asc2);
                    acc[8 * hh + j] = f2_fma(t, one2, acc[8 * hh + j]);
                }
                if (hh + 1 < NCH && hh != NCH - 2) tmem_ld_wait();
            }
        }
        const int64_t mi = mt * T_ROWS + row;
        const bool failed = *fail_s != 0;
        if (mi < p.m) {
            const int64_t col0 = n0 + c0, at = mi * p.out_stride + col0;
            const float nan = __int_as_float(0x7fc00000);
            if (p.out_dtype == B200KV_F32) {
                float* o = (float*)p.out + at;
#pragma unroll
                for (int j = 0; j < EC / 2; j++) {
                    const float2 v = failed ? make_float2(nan, nan) : f2_unpack(acc[j]);
                    if (col0 + 2 * j < p.n) o[2 * j] = v.x;
                    if (col0 + 2 * j + 1 < p.n) o[2 * j + 1] = v.y;
                }
            } else {
                uint16_t* o = (uint16_t*)p.out + at;
#pragma unroll
                for (int j = 0; j < EC / 2; j++) {
                    const float2 v = failed ? make_float2(nan, nan) : f2_unpack(acc[j]);
                    const uint16_t lo = p.out_dtype == B200KV_F16 ? __half_as_ushort(__float2half_rn(v.x)) : __bfloat16_as_ushort(__float2bfloat16_rn(v.x));
                    const uint16_t hi = p.out_dtype == B200KV_F16 ? __half_as_ushort(__float2half_rn(v.y)) : __bfloat16_as_ushort(__float2bfloat16_rn(v.y));
                    if (col0 + 2 * j < p.n) o[2 * j] = lo;
                    if (col0 + 2 * j + 1 < p.n) o[2 * j + 1] = hi;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*fail_s) {
        if (tid == 0) q40_status_fail(p.status, STATUS_WAIT_EXPIRED);
        __nanosleep(200000);  // copies that may still be in flight land before the CTA's memory is released
        __syncthreads();
    }
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// The prompt-pass GEMM: `act` holds the tiled layout (m >= Q_TC_MIN_ROWS).
int launch_q40_gemm_tc(const void* packed, const void* act, void* out, int* status, int64_t n, int64_t nb, int64_t out_stride, int32_t m,
                       int32_t out_dtype, cudaStream_t stream) {
    static thread_local int attr_device = -1;
    int dev = 0;
    B200KV_CUDA(cudaGetDevice(&dev));
    if (attr_device != dev) {
        B200KV_CUDA(cudaFuncSetAttribute(q40_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T_SMEM));
        attr_device = dev;
    }
    Q40TcGemm p{};
    p.packed = (const uint8_t*)packed, p.act = (const uint8_t*)act, p.out = out, p.status = status;
    p.n = n, p.nb = nb, p.out_stride = out_stride, p.m = m, p.out_dtype = out_dtype, p.one = 1.0f;
    const dim3 grid((unsigned)((n + T_COLS - 1) / T_COLS), (unsigned)q40_tc_row_tiles(m));
    B200KV_CUDA(launch_after_predecessor(q40_gemm_tc_kernel, grid, dim3(T_THREADS), T_SMEM, stream, p));
    return B200KV_OK;
}

}  // namespace b200kv
