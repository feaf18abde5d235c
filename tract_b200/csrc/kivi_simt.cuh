// CUDA-core decode attention over a KIVI cache: the kernel body, shared by kivi.cu (the kernel of its own) and
// kivi_mma.cu (whose extra CTAs run it for the sinks and the residual block).
#pragma once
#include "decode_common.h"
#include "kivi_common.cuh"

namespace b200kv {

constexpr int KTILE = 32;  // tokens per tile
constexpr int KGT = 4;     // query heads per CTA

struct KiviDecode {
    KiviView v;
    const void* q;
    int64_t qb, qh;
    float* part_o;
    float* part_ml;
    int32_t G, dtype, n_splits;
    int32_t f32_only;               // 1: only the tiles the tensor-core kernel leaves out (sinks, residual block)
    int32_t part_stride, part_off;  // partial of (batch b, split s) = b * part_stride + part_off + s
    float scale;
};

__device__ inline void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(__cvta_generic_to_global(src)) : "memory");
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ inline void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Tiles follow the stores: tile -1 is the f32 sinks, tile k >= 0 the 32 tokens 4 + 32k .. 4 + 32k + 31, i.e. exactly
// one key block (finalised: codes + per-channel parameters; the last, partial one: f32 residual rows) and 32
// per-token value rows.  The raw bytes of tile k + 1 are fetched with cp.async while tile k is being consumed.
template <int D>
struct KiviSimtSmem {
    static constexpr int RS = 144;  // row stride of the staged code rows: 16-byte aligned, and 36 words so that 8 rows hit 32 banks
    struct Stage {
        uint8_t kc[KTILE * RS], vc[KTILE * RS];  // code rows
        float kpar[2 * D];                       // lo[D], scale[D] of the key block
        float vpar[2 * KTILE];                   // (lo, scale) per value token
    };
    Stage st[2];
    float q_s[KGT * D], sc_s[KGT * KTILE], alpha_s[KGT], ml_s[KGT * 2];
};

// The body of the kernel, for a CTA of 128 threads working on batch entry / split `bx`, kv head `kvh`, head group `gz`,
// in `sm` (16-byte aligned shared memory).  Also run by the extra CTAs of the tensor-core kernel (kivi_mma.cu).
template <int D>
__device__ inline void kivi_simt_body(const KiviDecode& p, const InlineBatch& ib, KiviSimtSmem<D>& sm, int bx, int kvh_, int gz) {
    constexpr int RS = KiviSimtSmem<D>::RS;
    using Stage = typename KiviSimtSmem<D>::Stage;
    Stage* st = sm.st;
    float *q_s = sm.q_s, *sc_s = sm.sc_s, *alpha_s = sm.alpha_s, *ml_s = sm.ml_s;
    const KiviView& v = p.v;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = bx / p.n_splits, split = bx % p.n_splits;
    const int kvh = kvh_, g0 = gz * KGT, ng = min(KGT, p.G - g0);
    const int32_t seq = ib.ent[b].x;
    const int64_t len = ib.ent[b].y;
    const int n_after = (int)max((int64_t)0, len - SINK), n_fin = n_after / KBLOCK;
    const int tiles = (n_after + KTILE - 1) / KTILE;
    // split s takes tiles [lo, hi) of -1 .. tiles-1
    const int tile_lo = (int)((int64_t)(tiles + 1) * split / p.n_splits) - 1, tile_hi = (int)((int64_t)(tiles + 1) * (split + 1) / p.n_splits) - 1;
    // the tile after t: every tile, or (f32_only) the sinks and then the residual block, if there is one
    auto next_tile = [&](int t) { return p.f32_only ? (t < 0 ? n_fin : tiles) : t + 1; };
    const int first_staged = tile_lo >= 0 ? tile_lo : next_tile(tile_lo);  // tile -1 needs no staging
    const int row_bytes = v.row_bytes, chunks = row_bytes / 16;
    const bool mma_layout = kivi_mma_layout(v.bits, v.D);
    const int lfmt = kivi_layout_fmt(v.bits);
    // where channel `tid` sits in a staged V row: byte and, for int4, nibble
    const int v_pos = mma_layout ? code_pos(lfmt, 128, 1, tid & 127) : (v.bits == 8 ? tid : tid >> 1);
    const int v_nib = mma_layout ? code_nibble(lfmt, 128, 1, tid & 127) : (tid & 1);
    const float* sink_k = v.sinks + (((int64_t)seq * v.H + kvh) * 2 + 0) * SINK * D;
    const float* sink_v = v.sinks + (((int64_t)seq * v.H + kvh) * 2 + 1) * SINK * D;
    const float* resid = v.residual + (((int64_t)seq * v.H + kvh) * 2 + 0) * KBLOCK * D;

    auto prefetch = [&](int k) {  // raw bytes of tile k (>= 0) into stage k & 1
        Stage& s = st[k & 1];
        const int32_t pg = v.table[(int64_t)seq * v.max_pages_per_seq + (k * KTILE) / PAGE_TOKENS];
        const int slot0 = (k * KTILE) % PAGE_TOKENS;
        const int nrow = min(KTILE, n_after - k * KTILE);
        const uint8_t* vrow = v.codes[1] + (((int64_t)pg * v.H + kvh) * PAGE_TOKENS + slot0) * row_bytes;
        // (rows in the tensor-core layout are un-swizzled on the way in: the staged rows are in byte-position order)
        const uint8_t* vpage = v.codes[1] + ((int64_t)pg * v.H + kvh) * PAGE_TOKENS * row_bytes;
        for (int i = tid; i < nrow * chunks; i += 128) {
            const int rr = i / chunks, u = i % chunks;
            const uint8_t* src = mma_layout ? vpage + chunk_addr(lfmt, 128, 1, slot0 + rr, 16 * u) : vrow + rr * row_bytes + u * 16;
            cp_async16(s.vc + rr * RS + u * 16, src);
        }
        const float* vp = v.params[1] + (((int64_t)pg * v.H + kvh) * PAGE_TOKENS + slot0) * 2;
        if (tid < KTILE / 2) cp_async16(s.vpar + tid * 4, vp + tid * 4);  // whole 256-byte run; rows past nrow are ignored
        if (k < n_fin) {
            const uint8_t* krow = v.codes[0] + (((int64_t)pg * v.H + kvh) * PAGE_TOKENS + slot0) * row_bytes;
            const uint8_t* kpage = v.codes[0] + ((int64_t)pg * v.H + kvh) * PAGE_TOKENS * row_bytes;
            for (int i = tid; i < KTILE * chunks; i += 128) {
                const int rr = i / chunks, u = i % chunks;
                const uint8_t* src = mma_layout ? kpage + chunk_addr(lfmt, 128, 0, slot0 + rr, 16 * u) : krow + rr * row_bytes + u * 16;
                cp_async16(s.kc + rr * RS + u * 16, src);
            }
            const float* kp = v.params[0] + (((int64_t)pg * v.H + kvh) * 2 + slot0 / KBLOCK) * 2 * D;
            for (int i = tid; i < 2 * D / 4; i += 128) cp_async16(s.kpar + i * 4, kp + i * 4);
        }
    };
    if (first_staged < tile_hi) prefetch(first_staged);
    cp_async_commit();

    for (int idx = tid; idx < KGT * D; idx += 128) {
        const int g = idx / D;
        q_s[idx] = g < ng ? ld_as_f32(p.q, p.dtype, (int64_t)b * p.qb + (int64_t)(kvh * p.G + g0 + g) * p.qh + idx % D) : 0.f;
    }
    float m_run = -INFINITY, l_run = 0.f;   // warp g keeps the state of head g
    float acc[KGT] = {0.f, 0.f, 0.f, 0.f};  // thread = output channel
    const bool eight = v.bits == 8;

    for (int tile = tile_lo; tile < tile_hi; tile = next_tile(tile)) {
        // the next tile's bytes start moving before this one is touched
        const int nt = next_tile(tile);
        if (nt < tile_hi && nt != first_staged) prefetch(nt);
        cp_async_commit();
        if (tile >= 0) cp_async_wait<1>();  // everything but the group just committed has landed
        __syncthreads();
        const Stage& s = st[tile & 1];
        const int n_valid = tile < 0 ? (int)min((int64_t)SINK, len) : min(KTILE, n_after - tile * KTILE);
        const bool k_f32 = tile < 0 || tile >= n_fin;  // sinks / residual rows: f32 straight from global memory
        const float* kf = tile < 0 ? sink_k : resid;
        {  // scores: 4 threads per token; thread `part` takes the 4-channel words part, part + 4, ...
            const int tt = tid >> 2, part = tid & 3;
            float dot[KGT] = {0.f, 0.f, 0.f, 0.f};
            if (tt < n_valid) {
                for (int w = part; w < D / 4; w += 4) {
                    float kx[4];
                    if (k_f32) {
                        const float4 f = *(const float4*)(kf + tt * D + 4 * w);
                        kx[0] = f.x, kx[1] = f.y, kx[2] = f.z, kx[3] = f.w;
                    } else {
                        uint32_t codes[4];
                        if (eight) {
                            const uint32_t word = *(const uint32_t*)(s.kc + tt * RS + 4 * w);
#pragma unroll
                            for (int e = 0; e < 4; e++) codes[e] = (word >> (8 * e)) & 0xffu;
                        } else {
                            if (mma_layout) {  // channels 4w .. 4w+3 share a nibble position in four consecutive bytes
                                const uint32_t word = *(const uint32_t*)(s.kc + tt * RS + code_pos(B200KV_FMT_Q4_0, 128, 0, 4 * w));
                                const int sh = 4 * code_nibble(B200KV_FMT_Q4_0, 128, 0, 4 * w);
#pragma unroll
                                for (int e = 0; e < 4; e++) codes[e] = (word >> (8 * e + sh)) & 0xfu;
                            } else {
                                const uint32_t half = *(const uint16_t*)(s.kc + tt * RS + 2 * w);
#pragma unroll
                                for (int e = 0; e < 4; e++) codes[e] = (half >> (4 * e)) & 0xfu;
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 4; e++) kx[e] = kivi_dequant(codes[e], s.kpar[4 * w + e], s.kpar[D + 4 * w + e]);
                    }
#pragma unroll
                    for (int e = 0; e < 4; e++)
#pragma unroll
                        for (int g = 0; g < KGT; g++) dot[g] = fmaf(q_s[g * D + 4 * w + e], kx[e], dot[g]);
                }
            }
#pragma unroll
            for (int g = 0; g < KGT; g++) {
                dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 1);
                dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 2);
            }
            if (part == 0) {
#pragma unroll
                for (int g = 0; g < KGT; g++) sc_s[g * KTILE + tt] = dot[g] * p.scale;
            }
        }
        __syncthreads();
        if (warp < KGT) {  // online softmax of head `warp`: one lane per token of the tile
            const float sv = lane < n_valid ? sc_s[warp * KTILE + lane] : -INFINITY;
            float mx = sv;
#pragma unroll
            for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_new = fmaxf(m_run, mx);
            const float a = expf(m_run - m_new), pw = expf(sv - m_new);
            float sum = pw;
#pragma unroll
            for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            l_run = l_run * a + sum, m_run = m_new;
            sc_s[warp * KTILE + lane] = pw;
            if (lane == 0) alpha_s[warp] = a;
        }
        __syncthreads();
        if (tid < D) {
#pragma unroll
            for (int g = 0; g < KGT; g++) acc[g] *= alpha_s[g];
            for (int tt = 0; tt < n_valid; tt++) {
                float vx;
                if (tile < 0) {
                    vx = sink_v[tt * D + tid];
                } else {
                    const uint32_t byte = s.vc[tt * RS + v_pos];
                    const uint32_t code = eight ? byte : (v_nib ? byte >> 4 : byte & 0xfu);
                    vx = kivi_dequant(code, s.vpar[2 * tt], s.vpar[2 * tt + 1]);
                }
#pragma unroll
                for (int g = 0; g < KGT; g++) acc[g] = fmaf(sc_s[g * KTILE + tt], vx, acc[g]);
            }
        }
        __syncthreads();  // the stage and sc_s are free again
    }
    cp_async_wait<0>();
    if (warp < KGT && lane == 0) ml_s[warp * 2] = m_run, ml_s[warp * 2 + 1] = l_run;
    __syncthreads();
    const int64_t pbase = (((int64_t)b * p.part_stride + p.part_off + split) * v.H + kvh) * p.G + g0;
    if (tid < D)
        for (int g = 0; g < ng; g++) p.part_o[(pbase + g) * D + tid] = acc[g];
    if (tid < ng) p.part_ml[(pbase + tid) * 2] = ml_s[tid * 2], p.part_ml[(pbase + tid) * 2 + 1] = ml_s[tid * 2 + 1];
}

template <int D>
__global__ void __launch_bounds__(128) kivi_decode_kernel(KiviDecode p, const __grid_constant__ InlineBatch ib) {
    __shared__ __align__(16) KiviSimtSmem<D> sm;
    kivi_simt_body<D>(p, ib, sm, blockIdx.x, blockIdx.y, blockIdx.z);
}

}  // namespace b200kv
