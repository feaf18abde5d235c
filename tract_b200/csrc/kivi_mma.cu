// Tensor-core decode attention over the finalised part of a KIVI int8 / int4 cache (head_dim 128, 16-bit queries).
//
// The stores are those of transformers/src/ops/quant_dyn_kv_cache.rs: Keys per channel and 32-token block
// (K^[t][c] = lo_b[c] + scale_b[c] * u[t][c], :231-240), Values per token (V^[t][c] = lo_t + scale_t * u[t][c],
// :141-146).  The CPU op rebuilds the whole f32 cache every step (:432-449) and hands it to Sdpa; the CUDA-core
// kernel in kivi.cu dequantises element by element and is issue bound at a sixth of the HBM rate.  Here, as in
// decode_mma.cu, the q-head group sits in the N dimension of mma.sync.m16n8k16 (M = 16 cached tokens per warp):
//   K side: q . K^[t] = q . lo_b + sum_c (q[c] * scale_b[c]) * u[t][c].  Once per block the four warps rebuild the B
//           operand q' = q * scale_b as an f16 value plus its f16 remainder (two MMAs per k-step, exact to 2^-22) and
//           the scalar q . lo_b in f32; a code byte placed in the low byte of an f16 is the subnormal u * 2^-24, which
//           the tensor cores multiply exactly, so the codes enter the MMA after a byte permute and nothing else (int4:
//           a mask; the high nibbles are used in place as 16 * code, with 1/16 folded into the matching part of q');
//   V side: V^[t][c] = m_t + scale_t * (u[t][c] - k_t), with k_t the code of the value 0 (clamped to 0..255) and
//           m_t = lo_t + scale_t * k_t.  The per-token scale is folded into the softmax weights before they are rounded
//           to f16, the codes enter the MMA as u * 2^-24, and the scalars sum_t w_t k_t (rounded weights) and
//           sum_t p_t m_t (exact weights) are kept per head.  Centring on the code of zero makes the rounding of a
//           weight meet the value itself and not its distance from lo_t, which an outlier in the row makes large;
// A CTA walks a run of 64-token pages of one (sequence, kv head); the four arrays of a page (K codes, V codes,
// K parameters, V parameters) arrive by cp.async.bulk into one stage of a ring; one CTA barrier per page hands the
// stage back to thread 0, which refills it at once with a page id it fetched from the page table one iteration
// earlier.  (A ring with full / empty barrier pairs, a pair-of-warps barrier and a refill one page late measured 20 %
// slower: with three stages, one of which the look-ahead of the q' rebuild holds, a late refill leaves nothing in flight.)  Sinks, the f32 residual block and
// the value tokens that go with it are left to the CUDA-core formulation (kivi_simt.cuh), run by a few extra CTAs of
// the same grid, which publish them as one more partial per sequence.
#include <algorithm>

#include "decode_common.h"
#include "kivi_simt.cuh"
#include "mma_common.cuh"

namespace b200kv {

constexpr int KM_D = 128;
constexpr int KM_KP = 2 * 2 * KM_D * 4;                   // 2 blocks x (lo[D], scale[D]) f32
constexpr int KM_VP = PAGE_TOKENS * 2 * 4;                // (lo, scale) f32 per token
template <int BITS>
struct KGeo {
    static constexpr int FMT = BITS == 8 ? B200KV_FMT_Q8_1 : B200KV_FMT_Q4_0;  // the block format whose row layout the codes borrow
    static constexpr int KC = PAGE_TOKENS * KM_D * BITS / 8;                   // bytes of K (or V) codes per page and head
    static constexpr int STAGE = 2 * KC + KM_KP + KM_VP;                       // 18944 / 10752
    static constexpr float LV = BITS == 8 ? 255.f : 15.f;
    static constexpr int NS = 3;                     // stages
    static constexpr int CTAS = BITS == 8 ? 3 : 4;   // resident CTAs per SM (73.5 KB / 48.9 KB each); measured: a fourth CTA with 2 stages loses for int8
};
constexpr int KM_PARAMS = 2 * (2 * 8 * 32 * 16 + 2 * 2 * 8 * 4);  // two buffers of: q' fragments [2 blocks][8 k-steps][32 lanes], q . lo [2 blocks][2 halves][8 heads]
constexpr float KM_PSCALE = 64.f;                         // softmax weights * V scale are lifted away from the f16 subnormals

// First of the four channels that k-step s holds for the thread with lane % 4 = c.  int8: s = 2 grp + hh covers channels
// 32 grp + 8c + 4hh + {0,1 | 2,3}; int4: 32 grp + 16 hh + 4c + {0,1 | 2,3} (hh = 1: the high nibbles).
template <int BITS>
__host__ __device__ constexpr int kstep_channel(int s, int c) {
    return BITS == 8 ? 32 * (s >> 1) + 8 * c + 4 * (s & 1) : 32 * (s >> 1) + 16 * (s & 1) + 4 * c;
}

struct KiviMmaParams {
    KiviView v;
    const void* q;
    int64_t qb, qh;
    float* part_o;
    float* part_ml;
    int* status;
    int32_t G, dtype, n_splits, part_stride, part_off;
    int32_t n_mma_ctas;  // blockIdx.x below this: tensor-core work; from it on: the f32 tiles, one CTA per (sequence, group of 4 heads)
    float scale;
};

template <int BITS>
__global__ void __launch_bounds__(128, KGeo<BITS>::CTAS) kivi_mma_kernel(KiviMmaParams p, const __grid_constant__ InlineBatch ib) {
    using Kg = KGeo<BITS>;
    constexpr int KM_KC = Kg::KC, KM_STAGE = Kg::STAGE, CFMT = Kg::FMT, KM_NS = Kg::NS;
    constexpr float LOG2E = 1.4426950408889634f;
    constexpr float TWO24 = 16777216.f;
    extern __shared__ __align__(1024) uint8_t stages[];
    uint4* qp_s = (uint4*)(stages + (size_t)KM_NS * KM_STAGE);  // B fragments of q' = q * scale: {hi k0..1, hi k2..3, lo k0..1, lo k2..3}
    float* bias_s = (float*)(qp_s + 2 * 2 * 8 * 32);            // q . lo of each block, in two halves of the channels
    float* q_s = (float*)(qp_s + 2 * 8 * 32);                   // [8][128] f32 during the set-up only: the second q' buffer, first written after a barrier
    uint64_t* bars = (uint64_t*)(bias_s + 2 * 2 * 2 * 8);  // [NS] the bytes of the stage have landed

    const KiviView& v = p.v;
    const int kvh_simt = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, c = lane & 3;
    const int bxm = min((int)blockIdx.x, p.n_mma_ctas - 1);  // the extra CTAs (f32 tiles) branch off below; keep their indices in range
    const int b = bxm / p.n_splits, split = bxm % p.n_splits;
    const int kvh = blockIdx.y, g0 = blockIdx.z * 8, ng = min(8, p.G - g0);
    const int32_t seq = ib.ent[b].x;
    const int len = ib.ent[b].y;
    const int n_fin = max(len - SINK, 0) / KBLOCK;  // finalised key blocks; their 32 * n_fin tokens are this kernel's
    const int n_pg = (n_fin + 1) / 2;
    const int pg_lo = (int)((int64_t)n_pg * split / p.n_splits), pg_hi = (int)((int64_t)n_pg * (split + 1) / p.n_splits);
    const int n_tiles = pg_hi - pg_lo;

    const int32_t* trow_p = v.table + (int64_t)seq * v.max_pages_per_seq + pg_lo;
    auto issue = [&](int i, int32_t pg) {  // thread 0 only
        const int st = i % KM_NS;
        if (pg < 0 || pg >= v.n_pages) {
            atomicOr(p.status, STATUS_PAGE_OOB);
            pg = 0;
        }
        const int64_t ph = (int64_t)pg * v.H + kvh;
        uint8_t* dst = stages + (size_t)st * KM_STAGE;
        mbar_expect_tx(&bars[st], KM_STAGE);
        bulk_g2s(dst, v.codes[0] + ph * KM_KC, KM_KC, &bars[st]);
        bulk_g2s(dst + KM_KC, v.codes[1] + ph * KM_KC, KM_KC, &bars[st]);
        bulk_g2s(dst + 2 * KM_KC, v.params[0] + ph * (KM_KP / 4), KM_KP, &bars[st]);
        bulk_g2s(dst + 2 * KM_KC + KM_KP, v.params[1] + ph * (KM_VP / 4), KM_VP, &bars[st]);
    };
    grid_dependency_wait();    // the append that precedes this launch has written its pages
    grid_launch_dependents();
    if ((int)blockIdx.x >= p.n_mma_ctas) {  // CTA-uniform: sinks + residual block of one sequence on the CUDA cores
        if (blockIdx.z != 0) return;
        KiviDecode d;
        d.v = p.v, d.q = p.q, d.qb = p.qb, d.qh = p.qh, d.part_o = p.part_o, d.part_ml = p.part_ml;
        d.G = p.G, d.dtype = p.dtype, d.n_splits = 1, d.f32_only = 1, d.part_stride = p.part_stride, d.part_off = 0, d.scale = p.scale;
        const int nzs = (p.G + KGT - 1) / KGT, e = (int)blockIdx.x - p.n_mma_ctas;
        kivi_simt_body<KM_D>(d, ib, *reinterpret_cast<KiviSimtSmem<KM_D>*>(stages), e / nzs, kvh_simt, e % nzs);
        return;
    }
    int32_t pg_next = 0;  // thread 0: id of the next page to request
    if (tid == 0) {
        for (int s = 0; s < KM_NS; s++) mbar_init(&bars[s], 1);
        mbar_fence_init();
        int32_t first[KM_NS];
#pragma unroll
        for (int i = 0; i < KM_NS; i++) first[i] = i < n_tiles ? trow_p[i] : 0;  // the loads travel together
#pragma unroll
        for (int i = 0; i < KM_NS; i++)
            if (i < n_tiles) issue(i, first[i]);
        if (KM_NS < n_tiles) pg_next = trow_p[KM_NS];
    }
    // q of the group, rounded to the f16 operand the tensor cores will see; rows beyond the group zero
    for (int idx = tid; idx < 8 * KM_D; idx += 128) {
        const int g = idx / KM_D, ch = idx % KM_D;
        float x = 0.f;
        if (g < ng) x = ld_as_f32(p.q, p.dtype, (int64_t)b * p.qb + (int64_t)(kvh * p.G + g0 + g) * p.qh + ch);
        q_s[idx] = __half2float(__float2half_rn(x));
    }
    __syncthreads();
    // This thread's share of the per-block rebuild of q': head n = lane / 4, the 16 channels of k-steps 4 hf .. 4 hf + 3
    // (k-step s = 2 * grp + hh covers channels 32 grp + 8c + 4hh + {0,1 | 2,3}), hf = warp & 1.
    const int hf = warp & 1;
    float qf[16];
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) qf[4 * j + e] = q_s[r * KM_D + kstep_channel<BITS>(4 * hf + j, c) + e];
    const float sl2 = p.scale * LOG2E;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_part[2] = {0.f, 0.f};
    float o[8][4];            // O^T fragments: m-tile j = channels 16j..16j+15, columns = heads 2c, 2c+1
    float ob[2] = {0.f, 0.f};  // sum_t p_t * m_t over this thread's two token rows, heads 2c and 2c + 1
    float oc[2] = {0.f, 0.f};  // sum_t w_t * k_t with w_t the rounded f16 weights (p_t * scale_t * KM_PSCALE)
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[j][e] = 0.f;
    bool failed = false;
    const int tA = warp * 16 + r, tB = tA + 8;  // the two token rows of this thread's C fragments
    const int blk = warp >> 1;                  // the key block of this warp's tokens

    // q' = q * scale of this warp's key block of page i (k-steps 4 hf .. 4 hf + 3) and its share of q . lo, into buffer i & 1
    auto build = [&](int i) {
        const float* Kp = (const float*)(stages + (size_t)(i % KM_NS) * KM_STAGE + 2 * KM_KC);
        const int n_valid = min(PAGE_TOKENS, n_fin * KBLOCK - (pg_lo + i) * PAGE_TOKENS);
        uint4* qp_w = qp_s + (i & 1) * (2 * 8 * 32);
        float* bias_w = bias_s + (i & 1) * (2 * 2 * 8);
        if (warp * 16 < n_valid) {
            const float* lo_p = Kp + blk * 2 * KM_D;
            const float* sc_p = lo_p + KM_D;
            float bpart[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int ks = 4 * hf + j, k0 = kstep_channel<BITS>(ks, c);
                const float4 sc = *(const float4*)(sc_p + k0), lo = *(const float4*)(lo_p + k0);
                const float hn = (BITS == 4 && (ks & 1)) ? 0.0625f : 1.f;  // int4: the odd k-steps meet high nibbles in place, 16 * code
                const float x0 = qf[4 * j] * sc.x * hn, x1 = qf[4 * j + 1] * sc.y * hn, x2 = qf[4 * j + 2] * sc.z * hn, x3 = qf[4 * j + 3] * sc.w * hn;
                const __half2 h01 = __floats2half2_rn(x0, x1), h23 = __floats2half2_rn(x2, x3);
                const __half2 l01 = __floats2half2_rn(x0 - __low2float(h01), x1 - __high2float(h01));
                const __half2 l23 = __floats2half2_rn(x2 - __low2float(h23), x3 - __high2float(h23));
                qp_w[(blk * 8 + ks) * 32 + lane] =
                    make_uint4(*(const uint32_t*)&h01, *(const uint32_t*)&h23, *(const uint32_t*)&l01, *(const uint32_t*)&l23);
                bpart[j] = fmaf(qf[4 * j], lo.x, fmaf(qf[4 * j + 1], lo.y, fmaf(qf[4 * j + 2], lo.z, qf[4 * j + 3] * lo.w)));
            }
            float bsum = (bpart[0] + bpart[1]) + (bpart[2] + bpart[3]);
            bsum += __shfl_xor_sync(0xffffffffu, bsum, 1);
            bsum += __shfl_xor_sync(0xffffffffu, bsum, 2);
            if (c == 0) bias_w[(blk * 2 + hf) * 8 + r] = bsum;
        }
    };
    {  // page 0 is built before the loop, page i + 1 while page i is consumed: one barrier per page
        const bool ok0 = n_tiles == 0 || mbar_wait_bounded(&bars[0], 0);
        if (n_tiles && ok0) build(0);
        failed = __syncthreads_or(!ok0) != 0;
    }
    for (int i = 0; i < n_tiles && !failed; i++) {
        const int st = i % KM_NS;
        bool ok = true;
        if (i + 1 < n_tiles) {  // a warp whose wait ran out walks on to the CTA barrier below, where every warp learns of it
            ok = mbar_wait_bounded(&bars[(i + 1) % KM_NS], (uint32_t)(((i + 1) / KM_NS) & 1));
            if (ok) build(i + 1);
        }
        const uint8_t* Kc = stages + (size_t)st * KM_STAGE;
        const uint8_t* Vc = Kc + KM_KC;
        const float* Kp = (const float*)(Vc + KM_KC);
        const float* Vp = Kp + KM_KP / 4;
        const int n_valid = min(PAGE_TOKENS, n_fin * KBLOCK - (pg_lo + i) * PAGE_TOKENS);  // 32 or 64
        if (warp * 16 < n_valid) {  // warp-uniform; whole 16-token groups are live or dead (n_valid is 32 or 64)
            // ================= scores: S^T[16 tokens x 8 heads] = K^ . Q^T =================
            float sacc[4] = {0.f, 0.f, 0.f, 0.f};
            const uint4* qp = qp_s + (i & 1) * (2 * 8 * 32) + blk * 8 * 32 + lane;
#pragma unroll
            for (int g = 0; g < 4; g++) {
                uint32_t xa[2], xb[2];  // this thread's codes of channel group g, rows tA and tB, first and second k-step
                if constexpr (BITS == 8) {
                    const uint2 wa = *(const uint2*)(Kc + chunk_addr(CFMT, KM_D, 0, tA, 32 * g + 8 * c));
                    const uint2 wb = *(const uint2*)(Kc + chunk_addr(CFMT, KM_D, 0, tB, 32 * g + 8 * c));
                    xa[0] = wa.x, xa[1] = wa.y, xb[0] = wb.x, xb[1] = wb.y;
                } else {  // bytes 4c .. 4c+3 of the group: low nibbles = channels 32g + 4c + 0..3, high nibbles = 32g + 16 + 4c + 0..3
                    const uint32_t wa = *(const uint32_t*)(Kc + chunk_addr(CFMT, KM_D, 0, tA, 16 * g + 4 * c));
                    const uint32_t wb = *(const uint32_t*)(Kc + chunk_addr(CFMT, KM_D, 0, tB, 16 * g + 4 * c));
                    xa[0] = wa & 0x0f0f0f0fu, xa[1] = wa & 0xf0f0f0f0u, xb[0] = wb & 0x0f0f0f0fu, xb[1] = wb & 0xf0f0f0f0u;
                }
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const uint4 w = qp[(2 * g + hh) * 32];
                    uint32_t a[4];
                    a[0] = __byte_perm(xa[hh], 0, 0x4140), a[1] = __byte_perm(xb[hh], 0, 0x4140);
                    a[2] = __byte_perm(xa[hh], 0, 0x4342), a[3] = __byte_perm(xb[hh], 0, 0x4342);
                    mma_f16(sacc, a, w.x, w.y);
                    mma_f16(sacc, a, w.z, w.w);
                }
            }
            // ================= online softmax (log2 domain), heads 2c and 2c + 1 =================
            const float* bias_r = bias_s + (i & 1) * (2 * 2 * 8);
            const float2 bh0 = *(const float2*)(bias_r + (blk * 2) * 8 + 2 * c), bh1 = *(const float2*)(bias_r + (blk * 2 + 1) * 8 + 2 * c);
            const float bias0 = bh0.x + bh1.x, bias1 = bh0.y + bh1.y;
            const float s0 = fmaf(sacc[0], TWO24, bias0) * sl2, s1 = fmaf(sacc[1], TWO24, bias1) * sl2;
            const float s2 = fmaf(sacc[2], TWO24, bias0) * sl2, s3 = fmaf(sacc[3], TWO24, bias1) * sl2;
            // the reference maximum of a head is raised only when a score of this warp exceeds it by more than 2 (one
            // warp-wide vote per page instead of two cross-lane maxima, a rescale test and the correction exponentials)
            const float lm0 = fmaxf(s0, s2), lm1 = fmaxf(s1, s3);
            float al0 = 1.f, al1 = 1.f;
            const bool raise = __any_sync(0xffffffffu, lm0 > m_run[0] + 1.f || lm1 > m_run[1] + 1.f);
            if (raise) {
                const float mn0 = fmaxf(m_run[0], quad_row_max(lm0)), mn1 = fmaxf(m_run[1], quad_row_max(lm1));
                al0 = fast_ex2(m_run[0] - mn0), al1 = fast_ex2(m_run[1] - mn1);  // every token here is live: the maxima are finite
                m_run[0] = mn0, m_run[1] = mn1;
            }
            const float p0 = fast_ex2(s0 - m_run[0]), p1 = fast_ex2(s1 - m_run[1]), p2 = fast_ex2(s2 - m_run[0]), p3 = fast_ex2(s3 - m_run[1]);
            l_part[0] = fmaf(l_part[0], al0, p0 + p2);
            l_part[1] = fmaf(l_part[1], al1, p1 + p3);
            const float2 vpA = *(const float2*)(Vp + tA * 2), vpB = *(const float2*)(Vp + tB * 2);  // (lo, scale) of the two tokens
            const float kA = fminf(fmaxf(rintf(__fdividef(-vpA.x, vpA.y)), 0.f), Kg::LV);
            const float kB = fminf(fmaxf(rintf(__fdividef(-vpB.x, vpB.y)), 0.f), Kg::LV);
            const float mA = fmaf(kA, vpA.y, vpA.x), mB = fmaf(kB, vpB.y, vpB.x);
            // weights times the token's scale, rounded once to f16, then transposed into B fragments
            const float fA = vpA.y * KM_PSCALE, fB = vpB.y * KM_PSCALE;
            const uint32_t hA = pack_f16(p0 * fA, p1 * fA), hB = pack_f16(p2 * fB, p3 * fB);
            const float2 wA = __half22float2(*(const __half2*)&hA), wB = __half22float2(*(const __half2*)&hB);
            ob[0] = fmaf(ob[0], al0, fmaf(p0, mA, p2 * mB));
            ob[1] = fmaf(ob[1], al1, fmaf(p1, mA, p3 * mB));
            oc[0] = fmaf(oc[0], al0, fmaf(wA.x, kA, wB.x * kB));
            oc[1] = fmaf(oc[1], al1, fmaf(wA.y, kA, wB.y * kB));
            if (raise) {
#pragma unroll
                for (int j = 0; j < 8; j++) o[j][0] *= al0, o[j][1] *= al1, o[j][2] *= al0, o[j][3] *= al1;
            }
            // ================= O^T[128 ch x 8 heads] += V^T . P^T =================
            const uint32_t pb0 = movmatrix_trans(hA);  // tokens 2c, 2c+1 of head n
            const uint32_t pb1 = movmatrix_trans(hB);  // tokens 2c+8, 2c+9
            const int T0 = warp * 16 + 2 * c;
            if constexpr (BITS == 8) {
                uint4 x[4];  // 16 bytes at positions 16r.. of each row: channel slot (r | r + 8) of every m-tile
                x[0] = *(const uint4*)(Vc + chunk_addr(CFMT, KM_D, 1, T0, 16 * r));
                x[1] = *(const uint4*)(Vc + chunk_addr(CFMT, KM_D, 1, T0 + 1, 16 * r));
                x[2] = *(const uint4*)(Vc + chunk_addr(CFMT, KM_D, 1, T0 + 8, 16 * r));
                x[3] = *(const uint4*)(Vc + chunk_addr(CFMT, KM_D, 1, T0 + 9, 16 * r));
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint32_t w0 = (&x[0].x)[j >> 1], w1 = (&x[1].x)[j >> 1], w2 = (&x[2].x)[j >> 1], w3 = (&x[3].x)[j >> 1];
                    const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
                    const uint32_t u01 = __byte_perm(w0, w1, sel);  // [T0.b2j, T0.b2j+1, T1.b2j, T1.b2j+1]
                    const uint32_t u23 = __byte_perm(w2, w3, sel);
                    uint32_t a[4];
                    a[0] = __byte_perm(u01, 0, 0x4240), a[1] = __byte_perm(u01, 0, 0x4341);
                    a[2] = __byte_perm(u23, 0, 0x4240), a[3] = __byte_perm(u23, 0, 0x4341);
                    mma_f16(o[j], a, pb0, pb1);
                }
            } else {
                uint2 x[4];  // 8 bytes at positions 8r..: byte j = slot r (low nibble) | slot r + 8 (high) of m-tile j
                x[0] = *(const uint2*)(Vc + chunk_addr(CFMT, KM_D, 1, T0, 8 * r));
                x[1] = *(const uint2*)(Vc + chunk_addr(CFMT, KM_D, 1, T0 + 1, 8 * r));
                x[2] = *(const uint2*)(Vc + chunk_addr(CFMT, KM_D, 1, T0 + 8, 8 * r));
                x[3] = *(const uint2*)(Vc + chunk_addr(CFMT, KM_D, 1, T0 + 9, 8 * r));
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {  // m-tiles 2jj and 2jj + 1
                    const uint32_t w0 = (&x[0].x)[jj >> 1], w1 = (&x[1].x)[jj >> 1], w2 = (&x[2].x)[jj >> 1], w3 = (&x[3].x)[jj >> 1];
                    const uint32_t sel = (jj & 1) ? 0x7632u : 0x5410u;
                    const uint32_t u01 = __byte_perm(w0, w1, sel), u23 = __byte_perm(w2, w3, sel);
                    // high nibbles in place (16 * code): rows r + 8 of O^T come out 16 times too large, undone at the end
                    const uint32_t lo01 = u01 & 0x0f0f0f0fu, hi01 = u01 & 0xf0f0f0f0u;
                    const uint32_t lo23 = u23 & 0x0f0f0f0fu, hi23 = u23 & 0xf0f0f0f0u;
                    uint32_t a[4];
                    a[0] = __byte_perm(lo01, 0, 0x4240), a[1] = __byte_perm(hi01, 0, 0x4240);
                    a[2] = __byte_perm(lo23, 0, 0x4240), a[3] = __byte_perm(hi23, 0, 0x4240);
                    mma_f16(o[2 * jj], a, pb0, pb1);
                    a[0] = __byte_perm(lo01, 0, 0x4341), a[1] = __byte_perm(hi01, 0, 0x4341);
                    a[2] = __byte_perm(lo23, 0, 0x4341), a[3] = __byte_perm(hi23, 0, 0x4341);
                    mma_f16(o[2 * jj + 1], a, pb0, pb1);
                }
            }
        }
        if (__syncthreads_or(!ok)) {  // every warp is done with stage st and has built its share of the next page
            failed = true;
            break;
        }
        if (tid == 0 && i + KM_NS < n_tiles) {
            issue(i + KM_NS, pg_next);
            if (i + KM_NS + 1 < n_tiles) pg_next = trow_p[i + KM_NS + 1];
        }
    }

    // ---- merge the four warps and publish the partial of this split ----
    const int64_t pbase = (((int64_t)b * p.part_stride + p.part_off + split) * v.H + kvh) * p.G + g0;
    if (failed) {
        if (tid == 0) atomicOr(p.status, STATUS_WAIT_EXPIRED);
        for (int idx = tid; idx < ng * KM_D; idx += 128) p.part_o[(pbase + idx / KM_D) * KM_D + idx % KM_D] = 0.f;
        if (tid < ng) p.part_ml[(pbase + tid) * 2] = -INFINITY, p.part_ml[(pbase + tid) * 2 + 1] = 0.f;
        return;
    }
    float* om = (float*)stages;      // [4 warps][8 heads][128 ch]; every stage is consumed by now
    float* ml = om + 4 * 8 * KM_D;   // [4 warps][8 heads][2]
    const float l0 = quad_row_sum(l_part[0]), l1 = quad_row_sum(l_part[1]);
    // sum_t p_t m_t - sum_t w_t k_t / KM_PSCALE, complete over the warp's 16 tokens
    const float b0 = quad_row_sum(fmaf(oc[0], -1.f / KM_PSCALE, ob[0])), b1 = quad_row_sum(fmaf(oc[1], -1.f / KM_PSCALE, ob[1]));
    if (r == 0) {
        ml[(warp * 8 + 2 * c) * 2] = m_run[0], ml[(warp * 8 + 2 * c) * 2 + 1] = l0;
        ml[(warp * 8 + 2 * c + 1) * 2] = m_run[1], ml[(warp * 8 + 2 * c + 1) * 2 + 1] = l1;
    }
    constexpr float UNDO = TWO24 / KM_PSCALE, UNDO_HI = BITS == 4 ? UNDO / 16.f : UNDO;  // int4: rows r + 8 carry 16 * code
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float* base = om + (warp * 8 + 2 * c) * KM_D + 16 * j + r;
        base[0] = fmaf(o[j][0], UNDO, b0), base[KM_D] = fmaf(o[j][1], UNDO, b1);
        base[8] = fmaf(o[j][2], UNDO_HI, b0), base[KM_D + 8] = fmaf(o[j][3], UNDO_HI, b1);
    }
    __syncthreads();
    for (int idx = tid; idx < ng * KM_D; idx += 128) {
        const int g = idx / KM_D, ch = idx % KM_D;
        float M = -INFINITY;
#pragma unroll
        for (int wv = 0; wv < 4; wv++) M = fmaxf(M, ml[(wv * 8 + g) * 2]);
        float num = 0.f;
#pragma unroll
        for (int wv = 0; wv < 4; wv++) {
            const float mw = ml[(wv * 8 + g) * 2];
            if (mw > -INFINITY) num = fmaf(exp2f(mw - M), om[(wv * 8 + g) * KM_D + ch], num);
        }
        p.part_o[(pbase + g) * KM_D + ch] = num;
    }
    if (tid < ng) {
        float M = -INFINITY, den = 0.f;
        for (int wv = 0; wv < 4; wv++) M = fmaxf(M, ml[(wv * 8 + tid) * 2]);
        for (int wv = 0; wv < 4; wv++) {
            const float mw = ml[(wv * 8 + tid) * 2];
            if (mw > -INFINITY) den = fmaf(exp2f(mw - M), ml[(wv * 8 + tid) * 2 + 1], den);
        }
        p.part_ml[(pbase + tid) * 2] = M * 0.6931471805599453f;  // natural-log units for the combine pass
        p.part_ml[(pbase + tid) * 2 + 1] = den;
    }
}

bool kivi_mma_supported(const b200kv_cache* c, int dtype) {
    return c->cfg.head_dim == KM_D && c->cfg.has_values && (dtype == B200KV_F16 || dtype == B200KV_BF16);
}

int launch_kivi_mma(b200kv_cache* c, const void* q, const int64_t* qs, int n_seqs, int G, int dtype, float scale, int n_splits,
                    float* part_o, float* part_ml, const InlineBatch& ib, cudaStream_t stream) {
    KiviMmaParams p{};
    p.v = kivi_view(c);
    p.q = q, p.qb = qs[0], p.qh = qs[1];
    p.part_o = part_o, p.part_ml = part_ml, p.status = c->d_status;
    p.G = G, p.dtype = dtype, p.n_splits = n_splits, p.part_stride = n_splits + 1, p.part_off = 1;
    p.n_mma_ctas = n_seqs * n_splits;
    p.scale = scale;
    dim3 grid(n_seqs * n_splits + n_seqs * ((G + KGT - 1) / KGT), c->cfg.n_kv_heads, (G + 7) / 8);
    // ring (reused by the warp merge, 17 KB), q' fragments and q . lo, barriers
    if (c->kivi.bits == 8) {
        const size_t smem = (size_t)KGeo<8>::NS * KGeo<8>::STAGE + KM_PARAMS + 64;
        B200KV_CUDA(cudaFuncSetAttribute(kivi_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        B200KV_CUDA(launch_after_predecessor(kivi_mma_kernel<8>, grid, dim3(128), smem, stream, p, ib));
    } else {
        const size_t smem = (size_t)KGeo<4>::NS * KGeo<4>::STAGE + KM_PARAMS + 64;
        B200KV_CUDA(cudaFuncSetAttribute(kivi_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        B200KV_CUDA(launch_after_predecessor(kivi_mma_kernel<4>, grid, dim3(128), smem, stream, p, ib));
    }
    return B200KV_OK;
}

}  // namespace b200kv

namespace b200kv {
int kivi_mma_ctas_per_sm(int bits) { return bits == 8 ? KGeo<8>::CTAS : KGeo<4>::CTAS; }
}  // namespace b200kv
