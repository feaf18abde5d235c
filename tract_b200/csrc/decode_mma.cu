// Tensor-core formulation of the split-KV GQA decode kernel for head_dim 128 and 16-bit queries:
// f16 / bf16 caches and the block-quantised Q8_1 / Q4_0 caches.
//
// Why tensor cores in an HBM-bound kernel: with 4..8 query heads sharing every K/V byte, the dot
// products done on CUDA cores cost ~0.3 warp instructions per byte for int8 codes and the kernel
// becomes issue bound at a third of the HBM rate.  Here the q-head group is packed into the N
// dimension of mma.sync.m16n8k16 tiles (M = 16 cached tokens), which takes the FMAs out of the issue
// slots; what is left per byte is the widening of codes to f16, done with byte permutes only:
//   - an unsigned byte u placed in the low byte of an f16 is the subnormal u * 2^-24, exact, and the
//     tensor cores multiply subnormals exactly; the 2^24 is folded into the per-block scale;
//   - codes are stored offset-binary (Q8_1: code + 128, Q4_0: nibble = code + 8), so the offset is a
//     rank-one term: for K it is 128 * sum(q) per block (computed once per CTA), for V it is produced
//     by one extra mma per block whose A operand is the constant 128 (resp. 8).
// Scales are applied outside the integer products (per 32-channel block for K, folded into the
// probabilities for V), so the products themselves are exact as in the CPU's f32 dequantise-then-dot.
//
// Each warp owns 16 of the 64 tokens of a page with its own running (max, sum, O) state; warps meet
// once, at the end.  Chunks arrive by cp.async.bulk into a ring of stages, one mbarrier per stage; one
// CTA barrier per page hands the stage back to thread 0, which refills it at once with a page id it
// fetched from the page table one iteration earlier (the table read is off the critical path).
// (Measured against a ring with full / empty barrier pairs, no CTA barrier and a refill one page late:
// that lost 7 % on the 4-bit cache, because the ring runs one stage shallower.)
// Semantics: transformers/src/ops/flash_sdpa.rs:239-341 with S = 1; replaces the decode use of
// cuda/src/kernels/cu/flash_attn.cu.
#include <algorithm>
#include <cmath>
#include <vector>

#include "decode_common.h"
#include "mma_common.cuh"

namespace b200kv {

constexpr int MD = 128;  // head_dim of this kernel

template <int FMT>
struct MGeo {
    static constexpr bool QUANT = FMT == B200KV_FMT_Q8_1 || FMT == B200KV_FMT_Q4_0;
    static constexpr int ROW = FMT == B200KV_FMT_Q8_1 ? MD : FMT == B200KV_FMT_Q4_0 ? MD / 2 : MD * 2;
    static constexpr int DATA = PAGE_TOKENS * ROW;
    static constexpr int SCALES = QUANT ? PAGE_TOKENS * (MD / 32) * 2 : 0;
    static constexpr int CHUNK = DATA + SCALES;
    static constexpr int STAGE = 2 * CHUNK;
    static constexpr int NS = FMT == B200KV_FMT_Q4_0 ? 5 : (QUANT ? 4 : 3);
    // measured: Q8_1 is best with 3 CTAs x 4 stages, Q4_0 with 4 CTAs x 5 stages, the 16-bit formats are HBM bound at 2
    static constexpr int MIN_CTAS = FMT == B200KV_FMT_Q4_0 ? 4 : (QUANT ? 3 : 2);  // resident CTAs per SM the register budget is set for
};

// Shared memory after the stage ring: q as f32 [8][128], then the barriers.
constexpr size_t MMA_TAIL = 8 * MD * 4 + 32 * 4 + 128;

template <int FMT>
__global__ void __launch_bounds__(128, MGeo<FMT>::MIN_CTAS) decode_mma_kernel(DecodeParams p, const __grid_constant__ InlineBatch ib) {
    using Gm = MGeo<FMT>;
    constexpr int NS = Gm::NS;
    constexpr bool QUANT = Gm::QUANT;
    constexpr bool IS_BF16 = FMT == B200KV_FMT_BF16;
    constexpr float LOG2E = 1.4426950408889634f;
    // code offset (Q8_1 bytes hold code + 128, Q4_0 nibbles hold code + 8) and the constant A operand carrying it
    constexpr float OFFS = FMT == B200KV_FMT_Q8_1 ? 128.f : 8.f;
    constexpr uint32_t OFFS_FRAG = FMT == B200KV_FMT_Q8_1 ? 0x00800080u : 0x00080008u;
    constexpr float TWO24 = 16777216.f;
    constexpr float PSCALE = 1024.f;  // probabilities * V scale are lifted into the normal f16 range
    constexpr float LAZY_MAX = 1.f;   // see the softmax below

    // declared aligned (not rounded up by hand) so that the compiler keeps every access in the shared window
    extern __shared__ __align__(1024) uint8_t stages[];
    float* q_s = (float*)(stages + (size_t)NS * Gm::STAGE);  // [8][128]
    float* qsum_s = q_s + 8 * MD;                             // [8 heads][4 blocks]
    uint64_t* bars = (uint64_t*)(qsum_s + 32);     // [NS] the bytes of the stage have landed

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, c = lane & 3;
    const WorkItem w = ib.n ? resolve_work_item(ib, blockIdx.x) : p.items[blockIdx.x];
    const int kvh = blockIdx.y;
    const int g0 = blockIdx.z * 8;
    const int ng = min(8, p.G - g0);  // q heads of this CTA
    const int n_tiles = w.n_pages;

    const int32_t* trow_p = p.table + (int64_t)w.trow * p.max_pages_per_seq + w.page_begin;
    auto issue = [&](int i, int32_t pg) {  // thread 0 only
        int st = i % NS;
        if (pg < 0 || pg >= p.n_pages) {
            atomicOr(p.status, STATUS_PAGE_OOB);
            pg = 0;
        }
        const uint8_t* src = p.pool + (int64_t)pg * p.page_bytes + (int64_t)kvh * Gm::STAGE;
        mbar_expect_tx(&bars[st], Gm::STAGE);
        bulk_g2s(stages + (size_t)st * Gm::STAGE, src, Gm::STAGE, &bars[st]);
    };
    grid_dependency_wait();    // the append that precedes this launch has written its pages
    grid_launch_dependents();  // the combine pass may be scheduled; it waits for this grid before reading partials
    int32_t pg_next = 0;  // thread 0: id of the next page to request
    if (tid == 0) {
        for (int s = 0; s < NS; s++) mbar_init(&bars[s], 1);
        mbar_fence_init();
        // start streaming right away; the other threads first meet the barriers after the __syncthreads below
        const bool stalled = (int)blockIdx.x == p.stall_item && blockIdx.y == 0 && blockIdx.z == 0;  // test hook, see DecodeParams
        int32_t first[NS];
#pragma unroll
        for (int i = 0; i < NS; i++) first[i] = i < n_tiles ? trow_p[i] : 0;  // the loads travel together
#pragma unroll
        for (int i = 0; i < NS; i++)
            if (i < n_tiles && !stalled) issue(i, first[i]);
        if (NS < n_tiles) pg_next = trow_p[NS];
    }
    // q of the group as f32 in shared memory, rows beyond the group zero
    for (int idx = tid; idx < 8 * MD; idx += 128) {
        int g = idx / MD, ch = idx % MD;
        float v = 0.f;
        if (g < ng) v = load_query(p, MD, w.batch, kvh * p.G + g0 + g, ch);
        if (QUANT) v = __half2float(__float2half_rn(v));  // the operand the tensor cores will see
        q_s[idx] = v;
    }
    __syncthreads();

    // ---- B fragments of Q^T for the 8 k-steps (head n = lane / 4) --------------------------------------
    uint32_t qb[8][2];
    {
        const float* qrow = q_s + r * MD;  // r doubles as the head index n of a B fragment
#pragma unroll
        for (int s = 0; s < 8; s++) {
            int k0, k1;
            float qf = 1.f;
            if (FMT == B200KV_FMT_Q8_1) {  // k-step (block b = s/2, half hh = s%2): channels 32b + 8c + 4hh + {0,1 | 2,3}
                k0 = 32 * (s >> 1) + 8 * c + 4 * (s & 1);
                k1 = k0 + 2;
            } else if (FMT == B200KV_FMT_Q4_0) {  // channels 32b + 16hh + 4c + {0,1 | 2,3}; hh = 1 meets 16 * code
                k0 = 32 * (s >> 1) + 16 * (s & 1) + 4 * c;
                k1 = k0 + 2;
                qf = (s & 1) ? 0.0625f : 1.f;
            } else {  // natural order: channels 16s + 2c + {0,1 | 8,9}
                k0 = 16 * s + 2 * c;
                k1 = k0 + 8;
            }
            if (IS_BF16) {
                qb[s][0] = pack_bf16(qrow[k0], qrow[k0 + 1]);
                qb[s][1] = pack_bf16(qrow[k1], qrow[k1 + 1]);
            } else {
                qb[s][0] = pack_f16(qrow[k0] * qf, qrow[k0 + 1] * qf);
                qb[s][1] = pack_f16(qrow[k1] * qf, qrow[k1 + 1] * qf);
            }
        }
    }
    // offset term of the K side: OFFS * sum of q over each 32-channel block, for heads 2c and 2c + 1
    float kbias[QUANT ? 4 : 1][2];
    if (QUANT) {
        {  // 16 threads per head, 8 channels each; 4 neighbouring threads make up one block
            const float* src = q_s + (tid >> 4) * MD + (tid & 15) * 8;
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) sum += src[i];
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((tid & 3) == 0) qsum_s[(tid >> 4) * 4 + ((tid & 15) >> 2)] = sum;
        }
        __syncthreads();
#pragma unroll
        for (int b = 0; b < 4; b++)
#pragma unroll
            for (int h = 0; h < 2; h++) kbias[b][h] = OFFS * qsum_s[(2 * c + h) * 4 + b];
    }

    const float sl2 = p.scale * LOG2E;  // scores are kept in log2 units
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_part[2] = {0.f, 0.f};  // this thread's share of the row sums (its two token rows only)
    float o[8][4];                 // O^T fragments: m-tile j = channels 16j..16j+15, columns = heads 2c, 2c+1
    // offset term of the V side, one per block: rows r of the constant operand only (rows r + 8 give the same value, for
    // Q4_0 16 times it: exact either way), so the other half of each product lands in two registers nobody reads
    float ob[QUANT ? 4 : 1][2];
    float ob_unused0 = 0.f, ob_unused1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[j][e] = 0.f;
#pragma unroll
    for (int b = 0; b < (QUANT ? 4 : 1); b++) ob[b][0] = ob[b][1] = 0.f;
    bool failed = false;

    const int tA = warp * 16 + r, tB = tA + 8;  // the two token rows of this thread's C fragments

    for (int i = 0; i < n_tiles; i++) {
        const int st = i % NS;
        // (warp-uniform: every lane waits on the same phase)  A warp whose wait ran out still walks on to the CTA barrier
        // below, where every warp learns of it and the whole CTA leaves the loop together
        const bool ok = mbar_wait_bounded(&bars[st], (uint32_t)((i / NS) & 1), p.wait_ns);
        const uint8_t* Ks = stages + (size_t)st * Gm::STAGE;
        const uint8_t* Vs = Ks + Gm::CHUNK;
        const int n_valid = min(PAGE_TOKENS, w.len - (w.page_begin + i) * PAGE_TOKENS);
        const int n_first = max(0, w.first - (w.page_begin + i) * PAGE_TOKENS);  // slots below it lie before the window
        if (ok && warp * 16 < n_valid) {  // warp-uniform: this warp has at least one live token in the tile
            const bool vA = tA < n_valid && tA >= n_first, vB = tB < n_valid && tB >= n_first;

            // ================= scores: S^T[16 tokens x 8 heads] = K . Q^T =================
            float sacc[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (QUANT) {
                const float2* ksc = (const float2*)(Ks + Gm::DATA);  // 4 f16 scales = 8 bytes per token
                const float2 rawA = ksc[tA], rawB = ksc[tB];
                const float2 sA01 = __half22float2(*(const __half2*)&rawA.x), sA23 = __half22float2(*(const __half2*)&rawA.y);
                const float2 sB01 = __half22float2(*(const __half2*)&rawB.x), sB23 = __half22float2(*(const __half2*)&rawB.y);
                const float sA[4] = {sA01.x, sA01.y, sA23.x, sA23.y}, sB[4] = {sB01.x, sB01.y, sB23.x, sB23.y};
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    uint32_t a0[4], a1[4];
                    if constexpr (FMT == B200KV_FMT_Q8_1) {
                        // 8 codes of block b for this thread: channels 32b + 8c .. + 8
                        const uint2 wa = *(const uint2*)(Ks + chunk_addr(FMT, MD, 0, tA, 32 * b + 8 * c));
                        const uint2 wb = *(const uint2*)(Ks + chunk_addr(FMT, MD, 0, tB, 32 * b + 8 * c));
                        a0[0] = __byte_perm(wa.x, 0, 0x4140), a0[1] = __byte_perm(wb.x, 0, 0x4140);
                        a0[2] = __byte_perm(wa.x, 0, 0x4342), a0[3] = __byte_perm(wb.x, 0, 0x4342);
                        a1[0] = __byte_perm(wa.y, 0, 0x4140), a1[1] = __byte_perm(wb.y, 0, 0x4140);
                        a1[2] = __byte_perm(wa.y, 0, 0x4342), a1[3] = __byte_perm(wb.y, 0, 0x4342);
                    } else {
                        // GGML block bytes 4c .. 4c+3: the low nibbles are channels 32b + 4c + {0..3} (first k-step), the
                        // high nibbles channels 32b + 16 + 4c + {0..3} (second k-step).  The high nibbles are used in
                        // place, i.e. as 16 * code; the matching q operands carry the factor 1/16 (exact in f16).
                        const uint32_t wa = *(const uint32_t*)(Ks + chunk_addr(FMT, MD, 0, tA, 16 * b + 4 * c));
                        const uint32_t wb = *(const uint32_t*)(Ks + chunk_addr(FMT, MD, 0, tB, 16 * b + 4 * c));
                        const uint32_t la = wa & 0x0f0f0f0fu, ha = wa & 0xf0f0f0f0u, lb = wb & 0x0f0f0f0fu, hb = wb & 0xf0f0f0f0u;
                        a0[0] = __byte_perm(la, 0, 0x4140), a0[1] = __byte_perm(lb, 0, 0x4140);
                        a0[2] = __byte_perm(la, 0, 0x4342), a0[3] = __byte_perm(lb, 0, 0x4342);
                        a1[0] = __byte_perm(ha, 0, 0x4140), a1[1] = __byte_perm(hb, 0, 0x4140);
                        a1[2] = __byte_perm(ha, 0, 0x4342), a1[3] = __byte_perm(hb, 0, 0x4342);
                    }
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_f16(acc, a0, qb[2 * b][0], qb[2 * b][1]);
                    mma_f16(acc, a1, qb[2 * b + 1][0], qb[2 * b + 1][1]);
                    // scale * (sum q * (u - OFFS)) with u * 2^-24 inside the product
                    sacc[0] = fmaf(sA[b], fmaf(acc[0], TWO24, -kbias[b][0]), sacc[0]);
                    sacc[1] = fmaf(sA[b], fmaf(acc[1], TWO24, -kbias[b][1]), sacc[1]);
                    sacc[2] = fmaf(sB[b], fmaf(acc[2], TWO24, -kbias[b][0]), sacc[2]);
                    sacc[3] = fmaf(sB[b], fmaf(acc[3], TWO24, -kbias[b][1]), sacc[3]);
                }
            } else {
                // lane -> address of one 8x8 matrix row: token (lane & 7) + 8 * bit3, channel half = bit 4
                const int lt = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int lk = (lane >> 4) * 8;
#pragma unroll
                for (int s = 0; s < 8; s++) {
                    uint32_t a[4];
                    ldmatrix_x4(a, Ks + chunk_addr(FMT, MD, 0, lt, (16 * s + lk) * 2));
                    if (IS_BF16) mma_bf16(sacc, a, qb[s][0], qb[s][1]);
                    else mma_f16(sacc, a, qb[s][0], qb[s][1]);
                }
            }

            // ================= online softmax (log2 domain), heads 2c and 2c + 1 =================
            const float s0 = vA ? sacc[0] * sl2 : -INFINITY, s1 = vA ? sacc[1] * sl2 : -INFINITY;
            const float s2 = vB ? sacc[2] * sl2 : -INFINITY, s3 = vB ? sacc[3] * sl2 : -INFINITY;
            // The reference maximum of a head is raised only when a score of this warp exceeds it by more than 2^LAZY_MAX (a
            // warp-wide vote): most pages then cost no cross-lane maximum, no rescaling of O and no exponentials of the
            // correction factor, and the weights stay below 2^LAZY_MAX = 2, safe for the 16-bit operands they become.
            const float lm0 = fmaxf(s0, s2), lm1 = fmaxf(s1, s3);
            if (__any_sync(0xffffffffu, lm0 > m_run[0] + LAZY_MAX || lm1 > m_run[1] + LAZY_MAX)) {
                const float mn0 = fmaxf(m_run[0], quad_row_max(lm0)), mn1 = fmaxf(m_run[1], quad_row_max(lm1));
                // a head whose keys were all masked so far keeps -inf: its sums and outputs are zero, factor 1
                const float al0 = mn0 == -INFINITY ? 1.f : fast_ex2(m_run[0] - mn0), al1 = mn1 == -INFINITY ? 1.f : fast_ex2(m_run[1] - mn1);
                m_run[0] = mn0, m_run[1] = mn1;
                l_part[0] *= al0, l_part[1] *= al1;
#pragma unroll
                for (int j = 0; j < 8; j++) o[j][0] *= al0, o[j][1] *= al1, o[j][2] *= al0, o[j][3] *= al1;
                if (QUANT) {
#pragma unroll
                    for (int b = 0; b < (QUANT ? 4 : 1); b++) ob[b][0] *= al0, ob[b][1] *= al1;
                    ob_unused0 = ob_unused1 = 0.f;  // kept finite
                }
            }
            const float mu0 = m_run[0] == -INFINITY ? 0.f : m_run[0], mu1 = m_run[1] == -INFINITY ? 0.f : m_run[1];  // exp2(-inf - 0) = 0
            const float p0 = fast_ex2(s0 - mu0), p1 = fast_ex2(s1 - mu1), p2 = fast_ex2(s2 - mu0), p3 = fast_ex2(s3 - mu1);
            l_part[0] += p0 + p2;
            l_part[1] += p1 + p3;

            // ================= O^T[128 ch x 8 heads] += V^T . P^T =================
            if constexpr (QUANT) {
                // P^T B fragments: transpose the probabilities once, then fold the V scale of each block in with
                // one packed multiply.  The scale region of a V chunk holds, per token pair and block, the f16 pair
                // (scale of the even token, scale of the odd token): exactly the k-slot pairs of a B fragment.
                const uint32_t pt0 = movmatrix_trans(pack_f16(p0 * PSCALE, p1 * PSCALE));  // tokens 2c, 2c+1 of head n
                const uint32_t pt1 = movmatrix_trans(pack_f16(p2 * PSCALE, p3 * PSCALE));  // tokens 2c+8, 2c+9
                const int T0 = warp * 16 + 2 * c;
                uint4 sc01 = *(const uint4*)(Vs + Gm::DATA + (T0 >> 1) * 16);        // 4 blocks x (T0, T0+1)
                uint4 sc23 = *(const uint4*)(Vs + Gm::DATA + ((T0 >> 1) + 4) * 16);  // 4 blocks x (T0+8, T0+9)
                if (warp * 16 + 16 > n_valid) {
                    // a stale scale in a dead token slot must not turn 0 * inf into NaN: zero it
                    const uint32_t k01 = (T0 < n_valid ? 0x0000ffffu : 0u) | (T0 + 1 < n_valid ? 0xffff0000u : 0u);
                    const uint32_t k23 = (T0 + 8 < n_valid ? 0x0000ffffu : 0u) | (T0 + 9 < n_valid ? 0xffff0000u : 0u);
                    sc01.x &= k01, sc01.y &= k01, sc01.z &= k01, sc01.w &= k01;
                    sc23.x &= k23, sc23.y &= k23, sc23.z &= k23, sc23.w &= k23;
                }
                uint32_t pb[4][2];
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const __half2 h0 = __hmul2(*(const __half2*)&pt0, *(const __half2*)&(&sc01.x)[b]);
                    const __half2 h1 = __hmul2(*(const __half2*)&pt1, *(const __half2*)&(&sc23.x)[b]);
                    pb[b][0] = *(const uint32_t*)&h0, pb[b][1] = *(const uint32_t*)&h1;
                }
                // this thread's four V token rows: k-slots 2c, 2c+1, 2c+8, 2c+9 of the warp's 16 tokens
                if constexpr (FMT == B200KV_FMT_Q8_1) {
                    uint4 x[4];  // 16 bytes at positions 16r.. of each row: channel slot (r | r + 8) of every m-tile
                    x[0] = *(const uint4*)(Vs + chunk_addr(FMT, MD, 1, T0, 16 * r));
                    x[1] = *(const uint4*)(Vs + chunk_addr(FMT, MD, 1, T0 + 1, 16 * r));
                    x[2] = *(const uint4*)(Vs + chunk_addr(FMT, MD, 1, T0 + 8, 16 * r));
                    x[3] = *(const uint4*)(Vs + chunk_addr(FMT, MD, 1, T0 + 9, 16 * r));
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint32_t w0 = (&x[0].x)[j >> 1], w1 = (&x[1].x)[j >> 1], w2 = (&x[2].x)[j >> 1], w3 = (&x[3].x)[j >> 1];
                        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
                        const uint32_t v01 = __byte_perm(w0, w1, sel);  // [T0.b2j, T0.b2j+1, T1.b2j, T1.b2j+1]
                        const uint32_t v23 = __byte_perm(w2, w3, sel);
                        uint32_t a[4];
                        a[0] = __byte_perm(v01, 0, 0x4240), a[1] = __byte_perm(v01, 0, 0x4341);
                        a[2] = __byte_perm(v23, 0, 0x4240), a[3] = __byte_perm(v23, 0, 0x4341);
                        mma_f16(o[j], a, pb[j >> 1][0], pb[j >> 1][1]);
                    }
                } else {
                    uint2 x[4];  // 8 bytes at positions 8r..: byte j = slot r (low nibble) | slot r + 8 (high) of m-tile j
                    x[0] = *(const uint2*)(Vs + chunk_addr(FMT, MD, 1, T0, 8 * r));
                    x[1] = *(const uint2*)(Vs + chunk_addr(FMT, MD, 1, T0 + 1, 8 * r));
                    x[2] = *(const uint2*)(Vs + chunk_addr(FMT, MD, 1, T0 + 8, 8 * r));
                    x[3] = *(const uint2*)(Vs + chunk_addr(FMT, MD, 1, T0 + 9, 8 * r));
#pragma unroll
                    for (int jj = 0; jj < 4; jj++) {  // m-tiles 2jj and 2jj + 1 (both in block jj)
                        const uint32_t w0 = (&x[0].x)[jj >> 1], w1 = (&x[1].x)[jj >> 1], w2 = (&x[2].x)[jj >> 1], w3 = (&x[3].x)[jj >> 1];
                        const uint32_t sel = (jj & 1) ? 0x7632u : 0x5410u;
                        const uint32_t v01 = __byte_perm(w0, w1, sel), v23 = __byte_perm(w2, w3, sel);
                        // high nibbles in place (16 * code): rows r + 8 of O^T come out 16 times too large, undone at the end
                        const uint32_t lo01 = v01 & 0x0f0f0f0fu, hi01 = v01 & 0xf0f0f0f0u;
                        const uint32_t lo23 = v23 & 0x0f0f0f0fu, hi23 = v23 & 0xf0f0f0f0u;
                        uint32_t a[4];
                        a[0] = __byte_perm(lo01, 0, 0x4240), a[1] = __byte_perm(hi01, 0, 0x4240);
                        a[2] = __byte_perm(lo23, 0, 0x4240), a[3] = __byte_perm(hi23, 0, 0x4240);
                        mma_f16(o[2 * jj], a, pb[jj][0], pb[jj][1]);
                        a[0] = __byte_perm(lo01, 0, 0x4341), a[1] = __byte_perm(hi01, 0, 0x4341);
                        a[2] = __byte_perm(lo23, 0, 0x4341), a[3] = __byte_perm(hi23, 0, 0x4341);
                        mma_f16(o[2 * jj + 1], a, pb[jj][0], pb[jj][1]);
                    }
                }
                // offset term: the same (rounded) probabilities against a constant operand
                constexpr uint32_t OFFS_HI = FMT == B200KV_FMT_Q4_0 ? 0x00800080u : OFFS_FRAG;  // rows r + 8 of Q4_0: 16 * 8
                const uint32_t ofs[4] = {OFFS_FRAG, OFFS_HI, OFFS_FRAG, OFFS_HI};
#pragma unroll
                for (int b = 0; b < 4; b++) mma_f16(ob[b][0], ob[b][1], ob_unused0, ob_unused1, ofs, pb[b][0], pb[b][1]);
            } else {
                // lane -> address of one 8x8 matrix row of V: token (lane & 7) + 8 * bit4, channel half = bit 3
                const int lt = warp * 16 + (lane & 7) + ((lane >> 4) & 1) * 8;
                const int lc = ((lane >> 3) & 1) * 8;
                uint32_t pb0, pb1, pl0 = 0, pl1 = 0;
                if (IS_BF16) {
                    // bf16 keeps 8 bits of a probability: carry the remainder in a second operand
                    const uint32_t h0 = pack_bf16(p0, p1), h1 = pack_bf16(p2, p3);
                    const __nv_bfloat162 f0 = *(const __nv_bfloat162*)&h0, f1 = *(const __nv_bfloat162*)&h1;
                    pb0 = movmatrix_trans(h0), pb1 = movmatrix_trans(h1);
                    pl0 = movmatrix_trans(pack_bf16(p0 - __low2float(f0), p1 - __high2float(f0)));
                    pl1 = movmatrix_trans(pack_bf16(p2 - __low2float(f1), p3 - __high2float(f1)));
                } else {
                    pb0 = movmatrix_trans(pack_f16(p0, p1)), pb1 = movmatrix_trans(pack_f16(p2, p3));
                }
                // dead token slots of a partly filled page may hold anything: zero their V columns
                uint32_t keep01 = 0xffffffffu, keep23 = 0xffffffffu;
                if (warp * 16 + 16 > n_valid) {
                    const int k0 = warp * 16 + 2 * c;
                    keep01 = (k0 < n_valid ? 0x0000ffffu : 0u) | (k0 + 1 < n_valid ? 0xffff0000u : 0u);
                    keep23 = (k0 + 8 < n_valid ? 0x0000ffffu : 0u) | (k0 + 9 < n_valid ? 0xffff0000u : 0u);
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    uint32_t a[4];
                    ldmatrix_x4_trans(a, Vs + chunk_addr(FMT, MD, 1, lt, (16 * j + lc) * 2));
                    a[0] &= keep01, a[1] &= keep01, a[2] &= keep23, a[3] &= keep23;
                    if (IS_BF16) {
                        mma_bf16(o[j], a, pb0, pb1);
                        mma_bf16(o[j], a, pl0, pl1);
                    } else {
                        mma_f16(o[j], a, pb0, pb1);
                    }
                }
            }
        }
        if (__syncthreads_or(!ok)) {  // every warp is done with stage st; a wait that ran out anywhere ends the loop for all
            failed = true;
            break;
        }
        if (tid == 0 && i + NS < n_tiles) {
            issue(i + NS, pg_next);
            if (i + NS + 1 < n_tiles) pg_next = trow_p[i + NS + 1];
        }
    }

    // ---- merge the four warps and publish the partial of this split ----
    const int64_t pbase = ((int64_t)blockIdx.x * p.Hkv + kvh) * p.G + g0;
    if (failed) {
        if (tid == 0) atomicOr(p.status, STATUS_WAIT_EXPIRED);
        for (int idx = tid; idx < ng * MD; idx += 128) p.part_o[(pbase + idx / MD) * MD + idx % MD] = 0.f;
        if (tid < ng) p.part_ml[(pbase + tid) * 2] = -INFINITY, p.part_ml[(pbase + tid) * 2 + 1] = 0.f;
        return;
    }
    float* om = (float*)stages;                 // [4 warps][8 heads][128 ch]; every stage is consumed by now
    float* ml = om + 4 * 8 * MD;                // [4 warps][8 heads][2]
    const float l0 = quad_row_sum(l_part[0]), l1 = quad_row_sum(l_part[1]);
    if (r == 0) {
        ml[(warp * 8 + 2 * c) * 2] = m_run[0], ml[(warp * 8 + 2 * c) * 2 + 1] = l0;
        ml[(warp * 8 + 2 * c + 1) * 2] = m_run[1], ml[(warp * 8 + 2 * c + 1) * 2 + 1] = l1;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float v0 = o[j][0], v1 = o[j][1], v2 = o[j][2], v3 = o[j][3];
        if (QUANT) {  // remove the offset term and the 2^-24 * 1024 operand scaling
            constexpr float UNDO = TWO24 / PSCALE;
            const int b = j >> 1;
            constexpr float UNDO_HI = FMT == B200KV_FMT_Q4_0 ? UNDO / 16.f : UNDO;
            constexpr float HI = FMT == B200KV_FMT_Q4_0 ? 16.f : 1.f;  // rows r + 8 of Q4_0 carry 16 * code and 16 * offset
            v0 = (v0 - ob[b][0]) * UNDO, v1 = (v1 - ob[b][1]) * UNDO, v2 = (v2 - HI * ob[b][0]) * UNDO_HI, v3 = (v3 - HI * ob[b][1]) * UNDO_HI;
        }
        float* base = om + (warp * 8 + 2 * c) * MD + 16 * j + r;
        base[0] = v0, base[MD] = v1, base[8] = v2, base[MD + 8] = v3;
    }
    __syncthreads();
    for (int idx = tid; idx < ng * MD; idx += 128) {
        const int g = idx / MD, ch = idx % MD;
        float M = -INFINITY;
#pragma unroll
        for (int wv = 0; wv < 4; wv++) M = fmaxf(M, ml[(wv * 8 + g) * 2]);
        float num = 0.f;
#pragma unroll
        for (int wv = 0; wv < 4; wv++) {
            const float mw = ml[(wv * 8 + g) * 2];
            if (mw > -INFINITY) num = fmaf(exp2f(mw - M), om[(wv * 8 + g) * MD + ch], num);
        }
        p.part_o[(pbase + g) * MD + ch] = num;
    }
    if (tid < ng) {
        float M = -INFINITY, den = 0.f;
        for (int wv = 0; wv < 4; wv++) M = fmaxf(M, ml[(wv * 8 + tid) * 2]);
        for (int wv = 0; wv < 4; wv++) {
            const float mw = ml[(wv * 8 + tid) * 2];
            if (mw > -INFINITY) den = fmaf(exp2f(mw - M), ml[(wv * 8 + tid) * 2 + 1], den);
        }
        p.part_ml[(pbase + tid) * 2] = M * 0.6931471805599453f;  // back to natural-log units for the combine pass
        p.part_ml[(pbase + tid) * 2 + 1] = den;
    }
}

template <int FMT>
static int launch_mma_t(const DecodeParams& p, int n_items, cudaStream_t stream, const InlineBatch& ib) {
    using Gm = MGeo<FMT>;
    const size_t ring = (size_t)Gm::NS * Gm::STAGE;
    const size_t merge = (size_t)(4 * 8 * MD + 4 * 8 * 2) * 4;  // the warp merge reuses the ring
    const size_t smem = std::max(ring, merge) + MMA_TAIL;
    B200KV_CUDA(cudaFuncSetAttribute(decode_mma_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(n_items, p.Hkv, (p.G + 7) / 8);
    B200KV_CUDA(launch_after_predecessor(decode_mma_kernel<FMT>, grid, dim3(128), smem, stream, p, ib));
    return B200KV_OK;
}

bool decode_mma_supported(int fmt, int D, int dtype) {
    if (D != MD) return false;
    if (fmt == B200KV_FMT_F16) return dtype == B200KV_F16;
    if (fmt == B200KV_FMT_BF16) return dtype == B200KV_BF16;
    if (fmt == B200KV_FMT_Q8_1 || fmt == B200KV_FMT_Q4_0) return dtype == B200KV_F16 || dtype == B200KV_BF16;
    return false;
}

int launch_decode_mma(int fmt, const DecodeParams& p, int n_items, cudaStream_t stream, const InlineBatch* ibp) {
    const InlineBatch& ib = ibp ? *ibp : empty_inline_batch();
    switch (fmt) {
        case B200KV_FMT_F16: return launch_mma_t<B200KV_FMT_F16>(p, n_items, stream, ib);
        case B200KV_FMT_BF16: return launch_mma_t<B200KV_FMT_BF16>(p, n_items, stream, ib);
        case B200KV_FMT_Q8_1: return launch_mma_t<B200KV_FMT_Q8_1>(p, n_items, stream, ib);
        case B200KV_FMT_Q4_0: return launch_mma_t<B200KV_FMT_Q4_0>(p, n_items, stream, ib);
    }
    return fail("format %d has no tensor-core decode kernel", fmt);
}

}  // namespace b200kv
