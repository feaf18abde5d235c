// Flash-attention prefill over the paged cache on the 5th-generation tensor cores (tcgen05 + TMEM):
// the S > 1 case of b200kv_attend for f16 / bf16 caches at head_dim 128.
//
// Replaces the prefill use of cuda/src/kernels/cu/flash_attn.cu (`attention_fullq_*`: Ampere mma.sync,
// one q-head per CTA so every head of a GQA group re-streams K/V).  Semantics:
// transformers/src/ops/flash_sdpa.rs:239-341 (causal aligned bottom-right, scale, f32 accumulation).
//
// A query tile is 128 rows = (query, head-of-group) pairs of one (sequence, kv head), so the whole GQA group
// shares each K/V page.  A CTA owns NQ such tiles of consecutive queries (NQ = 2: one CTA per SM, both tiles
// read each K/V chunk from the same shared-memory stage; NQ = 1: two CTAs per SM, for launches too small to
// fill the GPU with double tiles).  Per tile and per page of 64 cached tokens:
//   S[128 x 64]  = Q . K^T      tcgen05.mma, A = Q tile in shared memory (K-major, 128-byte swizzle),
//                               B = the K chunk exactly as it lies in the page (same swizzle), D in TMEM;
//                               S is double-buffered, so the product for page j+1 runs under the softmax of page j
//   softmax                     one thread owns a row: it tcgen05.ld's the 64 scores, masks, exponentiates in the log2
//                               domain against a lazily raised reference maximum -- the exponentials issued as a software
//                               pipeline, so that the MUFU unit (one warp instruction per 8 cycles) always has the warp's
//                               next ones queued -- and writes P (16-bit) over the S buffer it came from with tcgen05.st
//   O[128 x 128] += P . V       tcgen05.mma, A = P from TMEM, B = the V chunk as it lies in the page (MN-major
//                               operand: channels contiguous), D accumulates in TMEM.  f16: one MMA per 16 tokens
//                               (P carries 11 bits); bf16: P goes in as its 16-bit value plus the 16-bit rounding
//                               remainder (two MMAs), or a row that sees few keys would carry the 2^-9 rounding
// Roles: 128 softmax threads per tile; one warp that issues the K / V bulk copies (untiled cp.async.bulk into
// two rings); one warp per tile that issues its MMAs and their commits.  Every wait is bounded; on expiry the
// CTA flags the status word, lets every role run to the end of its loop without waiting any more, frees its
// TMEM and returns.
#include <cmath>
#include "tc_common.cuh"

namespace b200kv {

constexpr int PD = 128;                        // head_dim
constexpr int PM = 128;                        // rows of a query tile
constexpr int P_CHUNK = PAGE_TOKENS * PD * 2;  // bytes of one K (or V) chunk: 16 KiB
constexpr int P_QBYTES = PM * PD * 2;          // 32 KiB per query tile
constexpr int SM_THREADS = 128;                // softmax threads per query tile: one per row

// TMEM columns of one query tile: O 0..127, S buffers at 128 and 192; P(j) overwrites S(j): value in columns
// 0..31 of the buffer, rounding remainder in 32..63
constexpr uint32_t COL_O = 0, COL_S = 128, COLS_PER_TILE = 256;
// (f16 P carries 11 bits: enough once a row's sum is spread over many keys, but a row whose few visible keys cancel
// keeps the full 2^-12 of each weight, which measured 2.4e-3 of the output's scale on a 512-token causal chunk;
// the remainder MMA removes it and is dropped page by page, see P_SKIP_FRACTION)

// per query tile and per parity of the page index: one flag per softmax warp (does the page need its remainder product)
constexpr int XCHG_FLOATS = 8;
// f16 weights skip the remainder MMA of a page once, for every row of the tile, sqrt(64) x the largest weight of the
// page is below this fraction of the row's running sum: what the rounding of such a page can add is then below
// 2^-12 / 8 of the row's scale
constexpr float P_SKIP_FRACTION = 0.125f;

template <int NQ>
struct PGeo {
    static constexpr int NK = NQ == 2 ? 4 : 2;  // K stages
    static constexpr int NV = NQ == 2 ? 5 : 2;  // V stages
    static constexpr int THREADS = NQ * SM_THREADS + 32 * (1 + NQ);  // softmax threads, the copy warp, one MMA warp per tile
    static constexpr int N_BARS = 2 * NK + 2 * NV + 6 * NQ;
    static constexpr size_t SMEM = (size_t)NQ * P_QBYTES + (size_t)(NK + NV) * P_CHUNK + N_BARS * 8 + 32 + NQ * 2 * XCHG_FLOATS * 4;
};

struct PrefillParams {
    const uint8_t* pool;
    const int32_t* table;
    const int32_t* desc;  // per batch entry: {table row, cached length}
    int* status;
    const void* q;
    void* out;
    int64_t qb, qh, qs, ob, oh, os;
    int64_t page_bytes;
    int32_t n_pages, max_pages_per_seq, Hkv, G, S, causal, is_bf16;
    uint32_t v_lbo, v_sbo;  // V operand descriptor strides (bytes)
    float scale;
    float skip_fraction;
};

// Softmax threads of tile qt: warp w of the tile addresses TMEM lanes 32 w .. + 32 (a warp may touch only the lane
// quarter of its index modulo 4, and every tile has four softmax warps); lane l owns row 32 w + l.
template <int NQ>
__global__ void __launch_bounds__(PGeo<NQ>::THREADS, NQ == 2 ? 1 : 2) prefill_tc_kernel(PrefillParams p) {
    using GEO = PGeo<NQ>;
    constexpr int NK = GEO::NK, NV = GEO::NV;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* q_s = smem;                                   // [NQ][2 planes][128 rows][128 B], swizzled
    uint8_t* k_ring = smem + NQ * P_QBYTES;                // NK K chunks
    uint8_t* v_ring = k_ring + NK * P_CHUNK;               // NV V chunks
    uint64_t* full_k = (uint64_t*)(v_ring + NV * P_CHUNK);  // [NK] bytes landed
    uint64_t* full_v = full_k + NK;                        // [NV]
    uint64_t* free_k = full_v + NV;                        // [NK] every tile's Q.K^T on the stage has completed
    uint64_t* free_v = free_k + NK;                        // [NV] every tile's P.V on the stage has completed
    uint64_t* bar_s = free_v + NV;                         // [NQ][2] S buffer written
    uint64_t* bar_p = bar_s + 2 * NQ;                      // [NQ][2] P written by the softmax warps
    uint64_t* bar_o = bar_p + 2 * NQ;                      // [NQ][2] P.V of page j completed, on barrier j & 1
    uint32_t* tmem_slot = (uint32_t*)(((uintptr_t)(bar_o + 2 * NQ) + 15) & ~(uintptr_t)15);
    volatile int* fail_s = (volatile int*)(tmem_slot + 1);
    float* xchg = (float*)(tmem_slot + 4);                 // [NQ][2 parities][XCHG_FLOATS]: remainder flags of the softmax warps

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y, b = blockIdx.z;
    const int G = p.G, qpt = PM / G;                       // queries per tile
    const int cta_tile = (int)(gridDim.x - 1 - blockIdx.x);  // late queries see the most keys: schedule them first
    const int32_t trow = p.desc[2 * b], T = p.desc[2 * b + 1];
    const int P0 = T - p.S;                                // cached tokens before the first new query
    const int cta_q0 = cta_tile * NQ * qpt;
    const int cta_q_last = min(cta_q0 + NQ * qpt, p.S) - 1;
    // every tile of the CTA walks the pages up to the last key its last tile sees; a tile that ends earlier finds
    // its extra page fully masked
    const int n_tiles = (p.causal ? P0 + cta_q_last : T - 1) / PAGE_TOKENS + 1;

    if (tid == 0) {
        for (int s = 0; s < NK; s++) mbar_init(&full_k[s], 1), mbar_init(&free_k[s], NQ);
        for (int s = 0; s < NV; s++) mbar_init(&full_v[s], 1), mbar_init(&free_v[s], NQ);
        for (int i = 0; i < 2 * NQ; i++) mbar_init(&bar_s[i], 1), mbar_init(&bar_p[i], SM_THREADS / 32);
        for (int i = 0; i < 2 * NQ; i++) mbar_init(&bar_o[i], 1);
        *fail_s = (smem_u32(smem) & 1023u) ? 1 : 0;  // the swizzled operand tiles need a 1024-byte aligned base
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, COLS_PER_TILE * NQ);

    // per-thread tile geometry (softmax threads only; the extra warp gets harmless values)
    const int qt = min(tid / SM_THREADS, NQ - 1), w4 = (tid % SM_THREADS) >> 5;
    const int row = w4 * 32 + lane;
    const int q0 = cta_q0 + qt * qpt;
    const int rq = row / G, rg = row % G;
    const bool live = rq < qpt && q0 + rq < p.S;
    const int q_last = max(min(q0 + qpt, p.S) - 1, 0);   // last live query of the tile (the tile may be all dead)
    const int my_q = live ? q0 + rq : min(q_last, p.S - 1);
    const int my_limit = p.causal ? P0 + my_q : T - 1;  // last visible key of this row
    const int min_limit = p.causal ? P0 + min(q0, p.S - 1) : T - 1;  // last key EVERY row of the tile sees
    const bool is_softmax = tid < NQ * SM_THREADS;

    // ---- Q tile -> shared memory, K-major with the 128-byte swizzle (row r: 16-byte unit u of plane pl at u ^ (r & 7));
    //      this thread moves its row ----
    if (is_softmax) {
        const int head = kvh * G + rg;
        const uint4* src = (const uint4*)((const uint16_t*)p.q + (int64_t)b * p.qb + (int64_t)head * p.qh + (int64_t)my_q * p.qs);
#pragma unroll
        for (int uu = 0; uu < 16; uu++) {
            uint4 v = live ? src[uu] : make_uint4(0, 0, 0, 0);
            *(uint4*)(q_s + qt * P_QBYTES + (uu >> 3) * (PM * 128) + row * 128 + (((uu & 7) ^ (row & 7)) << 4)) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (!is_softmax) {
        // Every lane of these warps walks the loop (the values stay warp-uniform); one elected lane issues.
        const int role = warp - NQ * (SM_THREADS / 32);  // 0: copies, 1 + t: MMAs of tile t
        if (role == 0) {
            // ================= K / V copies into the two rings =================
            const int32_t* trow_p = p.table + (int64_t)trow * p.max_pages_per_seq;
            int32_t pg_next = trow_p[0];
            for (int i = 0; i < n_tiles; i++) {
                int32_t pg = pg_next;
                if (i + 1 < n_tiles) pg_next = trow_p[i + 1];  // fetched one page ahead of its use
                if (pg < 0 || pg >= p.n_pages) {
                    if (lane == 0) atomicOr(p.status, STATUS_PAGE_OOB);
                    pg = 0;
                }
                const uint8_t* src = p.pool + (int64_t)pg * p.page_bytes + (int64_t)kvh * (2 * P_CHUNK);
                if (i >= NK) wait_or_fail(&free_k[i % NK], (uint32_t)((i / NK - 1) & 1), fail_s);
                if (elect_one()) {
                    mbar_expect_tx(&full_k[i % NK], P_CHUNK);
                    bulk_g2s(k_ring + (i % NK) * P_CHUNK, src, P_CHUNK, &full_k[i % NK]);
                }
                __syncwarp();
                if (i >= NV) wait_or_fail(&free_v[i % NV], (uint32_t)((i / NV - 1) & 1), fail_s);
                if (elect_one()) {
                    mbar_expect_tx(&full_v[i % NV], P_CHUNK);
                    bulk_g2s(v_ring + (i % NV) * P_CHUNK, src + P_CHUNK, P_CHUNK, &full_v[i % NV]);
                }
                __syncwarp();
            }
        } else {
            // ================= MMAs of tile t = role - 1 =================
            const int t = role - 1;
            const uint32_t tm = tmem + t * COLS_PER_TILE;
            const uint32_t idesc_s = instr_desc(p.is_bf16, 0, PM, PAGE_TOKENS);
            const uint32_t idesc_o = instr_desc(p.is_bf16, 1, PM, PD);
            // descriptors of the ring bases; a byte offset inside the 256 KiB window adds offset / 16 to the address field
            const uint64_t q_desc = smem_desc(smem_u32(q_s) + t * P_QBYTES, 0, 1024);
            const uint64_t k_desc = smem_desc(smem_u32(k_ring), 0, 1024);
            const uint64_t v_desc = smem_desc(smem_u32(v_ring), p.v_lbo, p.v_sbo);
            const bool adaptive = !p.is_bf16;
            // S(j) = Q . K(j)^T into buffer j & 1
            auto issue_qk = [&](int j) {
                wait_or_fail(&full_k[j % NK], (uint32_t)((j / NK) & 1), fail_s);
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t kd = k_desc + (uint64_t)(((j % NK) * P_CHUNK) >> 4);
#pragma unroll
                    for (int pl = 0; pl < 2; pl++)
#pragma unroll
                        for (int kk = 0; kk < 4; kk++) {
                            const uint64_t off = (uint64_t)((pl * (PM * 128) + kk * 32) >> 4);
                            tc_mma_ss(tm + COL_S + 64 * (j & 1), q_desc + off, kd + (uint64_t)((pl * (PAGE_TOKENS * 128) + kk * 32) >> 4),
                                      idesc_s, (pl | kk) ? 1u : 0u);
                        }
                    tc_commit(&bar_s[2 * t + (j & 1)]);
                    tc_commit(&free_k[j % NK]);
                }
                __syncwarp();
            };
            issue_qk(0);
            if (n_tiles > 1) issue_qk(1);
            for (int j = 0; j < n_tiles; j++) {
                // O += P(j) . V(j): 4 steps of 16 tokens; the V chunk is an MN-major operand
                wait_or_fail(&full_v[j % NV], (uint32_t)((j / NV) & 1), fail_s);
                wait_or_fail(&bar_p[2 * t + (j & 1)], (uint32_t)((j >> 1) & 1), fail_s);
                tc_fence_after();
                // the softmax warps say, one flag each, whether this page's weights need their remainder
                const int* flags = (const int*)(xchg + (2 * t + (j & 1)) * XCHG_FLOATS);
                const bool two = !adaptive || __any_sync(0xffffffffu, flags[lane & 3] != 0);
                if (elect_one()) {
                    const uint64_t vd = v_desc + (uint64_t)(((j % NV) * P_CHUNK) >> 4);
                    const uint32_t pa = tm + COL_S + 64 * (j & 1);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        tc_mma_ts(tm + COL_O, pa + kk * 8, vd + (uint64_t)((kk * 2048) >> 4), idesc_o, (j | kk) ? 1u : 0u);
                        if (two) tc_mma_ts(tm + COL_O, pa + 32 + kk * 8, vd + (uint64_t)((kk * 2048) >> 4), idesc_o, 1u);
                    }
                    tc_commit(&bar_o[2 * t + (j & 1)]);
                    tc_commit(&free_v[j % NV]);
                }
                __syncwarp();
                // S(j + 2) reuses the buffer P(j) sits in: the tensor core runs one thread's MMAs in issue order, so the
                // product just issued has read P before this one writes S
                if (j + 2 < n_tiles) issue_qk(j + 2);
            }
        }
    } else {

        // ================= softmax threads =================
        const uint32_t lane_base = tmem + qt * COLS_PER_TILE + ((uint32_t)(w4 * 32) << 16);  // this warp's lane quarter
        const bool adaptive = !p.is_bf16;
        const float sl2 = p.scale * 1.4426950408889634f;  // scores enter the exponent in log2 units
        float m_ref = -INFINITY, l_run = 0.f, log_thresh = -INFINITY;

        for (int j = 0; j < n_tiles; j++) {
            const uint32_t sbuf = lane_base + COL_S + 64 * (j & 1);
            wait_or_fail(&bar_s[2 * qt + (j & 1)], (uint32_t)((j >> 1) & 1), fail_s);
            tc_fence_after();
            // ---- the row's 64 scores ----
            uint32_t sr[64];
            tmem_ld32(sbuf, sr);
            tmem_ld32(sbuf + 32, sr + 32);
            tmem_ld_wait();
            if (j * PAGE_TOKENS + PAGE_TOKENS - 1 > min_limit) {  // only pages on the causal diagonal / past the end need a mask
                const int t0 = j * PAGE_TOKENS;
#pragma unroll
                for (int c = 0; c < 64; c++)
                    if (t0 + c > my_limit) sr[c] = 0xff800000u;  // -inf
            }
            float tmax = row_max64(sr);
            int* flags = (int*)(xchg + (2 * qt + (j & 1)) * XCHG_FLOATS);
            tmax *= sl2;
            // Two questions per row, answered for the warp with one reduction.  Bit 0: does this page need the remainder
            // product (see P_SKIP_FRACTION; compared in the log domain against log2(fraction x running sum), kept from the
            // page before; page 0 always keeps it).  Bit 1: is the reference maximum exceeded by more than 2^8 -- it is
            // raised only then, so the exponentials stay below 256, exact enough in 16 bits, and O is rescaled rarely.
            const bool mine = adaptive && (j == 0 || tmax - m_ref + 3.f > log_thresh);
            const bool raise = j > 0 && tmax > m_ref + 8.f;
            const uint32_t votes = __reduce_or_sync(0xffffffffu, (mine ? 1u : 0u) | (raise ? 2u : 0u));
            const bool two = !adaptive || (votes & 1u);
            if (adaptive && lane == 0) flags[w4] = two ? 1 : 0;  // the MMA warp issues the remainder product if any warp asks for it
            if (j == 0) m_ref = tmax;
            if (votes & 2u) {
                float alpha = 1.f;
                if (raise) {
                    alpha = fast_exp2(m_ref - tmax);
                    m_ref = tmax;
                    l_run *= alpha;
                }
                // O must hold every page before this one.  S(j) being there says that P.V(j - 2) has completed (Q.K(j) was
                // issued behind it); P.V(j - 1) may or may not have.  A parity wait tells only two consecutive phases of a
                // barrier apart, so the products alternate between two barriers: on barrier (j - 1) & 1 the phase before the one
                // waited for belongs to P.V(j - 3), known complete, and the one after it to P.V(j + 1), which needs this
                // thread's P(j) first -- the wait cannot mistake one for the other.
                wait_or_fail(&bar_o[2 * qt + ((j - 1) & 1)], (uint32_t)(((j - 1) >> 1) & 1), fail_s);
                tc_fence_after();
#pragma unroll
                for (int cc = 0; cc < 8; cc++) {  // the row's 128 output channels
                    uint32_t orow[16];
                    tmem_ld16(lane_base + COL_O + cc * 16, orow);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 16; c++) orow[c] = __float_as_uint(__uint_as_float(orow[c]) * alpha);
                    tmem_st16(lane_base + COL_O + cc * 16, orow);
                }
            }
            // ---- P = 2^(s * scale * log2 e - m_ref), its 16-bit value and (when the page needs it) what that rounding lost ----
            uint32_t pr[32], pr2[32];
            float page_sum;
            if (p.is_bf16) page_sum = softmax_exps<2>(sr, sl2, m_ref, pr, pr2);
            else if (two) page_sum = softmax_exps<1>(sr, sl2, m_ref, pr, pr2);
            else page_sum = softmax_exps<0>(sr, sl2, m_ref, pr, pr2);
            tmem_st32(sbuf + 32, pr2);
            tmem_st32(sbuf, pr);
            l_run += page_sum;
            log_thresh = fast_log2(p.skip_fraction * l_run);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_p[2 * qt + (j & 1)]);
        }
        // ---- epilogue: wait for the last P.V, normalise, store ----
        wait_or_fail(&bar_o[2 * qt + ((n_tiles - 1) & 1)], (uint32_t)(((n_tiles - 1) >> 1) & 1), fail_s);  // see the rescale above
        tc_fence_after();
        if (!*fail_s) {
            const float inv = 1.f / l_run;
            uint16_t* dst = (uint16_t*)p.out + (int64_t)b * p.ob + (int64_t)(kvh * G + rg) * p.oh + (int64_t)my_q * p.os;
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                uint32_t orow[32];
                tmem_ld32(lane_base + COL_O + cc * 32, orow);
                tmem_ld_wait();
                if (live) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float a = __uint_as_float(orow[c + 2 * e]) * inv, bb = __uint_as_float(orow[c + 2 * e + 1]) * inv;
                            if (p.is_bf16) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(a, bb);
                                w[e] = *(uint32_t*)&h;
                            } else {
                                __half2 h = __floats2half2_rn(a, bb);
                                w[e] = *(uint32_t*)&h;
                            }
                        }
                        *(uint4*)(dst + cc * 32 + c) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*fail_s) {
        if (tid == 0) atomicOr(p.status, STATUS_WAIT_EXPIRED);
        __nanosleep(200000);  // give copies that may still be in flight time to land before the CTA's memory is released
        __syncthreads();
    }
    if (warp == 0) tmem_dealloc(tmem, COLS_PER_TILE * NQ);
}

bool prefill_tc_supported(const b200kv_cache* c, int n_q_heads, int dtype, const void* q, const int64_t* qs, const void* out,
                          const int64_t* os) {
    if (c->L.D != PD) return false;
    if (!((c->L.fmt == B200KV_FMT_F16 && dtype == B200KV_F16) || (c->L.fmt == B200KV_FMT_BF16 && dtype == B200KV_BF16))) return false;
    const int G = n_q_heads / c->L.Hkv;
    if (G < 1 || G > PM) return false;
    // 16-byte vector access to the q and out rows
    auto aligned = [](const void* ptr, const int64_t* st) {
        return (uintptr_t)ptr % 16 == 0 && (st[0] * 2) % 16 == 0 && (st[1] * 2) % 16 == 0 && (st[2] * 2) % 16 == 0;
    };
    return aligned(q, qs) && aligned(out, os);
}

template <int NQ>
static cudaError_t launch_tiles(const PrefillParams& p, int n_seqs, cudaStream_t stream) {
    using GEO = PGeo<NQ>;
    cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEO::SMEM);
    if (e != cudaSuccess) return e;
    const int per_cta = NQ * (PM / p.G);
    dim3 grid((p.S + per_cta - 1) / per_cta, p.Hkv, n_seqs);
    prefill_tc_kernel<NQ><<<grid, GEO::THREADS, GEO::SMEM, stream>>>(p);
    return cudaGetLastError();
}

int launch_prefill_tc(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, int32_t n_new, const void* q,
                      const int64_t* qs, void* out, const int64_t* os, int32_t dtype, float scale, int causal,
                      cudaStream_t stream) {
    const int G = n_q_heads / c->L.Hkv;
    int slot;
    uint8_t *h, *d;
    if (staging_acquire(c, (size_t)n_seqs * 8, &slot, &h, &d) != B200KV_OK) return B200KV_KO;
    int32_t* hw = (int32_t*)h;
    for (int i = 0; i < n_seqs; i++) {
        hw[2 * i] = seqs[i];
        hw[2 * i + 1] = (int32_t)c->seqs[seqs[i]].len;
    }
    if (staging_upload(c, slot, (size_t)n_seqs * 8, stream) != B200KV_OK) {
        staging_release(c, slot, stream);
        return B200KV_KO;
    }
    PrefillParams p{};
    p.pool = c->pool, p.table = c->d_table, p.desc = (const int32_t*)d, p.status = c->d_status;
    p.q = q, p.out = out;
    p.qb = qs[0], p.qh = qs[1], p.qs = qs[2], p.ob = os[0], p.oh = os[1], p.os = os[2];
    p.page_bytes = c->L.page_bytes, p.n_pages = (int32_t)c->n_pages, p.max_pages_per_seq = c->max_pages_per_seq;
    p.Hkv = c->L.Hkv, p.G = G, p.S = n_new, p.causal = causal, p.is_bf16 = dtype == B200KV_BF16;
    // V chunk = 2 planes of 64 channels (8192 bytes apart), 8-token groups 1024 bytes apart
    p.v_lbo = 8192, p.v_sbo = 1024;
    p.scale = scale;
    p.skip_fraction = P_SKIP_FRACTION;
    // double tiles (one CTA per SM, K/V staged once for 2 x 128 rows) when they still fill the GPU
    const int qpt = PM / G;
    const int64_t double_ctas = (int64_t)((n_new + 2 * qpt - 1) / (2 * qpt)) * c->L.Hkv * n_seqs;
    cudaError_t e;
    {
        ProfScope ps(c, K_PREFILL, stream);
        e = double_ctas >= 148 /* SMs of a B200 */ ? launch_tiles<2>(p, n_seqs, stream) : launch_tiles<1>(p, n_seqs, stream);
    }
    staging_release(c, slot, stream);
    if (e != cudaSuccess) return fail("prefill launch failed: %s", cudaGetErrorString(e));
    return B200KV_OK;
}

}  // namespace b200kv
