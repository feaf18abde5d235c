// Flash-attention prefill over the paged cache on the 5th-generation tensor cores (tcgen05 + TMEM):
// the S > 1 case of b200kv_attend for f16 / bf16 caches at head_dim 128.
//
// Replaces the prefill use of cuda/src/kernels/cu/flash_attn.cu (`attention_fullq_*`: Ampere mma.sync,
// one q-head per CTA so every head of a GQA group re-streams K/V).  Semantics:
// transformers/src/ops/flash_sdpa.rs:239-341 (causal aligned bottom-right, scale, f32 accumulation).
//
// One CTA = one 128-row query tile of one (sequence, kv head): the rows are (query, head-of-group) pairs,
// so the whole GQA group shares each K/V page.  Per page of 64 cached tokens:
//   S[128 x 64]  = Q . K^T      tcgen05.mma, A = Q tile in shared memory (K-major, 128-byte swizzle),
//                               B = the K chunk exactly as it lies in the page (same swizzle), D in TMEM
//   softmax                     two threads own a row: each tcgen05.ld's 32 of its 64 scores, masks, exponentiates in the
//                               log2 domain against a lazily raised reference maximum, write P (16-bit)
//                               back to TMEM with tcgen05.st
//   O[128 x 128] += P . V       tcgen05.mma, A = P from TMEM (as a 16-bit value plus its 16-bit rounding remainder:
//                               two MMAs), B = the V chunk as it lies in the page
//                               (MN-major operand: channels contiguous), D accumulates in TMEM
// K/V chunks arrive by untiled cp.async.bulk into a two-stage ring; two CTAs fit per SM so that one CTA's
// softmax overlaps the other's MMAs.  Every wait is bounded; on expiry the CTA flags the status word,
// frees its TMEM and returns.
#include <cmath>

#include "internal.h"

namespace b200kv {

constexpr int PD = 128;        // head_dim
constexpr int PM = 128;        // rows of a query tile
constexpr int P_NS = 2;        // K/V stages
constexpr int P_CHUNK = PAGE_TOKENS * PD * 2;  // bytes of one K (or V) chunk: 16 KiB
constexpr int P_STAGE = 2 * P_CHUNK;
constexpr int P_QBYTES = PM * PD * 2;          // 32 KiB
constexpr uint32_t TMEM_COLS = 256;            // O: 128 columns, S: 64, P: 32 (16-bit pairs), P remainder: 32
constexpr uint32_t COL_O = 0, COL_S = 128, COL_P = 192, COL_P2 = 224;

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
};

// ---- tcgen05 wrappers -------------------------------------------------------------------------------
__device__ inline void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ inline void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ inline void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ inline void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] . B[smem]
__device__ inline void tc_mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]
__device__ inline void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane
__device__ inline void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ inline void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ inline void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ inline void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ inline void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 descriptor version.
__device__ inline uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((saddr & 0x3ffffu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: f32 accumulation, 16-bit operands, M x N tile.
__host__ __device__ constexpr uint32_t instr_desc(int bf16, int b_mn_major, int M, int N) {
    return (1u << 4) | ((uint32_t)bf16 << 7) | ((uint32_t)bf16 << 10) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ inline float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int P_THREADS = 256;

// Two threads share a row of the 128-row tile: warps w and w + 4 both address TMEM lanes 32 (w & 3) .. + 32;
// the first takes score columns 0..31 and output channels 0..63, the second the other halves.
__global__ void __launch_bounds__(P_THREADS, 2) prefill_tc_kernel(PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* q_s = smem;                    // [2 planes][128 rows][128 B], swizzled
    uint8_t* stages = smem + P_QBYTES;      // P_NS x (K chunk, V chunk)
    uint64_t* bar_full = (uint64_t*)(stages + P_NS * P_STAGE);  // [P_NS]
    uint64_t* bar_mma = bar_full + P_NS;                        // [1]
    uint32_t* tmem_slot = (uint32_t*)(bar_mma + 1);
    int* fail_s = (int*)(tmem_slot + 1);
    float* xchg = (float*)(fail_s + 1);     // [2 halves][128 rows]: row maxima, later row sums

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = (warp & 3) * 32 + lane, half = warp >> 2;
    const int kvh = blockIdx.y, b = blockIdx.z;
    const int G = p.G, qpt = PM / G;              // queries per tile
    const int q0 = blockIdx.x * qpt;              // first query of this tile
    const int32_t trow = p.desc[2 * b], T = p.desc[2 * b + 1];
    const int P0 = T - p.S;                       // cached tokens before the first new query
    // row -> (query, head of the group); rows past the tile's queries are dead
    const int rq = row / G, rg = row % G;
    const bool live = rq < qpt && q0 + rq < p.S;
    const int q_last = min(q0 + qpt, p.S) - 1;    // last live query of the tile
    const int my_q = live ? q0 + rq : q_last;
    const int my_limit = p.causal ? P0 + my_q : T - 1;           // last visible key of this row
    const int tile_limit = p.causal ? P0 + q_last : T - 1;       // last key any row of the tile sees
    const int min_limit = p.causal ? P0 + q0 : T - 1;            // last key EVERY row of the tile sees
    const int n_tiles = tile_limit / PAGE_TOKENS + 1;

    if (tid == 0) {
        for (int s = 0; s < P_NS; s++) mbar_init(&bar_full[s], 1);
        mbar_init(bar_mma, 1);
        *fail_s = (smem_u32(smem) & 1023u) ? 1 : 0;  // the swizzled operand tiles need a 1024-byte aligned base
        mbar_fence_init();
    }
    auto issue_load = [&](int j) {  // thread 0
        const int st = j % P_NS;
        int32_t pg = p.table[(int64_t)trow * p.max_pages_per_seq + j];
        if (pg < 0 || pg >= p.n_pages) {
            atomicOr(p.status, STATUS_PAGE_OOB);
            pg = 0;
        }
        mbar_expect_tx(&bar_full[st], P_STAGE);
        bulk_g2s(stages + st * P_STAGE, p.pool + (int64_t)pg * p.page_bytes + (int64_t)kvh * P_STAGE, P_STAGE, &bar_full[st]);
    };
    if (tid == 0)
        for (int j = 0; j < P_NS && j < n_tiles; j++) issue_load(j);
    if (warp == 0) tmem_alloc(tmem_slot, TMEM_COLS);

    // ---- Q tile -> shared memory, K-major with the 128-byte swizzle (row r: 16-byte unit u of plane pl at u ^ (r & 7));
    //      this thread moves the 64 channels of plane `half` of its row ----
    {
        const int head = kvh * G + rg;
        const uint4* src = (const uint4*)((const uint16_t*)p.q + (int64_t)b * p.qb + (int64_t)head * p.qh + (int64_t)my_q * p.qs) + half * 8;
#pragma unroll
        for (int uu = 0; uu < 8; uu++) {
            uint4 v = live ? src[uu] : make_uint4(0, 0, 0, 0);
            *(uint4*)(q_s + half * (PM * 128) + row * 128 + ((uu ^ (row & 7)) << 4)) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*fail_s) {
        if (tid == 0) atomicOr(p.status, STATUS_WAIT_EXPIRED);
        if (warp == 0) tmem_dealloc(*tmem_slot, TMEM_COLS);
        return;
    }
    const uint32_t tmem = *tmem_slot;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's quarter of the 128 lanes
    const uint32_t idesc_s = instr_desc(p.is_bf16, 0, PM, PAGE_TOKENS);
    const uint32_t idesc_o = instr_desc(p.is_bf16, 1, PM, PD);
    const uint32_t q_addr = smem_u32(q_s);

    auto issue_s = [&](int j) {  // thread 0: S = Q . K^T for tile j (8 MMAs of K = 16)
        const uint32_t k_addr = smem_u32(stages + (j % P_NS) * P_STAGE);
#pragma unroll
        for (int pl = 0; pl < 2; pl++)
#pragma unroll
            for (int kk = 0; kk < 4; kk++)
                tc_mma_ss(tmem + COL_S, smem_desc(q_addr + pl * (PM * 128) + kk * 32, 0, 1024),
                          smem_desc(k_addr + pl * (PAGE_TOKENS * 128) + kk * 32, 0, 1024), idesc_s, (pl | kk) ? 1u : 0u);
        tc_commit(bar_mma);
    };

    bool ok = true;
    if (tid == 0) {
        ok = mbar_wait_bounded(&bar_full[0], 0);
        if (ok) issue_s(0);
    }

    const float sl2 = p.scale * 1.4426950408889634f;  // scores enter the exponent in log2 units
    float m_ref = -INFINITY, l_run = 0.f;             // l_run: this thread's half of the row sum

    for (int j = 0; j < n_tiles; j++) {
        // S(j) ready; every MMA issued before it (P.V of tile j-1) has completed as well
        ok = ok && mbar_wait_bounded(bar_mma, (uint32_t)(j & 1));
        tc_fence_after();
        // ---- this thread's 32 of the row's 64 scores ----
        uint32_t sr[32];
        tmem_ld32(lane_base + COL_S + 32 * half, sr);
        tmem_ld_wait();
        float tmax = -INFINITY;
        if (j * PAGE_TOKENS + PAGE_TOKENS - 1 > min_limit) {  // only tiles on the causal diagonal / past the end need a mask
            const int t0 = j * PAGE_TOKENS + 32 * half;
#pragma unroll
            for (int c = 0; c < 32; c++) {
                const float s = (t0 + c <= my_limit) ? __uint_as_float(sr[c]) : -INFINITY;
                sr[c] = __float_as_uint(s);
                tmax = fmaxf(tmax, s);
            }
        } else {
#pragma unroll
            for (int c = 0; c < 32; c++) tmax = fmaxf(tmax, __uint_as_float(sr[c]));
        }
        xchg[half * PM + row] = tmax;
        if (__syncthreads_or(!ok)) {  // also the barrier of the maxima exchange
            ok = false;
            break;
        }
        // stage of tile j-1 is free now: refill it
        if (tid == 0 && j >= 1 && j - 1 + P_NS < n_tiles) issue_load(j - 1 + P_NS);
        tmax = fmaxf(tmax, xchg[(half ^ 1) * PM + row]) * sl2;
        // raise the reference maximum only when it is exceeded by more than 2^8: the exponentials stay below
        // 256, exact enough in 16 bits, and O has to be rescaled only rarely
        float alpha = 1.f;
        if (j == 0) {
            m_ref = tmax;
        } else if (tmax > m_ref + 8.f) {
            alpha = fast_exp2(m_ref - tmax);
            m_ref = tmax;
            l_run *= alpha;
        }
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {  // this thread's 64 of the row's 128 output channels
                uint32_t orow[32];
                tmem_ld32(lane_base + COL_O + 64 * half + cc * 32, orow);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; c++) orow[c] = __float_as_uint(__uint_as_float(orow[c]) * alpha);
                tmem_st32(lane_base + COL_O + 64 * half + cc * 32, orow);
            }
        }
        // P goes to the tensor core as two 16-bit operands, the rounded value and the rounding remainder:
        // a row that sees only a few keys gets no averaging of the 2^-11 (f16) / 2^-8 (bf16) rounding errors,
        // and with the remainder the product P . V is exact to ~2^-22
        uint32_t pr[16], pr2[16];
        float lsum = 0.f;
#pragma unroll
        for (int c = 0; c < 16; c++) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sr[2 * c]), sl2, -m_ref));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sr[2 * c + 1]), sl2, -m_ref));
            lsum += p0 + p1;
            if (p.is_bf16) {
                __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                __nv_bfloat162 l = __floats2bfloat162_rn(p0 - __low2float(h), p1 - __high2float(h));
                pr[c] = *(uint32_t*)&h, pr2[c] = *(uint32_t*)&l;
            } else {
                __half2 h = __floats2half2_rn(p0, p1);
                __half2 l = __floats2half2_rn(p0 - __low2float(h), p1 - __high2float(h));
                pr[c] = *(uint32_t*)&h, pr2[c] = *(uint32_t*)&l;
            }
        }
        l_run += lsum;
        tmem_st16(lane_base + COL_P + 16 * half, pr);
        tmem_st16(lane_base + COL_P2 + 16 * half, pr2);
        tmem_st_wait();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            // O (+)= P . V : 4 MMAs of K = 16 tokens; the V chunk is an MN-major operand
            const uint32_t v_addr = smem_u32(stages + (j % P_NS) * P_STAGE + P_CHUNK);
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                const uint64_t vdesc = smem_desc(v_addr + kk * 2048, p.v_lbo, p.v_sbo);
                tc_mma_ts(tmem + COL_O, tmem + COL_P + kk * 8, vdesc, idesc_o, (j | kk) ? 1u : 0u);
                tc_mma_ts(tmem + COL_O, tmem + COL_P2 + kk * 8, vdesc, idesc_o, 1u);
            }
            if (j + 1 < n_tiles) {
                ok = mbar_wait_bounded(&bar_full[(j + 1) % P_NS], (uint32_t)(((j + 1) / P_NS) & 1));
                if (ok) issue_s(j + 1);  // commits for S(j+1) and, in order, for P.V(j)
            } else {
                tc_commit(bar_mma);
            }
        }
    }
    // ---- epilogue: wait for the last P.V, normalise, store ----
    if (ok) ok = mbar_wait_bounded(bar_mma, (uint32_t)(n_tiles & 1));
    xchg[half * PM + row] = l_run;
    ok = !__syncthreads_or(!ok);
    if (ok) {
        tc_fence_after();
        const float inv = 1.f / (l_run + xchg[(half ^ 1) * PM + row]);
        uint16_t* dst = (uint16_t*)p.out + (int64_t)b * p.ob + (int64_t)(kvh * G + rg) * p.oh + (int64_t)my_q * p.os + 64 * half;
#pragma unroll
        for (int cc = 0; cc < 2; cc++) {
            uint32_t orow[32];
            tmem_ld32(lane_base + COL_O + 64 * half + cc * 32, orow);
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
    } else {
        if (tid == 0) atomicOr(p.status, STATUS_WAIT_EXPIRED);
        __nanosleep(200000);  // give copies that may still be in flight time to land before the CTA's memory is released
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
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
    if (staging_upload(c, slot, (size_t)n_seqs * 8, stream) != B200KV_OK) return B200KV_KO;
    PrefillParams p{};
    p.pool = c->pool, p.table = c->d_table, p.desc = (const int32_t*)d, p.status = c->d_status;
    p.q = q, p.out = out;
    p.qb = qs[0], p.qh = qs[1], p.qs = qs[2], p.ob = os[0], p.oh = os[1], p.os = os[2];
    p.page_bytes = c->L.page_bytes, p.n_pages = (int32_t)c->n_pages, p.max_pages_per_seq = c->max_pages_per_seq;
    p.Hkv = c->L.Hkv, p.G = G, p.S = n_new, p.causal = causal, p.is_bf16 = dtype == B200KV_BF16;
    // V chunk = 2 planes of 64 channels (8192 bytes apart), 8-token groups 1024 bytes apart
    p.v_lbo = 8192, p.v_sbo = 1024;
    p.scale = scale;
    const size_t smem = P_QBYTES + (size_t)P_NS * P_STAGE + 64 + 2 * PM * 4;
    B200KV_CUDA(cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int qpt = PM / G;
    dim3 grid((n_new + qpt - 1) / qpt, c->L.Hkv, n_seqs);
    {
        ProfScope ps(c, K_PREFILL, stream);
        prefill_tc_kernel<<<grid, P_THREADS, smem, stream>>>(p);
    }
    cudaError_t e = cudaGetLastError();
    staging_release(c, slot, stream);
    if (e != cudaSuccess) return fail("prefill launch failed: %s", cudaGetErrorString(e));
    return B200KV_OK;
}

}  // namespace b200kv
