// tcgen05 / TMEM wrappers and the small synchronisation helpers shared by the tensor-core attention kernels.
#pragma once
#include "f32x2.cuh"
#include "internal.h"

namespace b200kv {

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
// The same, saying what becomes of the A operand in the tensor core's collector buffer: the first product of a run that
// shares its A slice fills the buffer (KEEP), the last one takes it from there and releases it (REUSE_LAST).  A 128 x 16
// slice is 4 KB of shared-memory reads; measured on 128 x 64 x 16 products, back to back: 48 cycles each when every
// product loads its A, 76 per pair when the second reuses it.
enum { A_KEEP = 0, A_REUSE_LAST = 1 };
template <int USAGE>
__device__ inline void tc_mma_ss_a(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (USAGE == A_KEEP)
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16.collector::a::fill [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16.collector::a::lastuse [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
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
__device__ inline void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
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
__device__ inline void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]),
                 "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
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
// The same on bit patterns, and not to be moved past its neighbours: a run of these stays a run, so that the unit has a
// warp's exponentials in its queue instead of one at a time.
__device__ inline uint32_t ex2_in_order(uint32_t x) {
    uint32_t y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ inline float fast_log2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}


// ---- the softmax of one row of 64 scores, shared by the attention kernels (one thread per row) ----------------------
// One pair of exponentials in this many goes through a polynomial on the FMA pipe instead of the MUFU unit; 0: none.
// Measured on an 8192-token causal chunk: 0 -> 0.533 ms, 4 -> 0.532 ms, 3 -> 0.532 ms, 2 -> 0.556 ms; on 8 x 512 queries
// after 7680 tokens 0.644 / 0.656 / 0.658 / 0.683 ms: with the exponentials pipelined the MUFU unit is not what a tile
// waits for (its products queue behind the other tile's on the one tensor pipe), and the extra instructions cost power.
constexpr int SOFTMAX_POLY_EVERY = 0;
constexpr int SOFTMAX_LAG = 4;    // pairs between an exponential's issue and its use
constexpr int SOFTMAX_AHEAD = 2;  // pairs whose exponent is computed ahead of its exponential
__host__ __device__ constexpr bool softmax_poly_pair(int c) {
    return SOFTMAX_POLY_EVERY > 0 && c % (SOFTMAX_POLY_EVERY > 0 ? SOFTMAX_POLY_EVERY : 1) == SOFTMAX_POLY_EVERY - 1;
}
__device__ inline float row_max64(const uint32_t (&sr)[64]) {
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int c = 0; c < 64; c += 8)
#pragma unroll
        for (int e = 0; e < 4; e++) mx[e] = fmax3(mx[e], __uint_as_float(sr[c + 2 * e]), __uint_as_float(sr[c + 2 * e + 1]));
    return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}
// sr: the row's raw scores (bit patterns; overwritten).  P = 2^(s * sl2 - m), returned as its 16-bit roundings in pr (pairs
// of neighbouring columns) and, MODE 1 / 2, what the rounding lost in pr2 (MODE 0: zeros); the return value is the sum of
// the unrounded P.  MODE 0: f16 value only, 1: f16 value + remainder, 2: bf16 value + remainder.
// Written as a software pipeline, because a warp issues in order: pair c's exponentials go to the MUFU unit while the pair
// that left it SOFTMAX_LAG pairs ago is summed and rounded, so the unit (one warp instruction every 8 cycles) always has
// this warp's next exponentials queued and the issue slots in between carry the rest of the row's work.  A warp that
// consumes each result as it arrives keeps two in flight and waits out the unit's latency 32 times per row: measured 73
// cycles per pair against 16.
template <int MODE>
__device__ inline float softmax_exps(uint32_t (&sr)[64], float sl2, float m, uint32_t (&pr)[32], uint32_t (&pr2)[32]) {
    const uint64_t sl2_2 = f2_pack(sl2, sl2), negm2 = f2_pack(-m, -m);
    uint64_t ls[4] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};
    auto exponent = [&](int c) {
        const uint2 x = f2_unpack_bits(f2_fma(f2_pack_bits(sr[2 * c], sr[2 * c + 1]), sl2_2, negm2));
        sr[2 * c] = x.x, sr[2 * c + 1] = x.y;
    };
#pragma unroll
    for (int c = 0; c < SOFTMAX_AHEAD; c++) exponent(c);
#pragma unroll
    for (int c = 0; c < 32 + SOFTMAX_LAG; c++) {
        if (c + SOFTMAX_AHEAD < 32) exponent(c + SOFTMAX_AHEAD);
        if (c < 32) {
            if (softmax_poly_pair(c)) {
                const float2 e = exp2_poly2(f2_pack_bits(sr[2 * c], sr[2 * c + 1]));
                sr[2 * c] = __float_as_uint(e.x), sr[2 * c + 1] = __float_as_uint(e.y);
            } else {
                sr[2 * c] = ex2_in_order(sr[2 * c]), sr[2 * c + 1] = ex2_in_order(sr[2 * c + 1]);
            }
        }
        if (c >= SOFTMAX_LAG) {
            const int d = c - SOFTMAX_LAG;
            ls[d & 3] = f2_add(ls[d & 3], f2_pack_bits(sr[2 * d], sr[2 * d + 1]));
            const float e0 = __uint_as_float(sr[2 * d]), e1 = __uint_as_float(sr[2 * d + 1]);
            if (MODE == 2) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
                const __nv_bfloat162 l = __floats2bfloat162_rn(e0 - __low2float(h), e1 - __high2float(h));
                pr[d] = *(const uint32_t*)&h, pr2[d] = *(const uint32_t*)&l;
            } else {
                const __half2 h = __floats2half2_rn(e0, e1);
                pr[d] = *(const uint32_t*)&h;
                if (MODE == 1) {
                    const __half2 l = __floats2half2_rn(e0 - __low2float(h), e1 - __high2float(h));
                    pr2[d] = *(const uint32_t*)&l;
                } else {
                    pr2[d] = 0u;
                }
            }
        }
    }
    const float2 t = f2_unpack(f2_add(f2_add(ls[0], ls[1]), f2_add(ls[2], ls[3])));
    return t.x + t.y;
}

__device__ inline bool mbar_test(uint64_t* bar, uint32_t parity) {  // one look, never suspends
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for a barrier phase unless the CTA has already failed; gives up after ~1 s and marks the CTA failed.
__device__ inline void wait_or_fail(uint64_t* bar, uint32_t parity, volatile int* fail) {
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
// One lane of a converged warp (always the same one).
__device__ inline bool elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
    return pred != 0;
}
__device__ inline void pair_barrier(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

}  // namespace b200kv
