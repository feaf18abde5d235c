// Flash attention of many queries on the 5th-generation tensor cores (tcgen05 + TMEM) for every source the specialised
// f16 / bf16 head_dim-128 kernel of prefill_tc.cu does not read: block-quantised pages (Q8_1, Q4_0), head_dim 64, and
// dense strided K / V tensors with an optional additive mask (the lone Sdpa node), and the KIVI stores of
// QuantizedDynKeyValueCache at head_dim 128.
//
// Replaces cuda/src/kernels/cu/flash_attn.cu (`attention_kernel`, instantiated for head_dim 64 and 128, :587-627; Ampere
// mma.sync, one q-head per CTA) behind CudaFlashAttn::dispatch_eval (cuda/src/kernels/flash_attn.rs:82-189), and gives
// the quantised caches what the reference does by rebuilding the whole f32 cache for every chunk
// (transformers/src/ops/quant_dyn_kv_cache.rs:432-449): here a chunk of queries walks the pages it needs and nothing
// else, and each page is widened to 16 bits in shared memory on its way to the tensor cores.
// Semantics: transformers/src/ops/flash_sdpa.rs:239-341 (scale, additive mask or causal aligned bottom-right, f32
// accumulation); masks as transformers/src/ops/sdpa.rs:183-196 adds them.
//
// The pipeline is that of prefill_tc.cu: a query tile is 128 rows = (query, head-of-group) pairs of one (sequence, kv
// head); per tile and per 64 keys  S = Q . K^T  (tcgen05.mma, operands in shared memory with the 128-byte swizzle, S
// double-buffered in TMEM), softmax by one thread per row (tcgen05.ld, exponentials in the log2 domain against a
// lazily raised reference maximum, P written over S with tcgen05.st as a 16-bit value plus its rounding remainder),
// O += P . V  (A from TMEM, V as an MN-major operand).  What differs is who fills the K / V operand rings:
//   SRC_PAGES16  a copy warp: one untiled cp.async.bulk per chunk, the page bytes ARE the operand tile (head_dim 64 here)
//   SRC_Q8, _Q4  the raw quantised chunk pair of a page lands (cp.async.bulk) in a small ring; four converter warps turn
//                code * f32(f16 scale) (q8_1.rs:50-63, q4_0.rs:82-95) into f16 rows of the operand tiles, and the first of
//                them requests the raw pages.  The operands are f16 whatever the query type (bf16 queries are widened
//                to f16 on their way in: bf16 would keep 8 bits of a dequantised value), and K goes in as the rounded
//                product plus its exact remainder (two tiles, two products per score): with sharply peaked attention
//                the 2^-12 that rounding K to f16 loses is visible in the scores, while V tolerates it
//   SRC_KIVI8/4  the same for the stores of transformers/src/ops/quant_dyn_kv_cache.rs: keys 0 .. 3 are the f32 sinks, key
//                4 + i sits in slot i % 64 of storage page i / 64, so a tile of 64 keys is the last 4 slots of one page
//                (carried over in shared memory from the tile before) and the first 60 of the next; keys of finalised
//                32-token blocks are lo[c] + code * scale[c], the rest come from the f32 residual rows, values are
//                lo_t + code * scale_t (:141-146, :231-240)
//   SRC_DENSE    two loader warps gather 16-byte units of the strided K / V rows with cp.async straight into the
//                swizzled tile, two pages in flight; rows past the end of K / V are zero-filled
// Every wait is bounded; on expiry the CTA flags the status word, every role runs to the end of its loop without
// waiting any more, the CTA frees its TMEM and returns.
#include <cmath>
#include <type_traits>

#include "kivi_common.cuh"
#include "tc_common.cuh"

namespace b200kv {

constexpr int AM = 128;            // rows of a query tile
constexpr int A_SM_THREADS = 128;  // softmax threads per query tile: one per row
constexpr int A_FILL_THREADS = 64; // converter / loader threads (the KIVI converter and the dense loader; block formats: FT)
constexpr int A_XCHG = 8;          // per tile and page parity: one flag per softmax warp (does the page need its remainder product)
constexpr float A_SKIP_FRACTION = 0.125f;
enum { SRC_PAGES16 = 0, SRC_Q8 = 1, SRC_DENSE = 2, SRC_KIVI8 = 3, SRC_Q4 = 4, SRC_KIVI4 = 5 };
constexpr bool src_is_kivi(int src) { return src == SRC_KIVI8 || src == SRC_KIVI4; }
constexpr bool src_is_block(int src) { return src == SRC_Q8 || src == SRC_Q4; }
constexpr int A_KIVI_KP = 2 * 2 * 128 * 4;        // K parameters of a page: 2 blocks x (lo[128], scale[128]) f32
constexpr int A_KIVI_VP = PAGE_TOKENS * 2 * 4;    // V parameters of a page: (lo, scale) f32 per token
constexpr int A_CARRY = 2 * SINK * 128 * 2;      // f16 K and V rows of the last 4 slots of a KIVI page: they open the next tile (the K remainders follow)

template <int NQ, int D, int SRC, int FT = A_FILL_THREADS>
struct AGeo {
    static constexpr int PLANES = D / 64;             // 128-byte wide column slabs of a row
    static constexpr int CHUNK = PAGE_TOKENS * D * 2; // bytes of one K (or V) operand tile: 64 keys
    static constexpr int QBYTES = AM * D * 2;
    static constexpr bool FILL = SRC != SRC_PAGES16;
    static constexpr bool RAW = src_is_block(SRC) || src_is_kivi(SRC);  // a ring of raw page bytes beside the operand rings
    static constexpr int KPARTS = RAW ? 2 : 1;                          // K operand tiles per 64 keys: value, or value + remainder
    static constexpr int KSTAGE = KPARTS * CHUNK;
    static constexpr int NK = RAW ? 2 : (NQ == 2 ? 4 : 3);              // K stages
    static constexpr int NV = RAW ? 3 : (NQ == 2 ? 5 : 4);              // V stages
    static constexpr int NR = 2;                                        // raw stages
    static constexpr int RAW_STAGE = src_is_block(SRC) ? 2 * (PAGE_TOKENS * D + PAGE_TOKENS * (D / 32) * 2)   // a Q8_1 chunk pair (Q4_0: smaller)
                                     : src_is_kivi(SRC) ? 2 * PAGE_TOKENS * D + A_KIVI_KP + A_KIVI_VP         // int8 codes of K and V, their parameters
                                                        : 0;
    // softmax threads, one MMA warp per tile, then either the copy warp (16-bit pages) or the converter / loader warps
    static constexpr int THREADS = NQ * A_SM_THREADS + 32 * NQ + (FILL ? FT : 32);
    static constexpr int N_BARS = 2 * NK + 2 * NV + 6 * NQ + 2 * NR;
    static constexpr uint32_t COL_S = D, COLS_PER_TILE = 256;  // TMEM: O in columns 0 .. D-1, the two S buffers after it
    static constexpr size_t SMEM = (size_t)NQ * QBYTES + (size_t)NK * KSTAGE + (size_t)NV * CHUNK + (size_t)NR * RAW_STAGE + N_BARS * 8 + 32 +
                                   NQ * 2 * A_XCHG * 4 + (src_is_kivi(SRC) ? A_CARRY + A_CARRY / 2 : 0);
};

struct AttnParams {
    const void* q;
    void* out;
    int64_t qb, qh, qs, ob, oh, os;
    int* status;
    int32_t Hkv, G, S, causal, is_bf16;
    float scale, inv_scale, skip_fraction;
    // paged sources
    const uint8_t* pool;
    const int32_t* table;
    const int32_t* desc;  // per batch entry: {table row, cached length}
    int64_t page_bytes;
    int32_t n_pages, max_pages_per_seq, fmt, chunk_bytes;
    // dense source: K / V [B, Hkv, T, D] with strides {batch, head, row} in elements, T keys
    const void* k;
    const void* v;
    int64_t kb, kh, ks, vb, vh, vs;
    int32_t T;
    // additive mask [Mb, Mh, S, T], strides {batch, head, row, column} in elements (0 to broadcast); null: none
    const void* mask;
    int64_t mb, mh, mq, mk;
    int32_t mask_dtype;
    // KIVI stores; desc then holds {sequence, cached length} per batch entry
    KiviView kv;
};

__device__ inline void cp_async16_zfill(void* dst_smem, const void* src, bool live) {
    const uint32_t n = live ? 16u : 0u;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(__cvta_generic_to_global(src)), "r"(n) : "memory");
}
__device__ inline void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ inline void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ inline void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- block-quantised chunk -> f16 operand tile(s) ----------------------------------------------------------------------
// Codes become exact f16 integers with byte permutes and one packed subtraction (0x6400 | u is the f16 1024 + u), the
// product with the f16 scale is one packed multiply, rounded once: RN_f16(code * scale), what rounding the reference's
// exact f32 product to f16 gives; for K a packed FMA returns the remainder code * scale - RN(code * scale), exact.
constexpr uint32_t H_MAGIC = 0x64646464u;  // source of the 0x64 high bytes
__device__ inline uint32_t hsub2(uint32_t a, uint32_t b) {
    const __half2 r = __hsub2(*(const __half2*)&a, *(const __half2*)&b);
    return *(const uint32_t*)&r;
}
__device__ inline uint32_t hmul2(uint32_t a, uint32_t b) {
    const __half2 r = __hmul2(*(const __half2*)&a, *(const __half2*)&b);
    return *(const uint32_t*)&r;
}
__device__ inline uint32_t hfma2_rem(uint32_t a, uint32_t b, uint32_t prod) {  // a * b - prod
    const __half2 r = __hfma2(*(const __half2*)&a, *(const __half2*)&b, __hneg2(*(const __half2*)&prod));
    return *(const uint32_t*)&r;
}
// where unit u (8 channels, 16 bytes) of row `row` lies in an operand tile
__device__ inline uint32_t tile_off(int u, int row) { return (u / 8) * (PAGE_TOKENS * 128) + row * 128 + (((u % 8) ^ (row & 7)) << 4); }

// Thread t of the FT converter threads takes item t % (D / 16) -- 16 channels, two units of 8 -- of every (16 FT / D)-th
// token: the 16 codes of an item come from one 16- or 8-byte load of a natural row (Q4_0: low and high nibbles of the same
// 8 bytes are the two units), or from 8 two-byte (Q8_1) / one-byte (Q4_0) loads of a permuted V row.  `lo_tile` (K): the
// tile that takes the remainders.  Rows from n_valid on are zero-filled.
template <int FMT, int D, int KV, int FT, bool FULL>
__device__ inline void convert_rows(const uint8_t* raw, uint8_t* hi_tile, uint8_t* lo_tile, int n_valid, int t) {
    constexpr bool PERM = v_permuted(FMT, D, KV), Q8 = FMT == B200KV_FMT_Q8_1, SPLIT = KV == 0;
    constexpr int ITEMS = D / 16, TLN = FT / ITEMS;
    constexpr uint32_t BIAS = Q8 ? 0x64806480u : 0x64086408u;  // f16 pair 1024 + 128 | 1024 + 8: what the codes are offset by
    const int item = t % ITEMS, tl = t / ITEMS;
    const __half* scales = (const __half*)(raw + PAGE_TOKENS * fmt_row_bytes(FMT, D));
    // The two units the item yields, and their blocks.  At head_dim 128 a quarter warp (one 16-byte store phase) is the eight
    // items of one token, four per 64-channel plane, and the planes lie a multiple of the bank width apart: if every item
    // stored its lower unit first, the planes would collide two ways in every store.  The items of the second plane
    // therefore take their units in the other order (`sw`): each phase then covers eight different 16-byte slots.
    const bool sw = D == 128 && (item & 4);
    int ua, ub;
    if (Q8 || PERM) ua = 2 * item + (sw ? 1 : 0), ub = 2 * item + (sw ? 0 : 1);
    else ua = 4 * (item / 2) + (item % 2) + (sw ? 2 : 0), ub = 4 * (item / 2) + (item % 2) + (sw ? 0 : 2);  // Q4_0 natural: bytes 16b + 8q .. hold channels 32b + 8q .. (low) and + 16 (high)
    const int blk_a = ua / 4, blk_b = ub / 4;
    const uint32_t sel_a = sw ? 0x4341u : 0x4240u, sel_b = sw ? 0x4240u : 0x4341u;  // permuted Q8_1 rows: which byte of a pair
    const int sh_a = sw ? 4 : 0, sh_b = sw ? 0 : 4;                                  // permuted Q4_0 rows: which nibble
#pragma unroll 4
    for (int tt = 0; tt < PAGE_TOKENS / TLN; tt++) {  // independent tokens: unrolled so that their loads and chains overlap
        const int tok = tt * TLN + tl;
        uint32_t ca[4], cb[4];  // f16 pairs: the codes of unit ua / ub as 1024 + u
        if constexpr (Q8 && !PERM) {
            const uint4 x = *(const uint4*)(raw + chunk_addr(FMT, D, KV, tok, 16 * item));
            const uint32_t w0 = sw ? x.z : x.x, w1 = sw ? x.w : x.y, w2 = sw ? x.x : x.z, w3 = sw ? x.y : x.w;
            ca[0] = __byte_perm(w0, H_MAGIC, 0x4140), ca[1] = __byte_perm(w0, H_MAGIC, 0x4342);
            ca[2] = __byte_perm(w1, H_MAGIC, 0x4140), ca[3] = __byte_perm(w1, H_MAGIC, 0x4342);
            cb[0] = __byte_perm(w2, H_MAGIC, 0x4140), cb[1] = __byte_perm(w2, H_MAGIC, 0x4342);
            cb[2] = __byte_perm(w3, H_MAGIC, 0x4140), cb[3] = __byte_perm(w3, H_MAGIC, 0x4342);
        } else if constexpr (Q8) {  // permuted V row: bytes 16r + 2 item, + 1 hold channels 16 item + r and + 8
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t h0 = *(const uint16_t*)(raw + chunk_addr(FMT, D, KV, tok, 16 * (2 * i) + 2 * item));
                const uint32_t h1 = *(const uint16_t*)(raw + chunk_addr(FMT, D, KV, tok, 16 * (2 * i + 1) + 2 * item));
                const uint32_t both = __byte_perm(h0, h1, 0x5410);  // [low r, high r, low r + 1, high r + 1]
                ca[i] = __byte_perm(both, H_MAGIC, sel_a), cb[i] = __byte_perm(both, H_MAGIC, sel_b);
            }
        } else if constexpr (!PERM) {  // Q4_0 natural row
            const uint2 x = *(const uint2*)(raw + chunk_addr(FMT, D, KV, tok, 16 * (item / 2) + 8 * (item % 2)));
            const uint32_t l0 = (x.x >> sh_a) & 0x0f0f0f0fu, h0 = (x.x >> sh_b) & 0x0f0f0f0fu, l1 = (x.y >> sh_a) & 0x0f0f0f0fu, h1 = (x.y >> sh_b) & 0x0f0f0f0fu;
            ca[0] = __byte_perm(l0, H_MAGIC, 0x4140), ca[1] = __byte_perm(l0, H_MAGIC, 0x4342);
            ca[2] = __byte_perm(l1, H_MAGIC, 0x4140), ca[3] = __byte_perm(l1, H_MAGIC, 0x4342);
            cb[0] = __byte_perm(h0, H_MAGIC, 0x4140), cb[1] = __byte_perm(h0, H_MAGIC, 0x4342);
            cb[2] = __byte_perm(h1, H_MAGIC, 0x4140), cb[3] = __byte_perm(h1, H_MAGIC, 0x4342);
        } else {  // Q4_0 permuted V row: byte 8r + item holds channel 16 item + r (low nibble) and + 8 (high nibble)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t b0 = raw[chunk_addr(FMT, D, KV, tok, 8 * (2 * i) + item)], b1 = raw[chunk_addr(FMT, D, KV, tok, 8 * (2 * i + 1) + item)];
                const uint32_t both = b0 | (b1 << 16);
                ca[i] = ((both >> sh_a) & 0x000f000fu) | 0x64006400u, cb[i] = ((both >> sh_b) & 0x000f000fu) | 0x64006400u;
            }
        }
        const uint32_t sa16 = __half_as_ushort(scales[scale_index(FMT, D, KV, tok, blk_a)]);
        const uint32_t sb16 = __half_as_ushort(scales[scale_index(FMT, D, KV, tok, blk_b)]);
        const uint32_t sa = sa16 | (sa16 << 16), sb = sb16 | (sb16 << 16);
        uint32_t ha[4], hb[4], la[4], lb[4];
        const bool ok = FULL || tok < n_valid;  // a full page (all but, at most, the last) runs without the sixteen selects
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t xa = hsub2(ca[i], BIAS), xb = hsub2(cb[i], BIAS);  // the codes themselves
            ha[i] = ok ? hmul2(xa, sa) : 0u, hb[i] = ok ? hmul2(xb, sb) : 0u;
            if (SPLIT) la[i] = ok ? hfma2_rem(xa, sa, ha[i]) : 0u, lb[i] = ok ? hfma2_rem(xb, sb, hb[i]) : 0u;
        }
        *(uint4*)(hi_tile + tile_off(ua, tok)) = make_uint4(ha[0], ha[1], ha[2], ha[3]);
        *(uint4*)(hi_tile + tile_off(ub, tok)) = make_uint4(hb[0], hb[1], hb[2], hb[3]);
        if (SPLIT) {
            *(uint4*)(lo_tile + tile_off(ua, tok)) = make_uint4(la[0], la[1], la[2], la[3]);
            *(uint4*)(lo_tile + tile_off(ub, tok)) = make_uint4(lb[0], lb[1], lb[2], lb[3]);
        }
    }
}

template <int FMT, int D, int KV, int FT>
__device__ inline void convert_chunk(const uint8_t* raw, uint8_t* hi_tile, uint8_t* lo_tile, int n_valid, int t) {
    if (n_valid >= PAGE_TOKENS) convert_rows<FMT, D, KV, FT, true>(raw, hi_tile, lo_tile, n_valid, t);
    else convert_rows<FMT, D, KV, FT, false>(raw, hi_tile, lo_tile, n_valid, t);
}

template <int NQ, int D, int SRC, int FT>
__global__ void __launch_bounds__(AGeo<NQ, D, SRC, FT>::THREADS, 1) attn_tc_kernel(const __grid_constant__ AttnParams p) {
    using GEO = AGeo<NQ, D, SRC, FT>;
    constexpr int NK = GEO::NK, NV = GEO::NV, NR = GEO::NR, CHUNK = GEO::CHUNK, QBYTES = GEO::QBYTES, PLANES = GEO::PLANES;
    constexpr int KSTAGE = GEO::KSTAGE, KPARTS = GEO::KPARTS;
    constexpr bool RAW = GEO::RAW;  // converted sources: f16 operands whatever the query type
    constexpr uint32_t COL_O = 0, COL_S = GEO::COL_S, COLS_PER_TILE = GEO::COLS_PER_TILE;
    constexpr int FILL_ARRIVALS = SRC == SRC_PAGES16 ? 1 : FT / 32;
    static_assert(FT == A_FILL_THREADS || src_is_block(SRC) || src_is_kivi(SRC), "the dense loader and the copy warp have a fixed thread count");
    static_assert(!src_is_kivi(SRC) || D == 128, "the KIVI stores have their tensor-core layout at head_dim 128 only");
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* q_s = smem;                                    // [NQ][PLANES][128 rows][128 B], swizzled
    uint8_t* k_ring = smem + NQ * QBYTES;                   // NK K stages of KPARTS tiles
    uint8_t* v_ring = k_ring + NK * KSTAGE;                 // NV V tiles
    uint8_t* raw_ring = v_ring + NV * CHUNK;                // NR raw stages (converted sources)
    uint64_t* full_k = (uint64_t*)(raw_ring + NR * GEO::RAW_STAGE);  // [NK] the tile is complete
    uint64_t* full_v = full_k + NK;                         // [NV]
    uint64_t* free_k = full_v + NV;                         // [NK] every tile's Q.K^T on the stage has completed
    uint64_t* free_v = free_k + NK;                         // [NV] every tile's P.V on the stage has completed
    uint64_t* bar_s = free_v + NV;                          // [NQ][2] S buffer written
    uint64_t* bar_p = bar_s + 2 * NQ;                       // [NQ][2] P written by the softmax warps
    uint64_t* bar_o = bar_p + 2 * NQ;                       // [NQ][2] P.V of page j completed, on barrier j & 1
    uint64_t* full_raw = bar_o + 2 * NQ;                    // [NR] raw bytes landed
    uint64_t* free_raw = full_raw + NR;                     // [NR] every converter warp is done with the raw stage
    uint32_t* tmem_slot = (uint32_t*)(((uintptr_t)(free_raw + NR) + 15) & ~(uintptr_t)15);
    volatile int* fail_s = (volatile int*)(tmem_slot + 1);
    float* xchg = (float*)(tmem_slot + 4);                  // [NQ][2 parities][A_XCHG]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y, b = blockIdx.z;
    const int G = p.G, qpt = AM / G;                        // queries per tile
    const int cta_tile = (int)(gridDim.x - 1 - blockIdx.x);  // late queries see the most keys: schedule them first
    const int32_t trow = SRC == SRC_DENSE ? 0 : p.desc[2 * b], T = SRC == SRC_DENSE ? p.T : p.desc[2 * b + 1];
    const int P0 = T - p.S;                                 // keys before the first query's own position
    const int cta_q0 = cta_tile * NQ * qpt;
    const int cta_q_last = min(cta_q0 + NQ * qpt, p.S) - 1;
    // every tile of the CTA walks the pages up to the last key its last tile sees; a tile that ends earlier finds
    // its extra page fully masked
    const int n_tiles = (p.causal ? P0 + cta_q_last : T - 1) / PAGE_TOKENS + 1;

    if (tid == 0) {
        for (int s = 0; s < NK; s++) mbar_init(&full_k[s], FILL_ARRIVALS), mbar_init(&free_k[s], NQ);
        for (int s = 0; s < NV; s++) mbar_init(&full_v[s], FILL_ARRIVALS), mbar_init(&free_v[s], NQ);
        for (int i = 0; i < 2 * NQ; i++) mbar_init(&bar_s[i], 1), mbar_init(&bar_p[i], A_SM_THREADS / 32);
        for (int i = 0; i < 2 * NQ; i++) mbar_init(&bar_o[i], 1);
        for (int s = 0; s < NR; s++) mbar_init(&full_raw[s], 1), mbar_init(&free_raw[s], FT / 32);
        *fail_s = (smem_u32(smem) & 1023u) ? 1 : 0;  // the swizzled operand tiles need a 1024-byte aligned base
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, COLS_PER_TILE * NQ);

    // per-thread tile geometry (softmax threads only; the other warps get harmless values)
    const int qt = min(tid / A_SM_THREADS, NQ - 1), w4 = (tid % A_SM_THREADS) >> 5;
    const int row = w4 * 32 + lane;
    const int q0 = cta_q0 + qt * qpt;
    const int rq = row / G, rg = row % G;
    const bool live = rq < qpt && q0 + rq < p.S;
    const int q_last = max(min(q0 + qpt, p.S) - 1, 0);   // last live query of the tile (the tile may be all dead)
    const int my_q = live ? q0 + rq : min(q_last, p.S - 1);
    const int my_limit = p.causal ? P0 + my_q : T - 1;  // last visible key of this row
    const int min_limit = p.causal ? P0 + min(q0, p.S - 1) : T - 1;  // last key EVERY row of the tile sees
    const bool is_softmax = tid < NQ * A_SM_THREADS;
    const int mma_bf16 = RAW ? 0 : p.is_bf16;  // type of the tensor-core operands (Q, K, V, P)

    // ---- Q tile -> shared memory, K-major with the 128-byte swizzle (row r: 16-byte unit u of a plane at u ^ (r & 7));
    //      this thread moves its row ----
    if (is_softmax) {
        constexpr int NU = D / 8;  // 16-byte units per row
        const int head = kvh * G + rg;
        const uint4* src = (const uint4*)((const uint16_t*)p.q + (int64_t)b * p.qb + (int64_t)head * p.qh + (int64_t)my_q * p.qs);
#pragma unroll
        for (int uu = 0; uu < NU; uu++) {
            uint4 v = live ? src[uu] : make_uint4(0, 0, 0, 0);
            if (RAW && p.is_bf16) {  // bf16 queries over converted pages: every bf16 value is an f16 value (short of its range)
                uint32_t* w = &v.x;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const __half2 h = __floats2half2_rn(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xffff0000u));
                    w[e] = *(const uint32_t*)&h;
                }
            }
            const int plane = uu / 8, u8 = uu % 8;
            *(uint4*)(q_s + qt * QBYTES + plane * (AM * 128) + row * 128 + ((u8 ^ (row & 7)) << 4)) = v;
        }
        fence_async_proxy();  // generic-proxy writes -> visible to the tensor core
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (!is_softmax) {
        // Every lane of these warps walks its loop (the values stay warp-uniform); one elected lane issues.
        const int role = warp - NQ * (A_SM_THREADS / 32);  // 0 .. NQ - 1: MMAs of tile `role`; above: the copy warp, or the converter / loader warps
        if (role >= NQ && SRC == SRC_PAGES16) {
            // ================= page copies: the chunks of a 16-bit page are the operand tiles =================
            const int32_t* trow_p = p.table + (int64_t)trow * p.max_pages_per_seq;
            int32_t pg_next = trow_p[0];
            for (int i = 0; i < n_tiles; i++) {
                int32_t pg = pg_next;
                if (i + 1 < n_tiles) pg_next = trow_p[i + 1];  // fetched one page ahead of its use
                if (pg < 0 || pg >= p.n_pages) {
                    if (lane == 0) atomicOr(p.status, STATUS_PAGE_OOB);
                    pg = 0;
                }
                const uint8_t* src = p.pool + (int64_t)pg * p.page_bytes + (int64_t)kvh * (2 * p.chunk_bytes);
                if (i >= NK) wait_or_fail(&free_k[i % NK], (uint32_t)((i / NK - 1) & 1), fail_s);
                if (elect_one()) {
                    mbar_expect_tx(&full_k[i % NK], CHUNK);
                    bulk_g2s(k_ring + (i % NK) * CHUNK, src, CHUNK, &full_k[i % NK]);
                }
                __syncwarp();
                if (i >= NV) wait_or_fail(&free_v[i % NV], (uint32_t)((i / NV - 1) & 1), fail_s);
                if (elect_one()) {
                    mbar_expect_tx(&full_v[i % NV], CHUNK);
                    bulk_g2s(v_ring + (i % NV) * CHUNK, src + CHUNK, CHUNK, &full_v[i % NV]);
                }
                __syncwarp();
            }
        } else if (role < NQ) {
            // ================= MMAs of tile t = role =================
            const int t = role;
            const uint32_t tm = tmem + t * COLS_PER_TILE;
            const uint32_t idesc_s = instr_desc(mma_bf16, 0, AM, PAGE_TOKENS);
            const uint32_t idesc_o = instr_desc(mma_bf16, 1, AM, D);
            // descriptors of the ring bases; a byte offset inside the 256 KiB window adds offset / 16 to the address field
            const uint64_t q_desc = smem_desc(smem_u32(q_s) + t * QBYTES, 0, 1024);
            const uint64_t k_desc = smem_desc(smem_u32(k_ring), 0, 1024);
            // V tile: planes of 64 channels 8192 bytes apart (leading dimension), 8-key groups 1024 bytes apart
            const uint64_t v_desc = smem_desc(smem_u32(v_ring), PAGE_TOKENS * 128, 1024);
            const bool adaptive = !mma_bf16;
            auto issue_qk = [&](int j) {  // S(j) = Q . K(j)^T into buffer j & 1
                wait_or_fail(&full_k[j % NK], (uint32_t)((j / NK) & 1), fail_s);
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t kd = k_desc + (uint64_t)(((j % NK) * KSTAGE) >> 4);
#pragma unroll
                    for (int pl = 0; pl < PLANES; pl++)
#pragma unroll
                        for (int kk = 0; kk < 4; kk++) {
                            const uint64_t off = (uint64_t)((pl * (AM * 128) + kk * 32) >> 4);
                            const uint64_t koff = (uint64_t)((pl * (PAGE_TOKENS * 128) + kk * 32) >> 4);
                            if constexpr (KPARTS == 2) {
                                // K as value + remainder: the two products of a k-step land in the same S and share their Q
                                // slice, which the second takes from the collector buffer instead of shared memory
                                tc_mma_ss_a<A_KEEP>(tm + COL_S + 64 * (j & 1), q_desc + off, kd + koff, idesc_s, (pl | kk) ? 1u : 0u);
                                tc_mma_ss_a<A_REUSE_LAST>(tm + COL_S + 64 * (j & 1), q_desc + off, kd + (uint64_t)(CHUNK >> 4) + koff, idesc_s, 1u);
                            } else {
                                tc_mma_ss(tm + COL_S + 64 * (j & 1), q_desc + off, kd + koff, idesc_s, (pl | kk) ? 1u : 0u);
                            }
                        }
                    tc_commit(&bar_s[2 * t + (j & 1)]);
                    tc_commit(&free_k[j % NK]);
                }
                __syncwarp();
            };
            issue_qk(0);
            if (n_tiles > 1) issue_qk(1);
            for (int j = 0; j < n_tiles; j++) {
                // O += P(j) . V(j): 4 steps of 16 keys; the V tile is an MN-major operand
                wait_or_fail(&full_v[j % NV], (uint32_t)((j / NV) & 1), fail_s);
                wait_or_fail(&bar_p[2 * t + (j & 1)], (uint32_t)((j >> 1) & 1), fail_s);
                tc_fence_after();
                const int* flags = (const int*)(xchg + (2 * t + (j & 1)) * A_XCHG);
                const bool two = !adaptive || __any_sync(0xffffffffu, flags[lane & 3] != 0);
                if (elect_one()) {
                    const uint64_t vd = v_desc + (uint64_t)(((j % NV) * CHUNK) >> 4);
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
                // S(j + 2) reuses the buffer P(j) sits in: the tensor core runs one thread's MMAs in issue order
                if (j + 2 < n_tiles) issue_qk(j + 2);
            }
        } else {
            // ================= converter / loader warps: fill the operand rings =================
            const int ft = tid - (NQ * A_SM_THREADS + 32 * NQ);  // 0 .. FT - 1 (converters) or 0 .. 63 (loaders)
            if constexpr (src_is_block(SRC)) {
                constexpr int FMT = SRC == SRC_Q8 ? B200KV_FMT_Q8_1 : B200KV_FMT_Q4_0;
                const bool requester = ft < 32;  // the first converter warp also requests the raw pages
                const int32_t* trow_p = p.table + (int64_t)trow * p.max_pages_per_seq;
                auto request = [&](int i, int32_t pg) {  // raw chunk pair of page i into stage i % NR
                    if (pg < 0 || pg >= p.n_pages) {
                        if (lane == 0) atomicOr(p.status, STATUS_PAGE_OOB);
                        pg = 0;
                    }
                    if (elect_one()) {
                        const uint8_t* src = p.pool + (int64_t)pg * p.page_bytes + (int64_t)kvh * (2 * p.chunk_bytes);
                        mbar_expect_tx(&full_raw[i % NR], 2 * p.chunk_bytes);
                        bulk_g2s(raw_ring + (i % NR) * GEO::RAW_STAGE, src, 2 * p.chunk_bytes, &full_raw[i % NR]);
                    }
                    __syncwarp();
                };
                int32_t pg_next = 0;
                if (requester) {
                    for (int i = 0; i < NR && i < n_tiles; i++) request(i, trow_p[i]);
                    if (NR < n_tiles) pg_next = trow_p[NR];
                }
                for (int i = 0; i < n_tiles; i++) {
                    const uint8_t* raw = raw_ring + (i % NR) * GEO::RAW_STAGE;
                    const int n_valid = min(PAGE_TOKENS, T - i * PAGE_TOKENS);
                    wait_or_fail(&full_raw[i % NR], (uint32_t)((i / NR) & 1), fail_s);
                    if (i >= NK) wait_or_fail(&free_k[i % NK], (uint32_t)((i / NK - 1) & 1), fail_s);
                    convert_chunk<FMT, D, 0, FT>(raw, k_ring + (i % NK) * KSTAGE, k_ring + (i % NK) * KSTAGE + CHUNK, n_valid, ft);
                    fence_async_proxy();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full_k[i % NK]);
                    if (i >= NV) wait_or_fail(&free_v[i % NV], (uint32_t)((i / NV - 1) & 1), fail_s);
                    convert_chunk<FMT, D, 1, FT>(raw + p.chunk_bytes, v_ring + (i % NV) * CHUNK, nullptr, n_valid, ft);
                    fence_async_proxy();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full_v[i % NV]), mbar_arrive(&free_raw[i % NR]);
                    if (requester && i + NR < n_tiles) {  // the stage is free once the other converter warps have left it too
                        wait_or_fail(&free_raw[i % NR], (uint32_t)((i / NR) & 1), fail_s);
                        request(i + NR, pg_next);
                        if (i + NR + 1 < n_tiles) pg_next = trow_p[i + NR + 1];
                    }
                }
            } else if constexpr (src_is_kivi(SRC)) {
                constexpr int BITS = SRC == SRC_KIVI8 ? 8 : 4;
                const KiviView& kw = p.kv;
                const int32_t seq = trow;
                const int KC = PAGE_TOKENS * kw.row_bytes;          // bytes of the K (or V) codes of a page and head
                constexpr int lfmt = kivi_layout_fmt(BITS);         // the block format whose row layout the codes borrow
                constexpr bool int4 = BITS == 4;
                const int n_fin = max(T - SINK, 0) / KBLOCK;        // finalised key blocks
                const int n_sp = T > SINK ? (T - SINK + PAGE_TOKENS - 1) / PAGE_TOKENS : 0;  // storage pages the sequence holds
                const int n_need = min(n_sp, n_tiles);              // tile j reads page j (and, through the carry, page j - 1)
                uint8_t* carry = (uint8_t*)(xchg + NQ * 2 * A_XCHG);  // [K, V][4 rows][256 B]
                const bool requester = ft < 32;
                const int32_t* trow_p = kw.table + (int64_t)seq * kw.max_pages_per_seq;
                auto request = [&](int i, int32_t pg) {  // the four arrays of storage page i into raw stage i % NR
                    if (pg < 0 || pg >= kw.n_pages) {
                        if (lane == 0) atomicOr(p.status, STATUS_PAGE_OOB);
                        pg = 0;
                    }
                    if (elect_one()) {
                        const int64_t ph = (int64_t)pg * kw.H + kvh;
                        uint8_t* dst = raw_ring + (i % NR) * GEO::RAW_STAGE;
                        mbar_expect_tx(&full_raw[i % NR], 2 * KC + A_KIVI_KP + A_KIVI_VP);
                        bulk_g2s(dst, kw.codes[0] + ph * KC, KC, &full_raw[i % NR]);
                        bulk_g2s(dst + KC, kw.codes[1] + ph * KC, KC, &full_raw[i % NR]);
                        bulk_g2s(dst + 2 * KC, kw.params[0] + ph * (A_KIVI_KP / 4), A_KIVI_KP, &full_raw[i % NR]);
                        bulk_g2s(dst + 2 * KC + A_KIVI_KP, kw.params[1] + ph * (A_KIVI_VP / 4), A_KIVI_VP, &full_raw[i % NR]);
                    }
                    __syncwarp();
                };
                int32_t pg_next = 0;
                if (requester) {
                    for (int i = 0; i < NR && i < n_need; i++) request(i, trow_p[i]);
                    if (NR < n_need) pg_next = trow_p[NR];
                }
                constexpr int TLK = FT / 16;                          // token lanes
                const int u = ft % 16, tl = ft / 16, ch0 = 8 * u;   // this thread's 8 channels; token lane 0 .. TLK - 1
                const bool heads_row = tl < SINK;                    // the first 64 threads also place rows 0 .. 3 of a tile
                const int kpos0 = int4 ? (ch0 / 32) * 16 + ch0 % 16 : ch0, knib = int4 ? (ch0 % 32) / 16 : 0;
                int vpos[8];
#pragma unroll
                for (int e = 0; e < 8; e++) vpos[e] = code_pos(lfmt, 128, 1, ch0 + e);
                const int vnib = code_nibble(lfmt, 128, 1, ch0);
                const float* sink_base = kw.sinks + (((int64_t)seq * kw.H + kvh) * 2) * SINK * D;
                const float* resid = kw.residual + (((int64_t)seq * kw.H + kvh) * 2 + 0) * KBLOCK * D;
                // 8 f32 values -> their f16 roundings and (K) the f16 roundings of what that lost
                auto pack8 = [&](const float* f, uint4& hi, uint4& lo) {
                    uint32_t wh[4], wl[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const __half2 h = __floats2half2_rn(f[2 * e], f[2 * e + 1]);
                        const __half2 l = __floats2half2_rn(f[2 * e] - __low2float(h), f[2 * e + 1] - __high2float(h));
                        wh[e] = *(const uint32_t*)&h, wl[e] = *(const uint32_t*)&l;
                    }
                    hi = make_uint4(wh[0], wh[1], wh[2], wh[3]), lo = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                };
                auto pack8_hi = [&](const float* f, uint4& hi) {  // values only (V tolerates the rounding)
                    uint32_t wh[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const __half2 h = __floats2half2_rn(f[2 * e], f[2 * e + 1]);
                        wh[e] = *(const uint32_t*)&h;
                    }
                    hi = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                };
                auto tile_addr = [&](uint8_t* base, int row) { return base + tile_off(u, row); };
                uint8_t* carry_lo = carry + A_CARRY;  // the remainders of the carried K rows
                for (int j = 0; j < n_tiles; j++) {
                    const bool has_page = j < n_sp;
                    const uint8_t* raw = raw_ring + (j % NR) * GEO::RAW_STAGE;
                    if (has_page) wait_or_fail(&full_raw[j % NR], (uint32_t)((j / NR) & 1), fail_s);
                    // rows 0 .. 3 of the tile: the sinks (tile 0) or the last four slots of the page before; thread ft takes
                    // unit u of row ft / 16 for K and for V
                    uint4 head[2], head_lo = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                    for (int st = 0; st < 2; st++) {
                        head[st] = make_uint4(0u, 0u, 0u, 0u);
                        if (heads_row && j * PAGE_TOKENS + tl < T) {
                            uint4 lo4 = make_uint4(0u, 0u, 0u, 0u);
                            if (j == 0) {
                                const float4* src = (const float4*)(sink_base + ((int64_t)st * SINK + tl) * D + ch0);
                                const float4 a = src[0], b2 = src[1];
                                const float f[8] = {a.x, a.y, a.z, a.w, b2.x, b2.y, b2.z, b2.w};
                                pack8(f, head[st], lo4);
                            } else {
                                head[st] = *(const uint4*)(carry + ((st * SINK + tl) * 16 + u) * 16);
                                if (st == 0) lo4 = *(const uint4*)(carry_lo + (tl * 16 + u) * 16);
                            }
                            if (st == 0) head_lo = lo4;
                        }
                    }
                    asm volatile("bar.sync 9, %0;" ::"n"(FT) : "memory");  // every converter warp has read the carry: it may be rewritten
                    auto fill = [&](auto st_c) {  // K (0), then V (1): one body, specialised at compile time
                        constexpr int st = decltype(st_c)::value;
                        uint8_t* dst;
                        if (st == 0) {
                            if (j >= NK) wait_or_fail(&free_k[j % NK], (uint32_t)((j / NK - 1) & 1), fail_s);
                            dst = k_ring + (j % NK) * KSTAGE;
                            if (heads_row) *(uint4*)tile_addr(dst + CHUNK, tl) = head_lo;
                        } else {
                            if (j >= NV) wait_or_fail(&free_v[j % NV], (uint32_t)((j / NV - 1) & 1), fail_s);
                            dst = v_ring + (j % NV) * CHUNK;
                        }
                        if (heads_row) *(uint4*)tile_addr(dst, tl) = head[st];
                        const uint8_t* codes = raw + st * KC;
                        const float* kpar = (const float*)(raw + 2 * KC);
                        const float2* vpar = (const float2*)(raw + 2 * KC + A_KIVI_KP);
#pragma unroll 2
                        for (int tt = 0; tt < PAGE_TOKENS / TLK; tt++) {
                            const int s = tt * TLK + tl;                // slot in storage page j
                            const int i = j * PAGE_TOKENS + s;          // storage index; key i + 4
                            float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                            if (has_page && i + SINK < T) {
                                if (st == 0 && i >= n_fin * KBLOCK) {  // the partial key block: f32 rows, verbatim
                                    const float4* src = (const float4*)(resid + (int64_t)(i % KBLOCK) * D + ch0);
                                    const float4 a = src[0], b2 = src[1];
                                    f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b2.x, f[5] = b2.y, f[6] = b2.z, f[7] = b2.w;
                                } else {
                                    uint32_t cb[8];  // the byte that holds each channel's code
                                    if (st == 0) {
                                        const uint2 x = *(const uint2*)(codes + chunk_addr(lfmt, 128, 0, s, kpos0));
#pragma unroll
                                        for (int e = 0; e < 4; e++) cb[e] = __byte_perm(x.x, 0u, 0x4440 + e), cb[4 + e] = __byte_perm(x.y, 0u, 0x4440 + e);
                                    } else {
#pragma unroll
                                        for (int e = 0; e < 8; e++) cb[e] = codes[chunk_addr(lfmt, 128, 1, s, vpos[e])];
                                    }
                                    const int nib = st == 0 ? knib : vnib;
                                    if (st == 0) {  // per channel: (lo, scale) of the slot's 32-token block
                                        const float* par = kpar + (s / KBLOCK) * 2 * D + ch0;
#pragma unroll
                                        for (int e = 0; e < 8; e++) {
                                            const uint32_t code = int4 ? (cb[e] >> (4 * nib)) & 0xfu : cb[e];
                                            f[e] = kivi_dequant(code, par[e], par[D + e]);
                                        }
                                    } else {        // per token
                                        const float2 ls = vpar[s];
#pragma unroll
                                        for (int e = 0; e < 8; e++) {
                                            const uint32_t code = int4 ? (cb[e] >> (4 * nib)) & 0xfu : cb[e];
                                            f[e] = kivi_dequant(code, ls.x, ls.y);
                                        }
                                    }
                                }
                            }
                            uint4 w, wl = make_uint4(0u, 0u, 0u, 0u);
                            if (st == 0) pack8(f, w, wl);
                            else pack8_hi(f, w);
                            if (s < PAGE_TOKENS - SINK) {
                                *(uint4*)tile_addr(dst, s + SINK) = w;
                                if (st == 0) *(uint4*)tile_addr(dst + CHUNK, s + SINK) = wl;
                            } else {
                                *(uint4*)(carry + ((st * SINK + (s - (PAGE_TOKENS - SINK))) * 16 + u) * 16) = w;
                                if (st == 0) *(uint4*)(carry_lo + ((s - (PAGE_TOKENS - SINK)) * 16 + u) * 16) = wl;
                            }
                        }
                        fence_async_proxy();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(st == 0 ? &full_k[j % NK] : &full_v[j % NV]);
                    };
                    fill(std::integral_constant<int, 0>{});
                    fill(std::integral_constant<int, 1>{});
                    asm volatile("bar.sync 9, %0;" ::"n"(FT) : "memory");  // the new carry is complete before the next tile reads it
                    if (has_page) {
                        if (lane == 0) mbar_arrive(&free_raw[j % NR]);
                        if (requester && j + NR < n_need) {
                            wait_or_fail(&free_raw[j % NR], (uint32_t)((j / NR) & 1), fail_s);
                            request(j + NR, pg_next);
                            if (j + NR + 1 < n_need) pg_next = trow_p[j + NR + 1];
                        }
                    }
                }
            } else if constexpr (SRC == SRC_DENSE) {
                constexpr int LAG = 2;            // pages in flight behind the one being requested
                constexpr int UROW = D / 8;       // 16-byte units per row
                constexpr int PER_THREAD = PAGE_TOKENS * UROW / A_FILL_THREADS;
                const uint16_t* kbase = (const uint16_t*)p.k + (int64_t)b * p.kb + (int64_t)kvh * p.kh;
                const uint16_t* vbase = (const uint16_t*)p.v + (int64_t)b * p.vb + (int64_t)kvh * p.vh;
                for (int i = 0; i < n_tiles + LAG; i++) {
                    // Announce page i - LAG before waiting for room for page i: the products that free a stage are issued
                    // behind products that need the pages still to be announced, so the other order can wait for ever.
                    if (i >= LAG) {
                        cp_async_wait_group<LAG - 1>();  // all but the LAG - 1 newest groups: page i - LAG has landed
                        fence_async_proxy();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&full_k[(i - LAG) % NK]), mbar_arrive(&full_v[(i - LAG) % NV]);
                    }
                    if (i < n_tiles) {
                        if (i >= NK) wait_or_fail(&free_k[i % NK], (uint32_t)((i / NK - 1) & 1), fail_s);
                        if (i >= NV) wait_or_fail(&free_v[i % NV], (uint32_t)((i / NV - 1) & 1), fail_s);
                        uint8_t* kd = k_ring + (i % NK) * KSTAGE;
                        uint8_t* vd = v_ring + (i % NV) * CHUNK;
#pragma unroll
                        for (int e = 0; e < PER_THREAD; e++) {
                            const int x = e * A_FILL_THREADS + ft, r = x / UROW, u = x % UROW;
                            const int key = i * PAGE_TOKENS + r;
                            const bool ok = key < T;
                            const int64_t kr = ok ? key : 0;
                            const int off = tile_off(u, r);
                            cp_async16_zfill(kd + off, kbase + kr * p.ks + u * 8, ok);
                            cp_async16_zfill(vd + off, vbase + kr * p.vs + u * 8, ok);
                        }
                    }
                    cp_async_commit_group();
                }
                cp_async_wait_group<0>();
            }
        }
    } else {
        // ================= softmax threads =================
        const uint32_t lane_base = tmem + qt * COLS_PER_TILE + ((uint32_t)(w4 * 32) << 16);  // this warp's lane quarter
        const bool adaptive = !mma_bf16;
        const float sl2 = p.scale * 1.4426950408889634f;  // scores enter the exponent in log2 units
        float m_ref = -INFINITY, l_run = 0.f, log_thresh = -INFINITY;
        // this row's mask values (dense source): element (my_q, key) at mrow + key * mk
        const bool masked = SRC == SRC_DENSE && p.mask != nullptr;
        const int64_t mrow = masked ? (int64_t)b * p.mb + (int64_t)(kvh * G + rg) * p.mh + (int64_t)my_q * p.mq : 0;

        for (int j = 0; j < n_tiles; j++) {
            const uint32_t sbuf = lane_base + COL_S + 64 * (j & 1);
            wait_or_fail(&bar_s[2 * qt + (j & 1)], (uint32_t)((j >> 1) & 1), fail_s);
            tc_fence_after();
            // ---- the row's 64 scores ----
            uint32_t sr[64];
            tmem_ld32(sbuf, sr);
            tmem_ld32(sbuf + 32, sr + 32);
            tmem_ld_wait();
            const int t0 = j * PAGE_TOKENS;
            if (masked) {  // the mask is added to the scaled score: the raw score takes mask / scale
#pragma unroll
                for (int c = 0; c < 64; c++) {
                    float sc = -INFINITY;
                    if (t0 + c <= my_limit) sc = fmaf(ld_as_f32(p.mask, p.mask_dtype, mrow + (int64_t)(t0 + c) * p.mk), p.inv_scale, __uint_as_float(sr[c]));
                    sr[c] = __float_as_uint(sc);
                }
            } else if (t0 + PAGE_TOKENS - 1 > min_limit) {  // only pages on the causal diagonal / past the end need a mask
#pragma unroll
                for (int c = 0; c < 64; c++)
                    if (t0 + c > my_limit) sr[c] = 0xff800000u;  // -inf
            }
            const float tmax = row_max64(sr) * sl2;
            int* flags = (int*)(xchg + (2 * qt + (j & 1)) * A_XCHG);
            // Two questions per row, answered for the warp with one reduction.  Bit 0: f16 weights skip the remainder product of
            // a page once, for every row of the tile, what the rounding of the page can add is below 2^-12 / 8 of the row's scale
            // (sqrt(64) x the largest weight against skip_fraction x the running sum, compared in the log domain; page 0 always
            // keeps it).  Bit 1: is the reference maximum exceeded by more than 2^8 -- it is raised only then (and set by the
            // first page that shows the row a key), so the exponentials stay below 256, exact enough in 16 bits, and O is
            // rescaled rarely.
            const bool mine = adaptive && (j == 0 || !(tmax - m_ref + 3.f <= log_thresh));
            const bool raise = tmax > m_ref + 8.f || (m_ref == -INFINITY && tmax > -INFINITY);
            const uint32_t votes = __reduce_or_sync(0xffffffffu, (mine ? 1u : 0u) | (raise && j > 0 ? 2u : 0u));
            const bool two = !adaptive || (votes & 1u);
            if (adaptive && lane == 0) flags[w4] = two ? 1 : 0;  // the MMA warp issues the remainder product if any warp asks for it
            float alpha = 1.f;
            if (raise) {
                alpha = fast_exp2(m_ref - tmax);  // m_ref = -inf (every key so far masked out): 0
                m_ref = tmax;
                l_run *= alpha;
            }
            if (votes & 2u) {
                // O must hold every page before this one: see prefill_tc.cu for why the wait on barrier (j - 1) & 1 cannot
                // mistake the completion of P.V(j - 3) or P.V(j + 1) for that of P.V(j - 1)
                wait_or_fail(&bar_o[2 * qt + ((j - 1) & 1)], (uint32_t)(((j - 1) >> 1) & 1), fail_s);
                tc_fence_after();
#pragma unroll
                for (int cc = 0; cc < D / 16; cc++) {  // the row's output channels
                    uint32_t orow[16];
                    tmem_ld16(lane_base + COL_O + cc * 16, orow);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 16; c++) orow[c] = __float_as_uint(__uint_as_float(orow[c]) * alpha);
                    tmem_st16(lane_base + COL_O + cc * 16, orow);
                }
            }
            // a row that has seen no key yet has m_ref = -inf: its weights are exp2(-inf - 0) = 0, not exp2(-inf + inf)
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            uint32_t pr[32], pr2[32];
            float page_sum;
            if (mma_bf16) page_sum = softmax_exps<2>(sr, sl2, m_use, pr, pr2);
            else if (two) page_sum = softmax_exps<1>(sr, sl2, m_use, pr, pr2);
            else page_sum = softmax_exps<0>(sr, sl2, m_use, pr, pr2);
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
        wait_or_fail(&bar_o[2 * qt + ((n_tiles - 1) & 1)], (uint32_t)(((n_tiles - 1) >> 1) & 1), fail_s);
        tc_fence_after();
        if (!*fail_s) {
            const float inv = 1.f / l_run;  // no visible key: 0 * inf = NaN, as 0 / 0 in the reference
            uint16_t* dst = (uint16_t*)p.out + (int64_t)b * p.ob + (int64_t)(kvh * G + rg) * p.oh + (int64_t)my_q * p.os;
#pragma unroll
            for (int cc = 0; cc < D / 32; cc++) {
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
                                const __nv_bfloat162 h = __floats2bfloat162_rn(a, bb);
                                w[e] = *(const uint32_t*)&h;
                            } else {
                                const __half2 h = __floats2half2_rn(a, bb);
                                w[e] = *(const uint32_t*)&h;
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

// ---- host side ------------------------------------------------------------------------------------------

static bool aligned16(const void* ptr, const int64_t* st, int n) {
    if ((uintptr_t)ptr % 16) return false;
    for (int i = 0; i < n; i++)
        if ((st[i] * 2) % 16) return false;
    return true;
}

template <int NQ, int D, int SRC, int FT = A_FILL_THREADS>
static cudaError_t launch_attn(const AttnParams& p, int n_batch, cudaStream_t stream) {
    using GEO = AGeo<NQ, D, SRC, FT>;
    static_assert(GEO::SMEM <= 227 * 1024, "the operand rings do not fit the shared memory of an SM");
    cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel<NQ, D, SRC, FT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEO::SMEM);
    if (e != cudaSuccess) return e;
    const int per_cta = NQ * (AM / p.G);
    dim3 grid((p.S + per_cta - 1) / per_cta, p.Hkv, n_batch);
    attn_tc_kernel<NQ, D, SRC, FT><<<grid, GEO::THREADS, GEO::SMEM, stream>>>(p);
    return cudaGetLastError();
}

template <int D, int SRC>
static cudaError_t launch_attn_nq(const AttnParams& p, int n_batch, cudaStream_t stream) {
    // double tiles (K / V staged once for 2 x 128 rows) when they still fill the GPU
    const int qpt = AM / p.G;
    const int64_t double_ctas = (int64_t)((p.S + 2 * qpt - 1) / (2 * qpt)) * p.Hkv * n_batch;
    // converted sources: four converter warps (measured on 8 x 512 queries after 7680 int8 tokens: 1.32 ms with two, 1.02 ms
    // with four; the softmax threads then work with 80 registers instead of 96)
    if constexpr (src_is_block(SRC) || src_is_kivi(SRC))
        return double_ctas >= 148 ? launch_attn<2, D, SRC, 128>(p, n_batch, stream) : launch_attn<1, D, SRC, 128>(p, n_batch, stream);
    else
    return double_ctas >= 148 /* SMs of a B200 */ ? launch_attn<2, D, SRC>(p, n_batch, stream) : launch_attn<1, D, SRC>(p, n_batch, stream);
}

// Several queries per sequence over a paged cache: which caches this kernel reads (the f16 / bf16 head_dim-128 caches
// have the kernel of prefill_tc.cu).
bool attn_tc_supported(const b200kv_cache* c, int n_q_heads, int dtype, const void* q, const int64_t* qs, const void* out, const int64_t* os) {
    const int fmt = c->L.fmt, D = c->L.D;
    if (D != 64 && D != 128) return false;
    if (dtype != B200KV_F16 && dtype != B200KV_BF16) return false;
    const bool pages16 = (fmt == B200KV_FMT_F16 && dtype == B200KV_F16) || (fmt == B200KV_FMT_BF16 && dtype == B200KV_BF16);
    const bool kivi = fmt_is_kivi(fmt) && D == 128 && c->L.has_v;
    if (!(pages16 && D == 64) && !fmt_is_block_quant(fmt) && !kivi) return false;
    const int G = n_q_heads / c->L.Hkv;
    if (G < 1 || G > AM) return false;
    return aligned16(q, qs, 3) && aligned16(out, os, 3);
}

int launch_attn_tc_paged(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, int32_t n_new, const void* q, const int64_t* qs,
                         void* out, const int64_t* os, int32_t dtype, float scale, int causal, cudaStream_t stream) {
    int slot;
    uint8_t *h, *d;
    if (staging_acquire(c, (size_t)n_seqs * 8, &slot, &h, &d) != B200KV_OK) return B200KV_KO;
    int32_t* hw = (int32_t*)h;
    for (int i = 0; i < n_seqs; i++) hw[2 * i] = seqs[i], hw[2 * i + 1] = (int32_t)c->seqs[seqs[i]].len;
    if (staging_upload(c, slot, (size_t)n_seqs * 8, stream) != B200KV_OK) {
        staging_release(c, slot, stream);
        return B200KV_KO;
    }
    AttnParams p{};
    p.q = q, p.out = out, p.qb = qs[0], p.qh = qs[1], p.qs = qs[2], p.ob = os[0], p.oh = os[1], p.os = os[2];
    p.status = c->d_status;
    p.Hkv = c->L.Hkv, p.G = n_q_heads / c->L.Hkv, p.S = n_new, p.causal = causal, p.is_bf16 = dtype == B200KV_BF16;
    p.scale = scale, p.inv_scale = 1.f / scale, p.skip_fraction = A_SKIP_FRACTION;
    p.pool = c->pool, p.table = c->d_table, p.desc = (const int32_t*)d, p.page_bytes = c->L.page_bytes;
    p.n_pages = (int32_t)c->n_pages, p.max_pages_per_seq = c->max_pages_per_seq, p.fmt = c->L.fmt, p.chunk_bytes = c->L.chunk_bytes;
    cudaError_t e;
    {
        ProfScope ps(c, K_PREFILL, stream);
        if (fmt_is_kivi(c->L.fmt)) {
            p.kv = kivi_view(c);
            e = c->L.fmt == B200KV_FMT_KIVI8 ? launch_attn_nq<128, SRC_KIVI8>(p, n_seqs, stream) : launch_attn_nq<128, SRC_KIVI4>(p, n_seqs, stream);
        } else if (c->L.fmt == B200KV_FMT_Q8_1)
            e = c->L.D == 128 ? launch_attn_nq<128, SRC_Q8>(p, n_seqs, stream) : launch_attn_nq<64, SRC_Q8>(p, n_seqs, stream);
        else if (c->L.fmt == B200KV_FMT_Q4_0)
            e = c->L.D == 128 ? launch_attn_nq<128, SRC_Q4>(p, n_seqs, stream) : launch_attn_nq<64, SRC_Q4>(p, n_seqs, stream);
        else
            e = launch_attn_nq<64, SRC_PAGES16>(p, n_seqs, stream);
    }
    staging_release(c, slot, stream);
    if (e != cudaSuccess) return fail("attention launch failed: %s", cudaGetErrorString(e));
    return B200KV_OK;
}

// The lone Sdpa on dense tensors: 0 when this kernel cannot take the call (the caller then runs the generic kernel).
bool attn_tc_dense_supported(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v, const int64_t* vs,
                             const void* mask, int mask_dtype, const void* out, const int64_t* os, int B, int Hq, int Hkv, int S, int T, int D,
                             int dtype, int causal) {
    if (D != 64 && D != 128) return false;
    if (dtype != B200KV_F16 && dtype != B200KV_BF16) return false;
    if (B <= 0 || S <= 0 || T <= 0 || B > 65535 || Hkv > 65535) return false;
    if (causal && T < S) return false;  // queries that see no key at all: left to the generic kernel
    if (mask && (mask_dtype < B200KV_F32 || mask_dtype > B200KV_BF16)) return false;
    const int G = Hq / Hkv;
    if (G < 1 || G > AM) return false;
    return aligned16(q, qs, 3) && aligned16(out, os, 3) && aligned16(k, ks, 3) && aligned16(v, vs, 3);
}

int launch_attn_tc_dense(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v, const int64_t* vs, const void* mask,
                         const int64_t* ms, int mask_dtype, void* out, const int64_t* os, int B, int Hq, int Hkv, int S, int T, int D, int dtype,
                         float scale, int causal, int* status, cudaStream_t stream) {
    AttnParams p{};
    p.q = q, p.out = out, p.qb = qs[0], p.qh = qs[1], p.qs = qs[2], p.ob = os[0], p.oh = os[1], p.os = os[2];
    p.status = status;
    p.Hkv = Hkv, p.G = Hq / Hkv, p.S = S, p.causal = causal, p.is_bf16 = dtype == B200KV_BF16;
    p.scale = scale, p.inv_scale = 1.f / scale, p.skip_fraction = A_SKIP_FRACTION;
    p.k = k, p.v = v, p.kb = ks[0], p.kh = ks[1], p.ks = ks[2], p.vb = vs[0], p.vh = vs[1], p.vs = vs[2], p.T = T;
    if (mask) p.mask = mask, p.mb = ms[0], p.mh = ms[1], p.mq = ms[2], p.mk = ms[3], p.mask_dtype = mask_dtype;
    const cudaError_t e = D == 128 ? launch_attn_nq<128, SRC_DENSE>(p, B, stream) : launch_attn_nq<64, SRC_DENSE>(p, B, stream);
    if (e != cudaSuccess) return fail("attention launch failed: %s", cudaGetErrorString(e));
    return B200KV_OK;
}

}  // namespace b200kv
