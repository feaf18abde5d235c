// Split-KV GQA decode attention over the paged cache (one new query per sequence), and the
// second pass that combines the split partials.
//
// Replaces the decode use of cuda/src/kernels/cu/flash_attn.cu (`attention_tailq_*`: one CTA per
// (batch, q-head), 1 of 64 MMA rows useful, every q-head of a GQA group re-streams the same K/V,
// no split along the sequence).  Here one CTA owns a run of pages of one (sequence, kv head) for
// ALL q-heads of the group, page chunks arrive by untiled bulk copies (cp.async.bulk) into a
// shared-memory ring guarded by mbarriers, quantised pages are dequantised in registers, and the
// softmax is reduced with warp shuffles.  Semantics: transformers/src/ops/flash_sdpa.rs:239-341
// with S = 1 (causal masking is vacuous for the last position).
#include <algorithm>
#include <cmath>
#include <vector>

#include "decode_common.h"
#include "q40_common.cuh"

namespace b200kv {

template <int FMT, int D>
struct Geo {
    static constexpr int ROW = FMT == B200KV_FMT_F32 ? D * 4
                             : (FMT == B200KV_FMT_F16 || FMT == B200KV_FMT_BF16) ? D * 2
                             : FMT == B200KV_FMT_Q8_1 ? D
                                                      : D / 2;
    static constexpr bool QUANT = FMT == B200KV_FMT_Q8_1 || FMT == B200KV_FMT_Q4_0;
    static constexpr int PW = ROW < 128 ? ROW : 128;
    static constexpr int DATA = PAGE_TOKENS * ROW;
    static constexpr int SCALES = QUANT ? PAGE_TOKENS * (D / 32) * 2 : 0;
    static constexpr int CHUNK = DATA + SCALES;
    static constexpr int STAGE = 2 * CHUNK;  // K chunk then V chunk, adjacent in the page
    static constexpr int NS_RAW = 98304 / STAGE;
    static constexpr int NS = NS_RAW < 2 ? 2 : (NS_RAW > 4 ? 4 : NS_RAW);
    // score phase: 8 lanes share a token, each reads LB bytes of its row in pieces of PB bytes
    static constexpr int LB = ROW / 8;
    static constexpr int PB = LB < 16 ? LB : 16;
    static constexpr int NPC = LB / PB;
    static constexpr int EPP = elems_in_bytes<FMT>(PB);
    static constexpr int EPL = NPC * EPP;  // = D / 8 channels per lane
    // value phase: 16 threads share a token
    static constexpr int TB = ROW / 16;
    static constexpr int PB2 = TB < 16 ? TB : 16;
    static constexpr int NPC2 = TB / PB2;
    static constexpr int EPP2 = elems_in_bytes<FMT>(PB2);
    static constexpr int CPT = NPC2 * EPP2;  // = D / 16 channels per thread
};

template <int GT>
__host__ __device__ constexpr size_t decode_tail_bytes() {
    // scores [GT][64] + probabilities [64][GT] + alpha [GT] + (m, l) [GT][2] + barriers
    return (size_t)(GT * 64 + 64 * GT + GT + 2 * GT) * 4 + 16 + 4 * 8;
}

__device__ inline float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ inline float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int FMT, int D, int GT>
__global__ void __launch_bounds__(128) decode_kernel(DecodeParams p, const __grid_constant__ InlineBatch ib) {
    using Gm = Geo<FMT, D>;
    const bool PRECISE = p.dtype == B200KV_F32;  // f32 callers get expf, 16-bit callers the fast exponential
    constexpr int NS = Gm::NS;
    // declared aligned (not rounded up by hand) so that the compiler keeps every access in the shared window
    extern __shared__ __align__(1024) uint8_t stages[];
    float* sc = (float*)(stages + (size_t)NS * Gm::STAGE);  // [GT][64]
    float* pT = sc + GT * 64;                                // [64][GT]
    float* alpha_s = pT + 64 * GT;                           // [GT]
    float* ml_s = alpha_s + GT;                              // [GT][2]
    uint64_t* bars = (uint64_t*)(ml_s + 2 * GT + (GT & 1));  // 8-byte aligned: the counts before it are even

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int sub = lane & 7, tl = lane >> 3;
    const int tg = tid >> 4, cu = tid & 15;
    const WorkItem w = ib.n ? resolve_work_item(ib, blockIdx.x) : p.items[blockIdx.x];
    const int kvh = blockIdx.y;
    const int g0 = blockIdx.z * GT;
    const int n_tiles = w.n_pages;

    auto issue = [&](int i) {  // thread 0 only
        int st = i % NS;
        int32_t pg = p.table[(int64_t)w.trow * p.max_pages_per_seq + w.page_begin + i];
        if (pg < 0 || pg >= p.n_pages) {
            atomicOr(p.status, STATUS_PAGE_OOB);
            pg = 0;  // keep the barrier protocol going; the result is flagged invalid
        }
        const uint8_t* src = p.pool + (int64_t)pg * p.page_bytes + (int64_t)kvh * Gm::STAGE;
        mbar_expect_tx(&bars[st], Gm::STAGE);
        bulk_g2s(stages + (size_t)st * Gm::STAGE, src, Gm::STAGE, &bars[st]);
    };

    grid_dependency_wait();    // the append that precedes this launch has written its pages
    grid_launch_dependents();  // the combine pass may be scheduled; it waits for this grid before reading partials
    if (tid == 0) {
        for (int s = 0; s < NS; s++) mbar_init(&bars[s], 1);
        mbar_fence_init();
        // start streaming right away; the other threads first meet the barriers after the __syncthreads below
        const bool stalled = (int)blockIdx.x == p.stall_item && blockIdx.y == 0 && blockIdx.z == 0;  // test hook, see DecodeParams
        for (int i = 0; i < NS && i < n_tiles && !stalled; i++) issue(i);
    }
    __syncthreads();

    // the query rows of this group, as f32 registers laid out like the pieces each lane reads
    float qr[GT][Gm::EPL];
#pragma unroll
    for (int g = 0; g < GT; g++) {
        int head = kvh * p.G + min(g0 + g, p.G - 1);
#pragma unroll
        for (int pc = 0; pc < Gm::NPC; pc++) {
            int rb = pc * (8 * Gm::PB) + sub * Gm::PB;
#pragma unroll
            for (int e = 0; e < Gm::EPP; e++)
                qr[g][pc * Gm::EPP + e] = load_query(p, D, w.batch, head, row_channel<FMT>(rb, e, Gm::PB));
        }
    }

    float m_run = -INFINITY, l_run = 0.f;  // live in warp g (< GT), uniform over its lanes
    float acc[GT][Gm::CPT];
#pragma unroll
    for (int g = 0; g < GT; g++)
#pragma unroll
        for (int e = 0; e < Gm::CPT; e++) acc[g][e] = 0.f;
    bool failed = false;

    for (int i = 0; i < n_tiles; i++) {
        const int st = i % NS;
        const bool ok = mbar_wait_bounded(&bars[st], (uint32_t)((i / NS) & 1), p.wait_ns);
        if (__syncthreads_or(!ok)) {
            if (tid == 0) atomicOr(p.status, STATUS_WAIT_EXPIRED);
            failed = true;
            break;
        }
        const uint8_t* Ks = stages + (size_t)st * Gm::STAGE;
        const uint8_t* Vs = Ks + Gm::CHUNK;
        const int n_valid = min(PAGE_TOKENS, w.len - (w.page_begin + i) * PAGE_TOKENS);
        const int n_first = max(0, w.first - (w.page_begin + i) * PAGE_TOKENS);  // slots below it lie before the window

        // ---- scores: warp w takes tokens [16w, 16w+16), 4 at a time, 8 lanes per token ----
#pragma unroll
        for (int it = 0; it < 4; it++) {
            const int t = warp * 16 + it * 4 + tl;
            float dot[GT];
#pragma unroll
            for (int g = 0; g < GT; g++) dot[g] = 0.f;
#pragma unroll
            for (int pc = 0; pc < Gm::NPC; pc++) {
                const int rb = pc * (8 * Gm::PB) + sub * Gm::PB;
                float vals[Gm::EPP];
                load_piece<FMT, Gm::PB>(Ks + chunk_addr(FMT, D, 0, t, rb), vals);
                if (Gm::QUANT) {
                    const int blk = (FMT == B200KV_FMT_Q8_1 ? rb : rb * 2) / 32;
                    const float d = __half2float(((const __half*)(Ks + Gm::DATA))[t * (D / 32) + blk]);
#pragma unroll
                    for (int g = 0; g < GT; g++) {
                        float part = 0.f;
#pragma unroll
                        for (int e = 0; e < Gm::EPP; e++) part = fmaf(qr[g][pc * Gm::EPP + e], vals[e], part);
                        dot[g] = fmaf(d, part, dot[g]);
                    }
                } else {
#pragma unroll
                    for (int g = 0; g < GT; g++)
#pragma unroll
                        for (int e = 0; e < Gm::EPP; e++) dot[g] = fmaf(qr[g][pc * Gm::EPP + e], vals[e], dot[g]);
                }
            }
#pragma unroll
            for (int g = 0; g < GT; g++) {
                dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 1);
                dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 2);
                dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 4);
            }
            float mine = dot[0];
#pragma unroll
            for (int g = 1; g < GT; g++)
                if (sub == g) mine = dot[g];
            if (sub < GT) sc[sub * 64 + t] = mine * p.scale;
        }
        __syncthreads();

        // ---- online softmax: warp g owns q-head g of the group ----
        if (warp < GT) {
            float s0 = (lane < n_valid && lane >= n_first) ? sc[warp * 64 + lane] : -INFINITY;
            float s1 = (lane + 32 < n_valid && lane + 32 >= n_first) ? sc[warp * 64 + lane + 32] : -INFINITY;
            float m_new = fmaxf(m_run, warp_max(fmaxf(s0, s1)));
            float a, p0, p1;
            if (PRECISE) {
                a = expf(m_run - m_new), p0 = expf(s0 - m_new), p1 = expf(s1 - m_new);
            } else {
                a = __expf(m_run - m_new), p0 = __expf(s0 - m_new), p1 = __expf(s1 - m_new);
            }
            l_run = l_run * a + warp_sum(p0 + p1);
            m_run = m_new;
            pT[lane * GT + warp] = p0;
            pT[(lane + 32) * GT + warp] = p1;
            if (lane == 0) alpha_s[warp] = a;
        }
        __syncthreads();

        // ---- values: 16 threads per token, 8 tokens at a time; each thread keeps D/16 channels ----
        {
            float al[GT];
            bool rescale = false;
#pragma unroll
            for (int g = 0; g < GT; g++) {
                al[g] = alpha_s[g];
                rescale |= al[g] != 1.f;
            }
            if (rescale) {
#pragma unroll
                for (int g = 0; g < GT; g++)
#pragma unroll
                    for (int e = 0; e < Gm::CPT; e++) acc[g][e] *= al[g];
            }
#pragma unroll 2
            for (int tt = 0; tt < 8; tt++) {
                const int t = tt * 8 + tg;
                if (t < n_valid) {
                    float pr[GT];
#pragma unroll
                    for (int g = 0; g < GT; g++) pr[g] = pT[t * GT + g];
#pragma unroll
                    for (int pc = 0; pc < Gm::NPC2; pc++) {
                        const int rb = pc * (16 * Gm::PB2) + cu * Gm::PB2;
                        float vals[Gm::EPP2];
                        load_piece<FMT, Gm::PB2>(Vs + chunk_addr(FMT, D, 1, t, rb), vals);
                        if constexpr (v_permuted(FMT, D, 1)) {
                            // permuted V row: this thread's elements fall into blocks 2(cu & 1) and 2(cu & 1) + 1
                            const __half* vsc = (const __half*)(Vs + Gm::DATA);
                            const float2 d2 = make_float2(__half2float(vsc[scale_index(FMT, D, 1, t, 2 * (cu & 1))]),
                                                          __half2float(vsc[scale_index(FMT, D, 1, t, 2 * (cu & 1) + 1)]));
#pragma unroll
                            for (int e = 0; e < Gm::EPP2; e++) {
                                const bool upper = FMT == B200KV_FMT_Q8_1 ? (e >= 4) : ((e % 4) >= 2);
                                vals[e] *= upper ? d2.y : d2.x;
                            }
#pragma unroll
                            for (int g = 0; g < GT; g++)
#pragma unroll
                                for (int e = 0; e < Gm::EPP2; e++) acc[g][e] = fmaf(pr[g], vals[e], acc[g][e]);
                        } else {
                            float d = 1.f;
                            if (Gm::QUANT) {
                                const int blk = (FMT == B200KV_FMT_Q8_1 ? rb : rb * 2) / 32;
                                d = __half2float(((const __half*)(Vs + Gm::DATA))[t * (D / 32) + blk]);
                            }
#pragma unroll
                            for (int g = 0; g < GT; g++) {
                                const float pd = Gm::QUANT ? pr[g] * d : pr[g];
#pragma unroll
                                for (int e = 0; e < Gm::EPP2; e++)
                                    acc[g][pc * Gm::EPP2 + e] = fmaf(pd, vals[e], acc[g][pc * Gm::EPP2 + e]);
                            }
                        }
                    }
                }
            }
        }
        __syncthreads();  // every thread is done with stage st
        if (tid == 0 && i + NS < n_tiles) issue(i + NS);
    }

    // ---- write the partial of this split ----
    const int64_t pbase = ((int64_t)blockIdx.x * p.Hkv + kvh) * p.G;
    if (failed) {
        // outstanding copies (if any) are left to land in this CTA's shared memory, which nothing
        // reads any more; publish an empty partial so the combine pass ignores this split
        for (int idx = tid; idx < GT * D; idx += 128) {
            int g = idx / D;
            if (g0 + g < p.G) p.part_o[(pbase + g0 + g) * D + idx % D] = 0.f;
        }
        if (tid < GT && g0 + tid < p.G) {
            p.part_ml[(pbase + g0 + tid) * 2] = -INFINITY;
            p.part_ml[(pbase + g0 + tid) * 2 + 1] = 0.f;
        }
        return;
    }
    if (warp < GT && lane == 0) {
        ml_s[warp * 2] = m_run;
        ml_s[warp * 2 + 1] = l_run;
    }
    float* red = (float*)stages;  // [8 token groups][GT][D]; all stages are consumed by now
#pragma unroll
    for (int g = 0; g < GT; g++)
#pragma unroll
        for (int pc = 0; pc < Gm::NPC2; pc++) {
            const int rb = pc * (16 * Gm::PB2) + cu * Gm::PB2;
#pragma unroll
            for (int e = 0; e < Gm::EPP2; e++)
                red[(tg * GT + g) * D + (v_permuted(FMT, D, 1) ? row_channel_vperm<FMT>(rb, e, Gm::PB2) : row_channel<FMT>(rb, e, Gm::PB2))] =
                    acc[g][pc * Gm::EPP2 + e];
        }
    __syncthreads();
    for (int idx = tid; idx < GT * D; idx += 128) {
        const int g = idx / D, ch = idx % D;
        float sum = 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++) sum += red[(k * GT + g) * D + ch];
        if (g0 + g < p.G) p.part_o[(pbase + g0 + g) * D + ch] = sum;
    }
    if (tid < GT && g0 + tid < p.G) {
        p.part_ml[(pbase + g0 + tid) * 2] = ml_s[tid * 2];
        p.part_ml[(pbase + g0 + tid) * 2 + 1] = ml_s[tid * 2 + 1];
    }
}

struct CombineParams {
    const float* part_o;
    const float* part_ml;
    const int32_t* batch_info;  // per batch entry: {first item, item count}
    void* out;  // may be null when `act` is given
    int64_t ob, oh;
    int32_t Hkv, G, D, dtype;
    // The result as the quantised activation of a W4A8 GEMM (rows = batch entries, columns = (q head, channel)): null, or
    // the block records of q40_common.cuh.  The grid then covers the rows up to the next multiple of 8, which are zero.
    uint8_t* act;
    int* act_status;
    int32_t n_rows;
};

// Second pass: out = sum_i e^{m_i - M} O_i / sum_i e^{m_i - M} l_i over the splits of one (sequence, q-head).
// The pass is pure latency (a few KB per CTA), so nothing in it forms a chain of dependent round trips: the
// (max, sum) pairs of all splits are fetched at once, and so are the partial outputs of each channel.
__global__ void combine_kernel(CombineParams p, const __grid_constant__ InlineBatch ib) {
    __shared__ float wgt_s[MAX_SPLITS], sum_s[MAX_SPLITS];
    __shared__ float den_s;
    const int b = blockIdx.x, hq = blockIdx.y, ch = threadIdx.x;
    const int kvh = hq / p.G, g = hq % p.G;
    grid_dependency_wait();  // the decode kernel has published every partial
    const int64_t act_nb = (int64_t)p.Hkv * p.G * p.D / QK, act_blk = (int64_t)hq * (p.D / QK) + (ch >> 5);
    if (p.act) {  // a warp holds one block of 32 columns of row b
        if (b == 0 && hq == 0 && ch == 0) q40_status_begin(p.act_status);
        if (b >= p.n_rows) {
            q40_quantize_block(0.f, false, p.act, p.n_rows, act_nb, b, act_blk, ch & 31);
            return;
        }
    }
    const int first = ib.n ? ib.ent[b].z : p.batch_info[2 * b], n = ib.n ? ib.ent[b].w : p.batch_info[2 * b + 1];
    const int64_t stride = (int64_t)p.Hkv * p.G;
    const int64_t base = ((int64_t)first * p.Hkv + kvh) * p.G + g;
    // the first eight partial outputs of this channel do not depend on the weights: they travel while the weights are made
    const float* src = p.part_o + base * p.D + ch;
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = (k < n) ? src[(int64_t)k * stride * p.D] : 0.f;
    if (ch < n) {
        const float2 ml = *(const float2*)(p.part_ml + (base + ch * stride) * 2);
        wgt_s[ch] = ml.x, sum_s[ch] = ml.y;
    }
    __syncthreads();
    if (ch == 0) {
        float M = -INFINITY, den = 0.f;
        for (int i = 0; i < n; i++) M = fmaxf(M, wgt_s[i]);
        for (int i = 0; i < n; i++) {
            const float wgt = expf(wgt_s[i] - M);
            den = fmaf(wgt, sum_s[i], den);
            wgt_s[i] = wgt;
        }
        den_s = den;
    }
    __syncthreads();
    float num = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) num = fmaf((k < n) ? wgt_s[k] : 0.f, v[k], num);
#pragma unroll 1
    for (int i0 = 8; i0 < n; i0 += 8) {  // eight partials in flight per round
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = (i0 + k < n) ? src[(int64_t)(i0 + k) * stride * p.D] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++) num = fmaf((i0 + k < n) ? wgt_s[i0 + k] : 0.f, v[k], num);
    }
    const float res = num / den_s;
    if (p.out) st_from_f32(p.out, p.dtype, (int64_t)b * p.ob + (int64_t)hq * p.oh + ch, res);
    if (p.act) q40_quantize_block(round_to_dtype(res, p.dtype), true, p.act, p.n_rows, act_nb, b, act_blk, ch & 31);  // what a quantiser would read back from `out`
}

template <int FMT, int D, int GT>
static int launch_decode_t(const DecodeParams& p, int n_items, cudaStream_t stream, const InlineBatch& ib) {
    using Gm = Geo<FMT, D>;
    const size_t smem = (size_t)Gm::NS * Gm::STAGE + decode_tail_bytes<GT>();
    B200KV_CUDA(cudaFuncSetAttribute(decode_kernel<FMT, D, GT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(n_items, p.Hkv, (p.G + GT - 1) / GT);
    B200KV_CUDA(launch_after_predecessor(decode_kernel<FMT, D, GT>, grid, dim3(128), smem, stream, p, ib));
    return B200KV_OK;
}

template <int FMT>
static int launch_decode_f(const DecodeParams& p, int D, int n_items, cudaStream_t stream, const InlineBatch& ib) {
    if (p.G == 1) return D == 128 ? launch_decode_t<FMT, 128, 1>(p, n_items, stream, ib) : launch_decode_t<FMT, 64, 1>(p, n_items, stream, ib);
    return D == 128 ? launch_decode_t<FMT, 128, 4>(p, n_items, stream, ib) : launch_decode_t<FMT, 64, 4>(p, n_items, stream, ib);
}

// The two launch steps of a decode call, for callers in other translation units.
const InlineBatch& empty_inline_batch() {
    static const InlineBatch e = {};
    return e;
}

int launch_decode_simt(int fmt, int D, const DecodeParams& p, int n_items, cudaStream_t stream, const InlineBatch* ibp) {
    const InlineBatch& ib = ibp ? *ibp : empty_inline_batch();
    switch (fmt) {
        case B200KV_FMT_F32: return launch_decode_f<B200KV_FMT_F32>(p, D, n_items, stream, ib);
        case B200KV_FMT_F16: return launch_decode_f<B200KV_FMT_F16>(p, D, n_items, stream, ib);
        case B200KV_FMT_BF16: return launch_decode_f<B200KV_FMT_BF16>(p, D, n_items, stream, ib);
        case B200KV_FMT_Q8_1: return launch_decode_f<B200KV_FMT_Q8_1>(p, D, n_items, stream, ib);
        case B200KV_FMT_Q4_0: return launch_decode_f<B200KV_FMT_Q4_0>(p, D, n_items, stream, ib);
    }
    return fail("format %d has no decode kernel", fmt);
}
int launch_combine(const DecodeParams& p, const int32_t* batch_info, void* out, int64_t ob, int64_t oh, int n_seqs,
                   int n_q_heads, int D, cudaStream_t stream, const InlineBatch* ibp) {
    const InlineBatch& ib = ibp ? *ibp : empty_inline_batch();
    for (int i = 0; i < ib.n; i++)  // the combine pass holds the weights of one sequence's splits in MAX_SPLITS shared-memory slots
        if (ib.ent[i].w > MAX_SPLITS) return fail("batch entry %d has %d splits, the combine pass takes at most %d", i, ib.ent[i].w, MAX_SPLITS);
    CombineParams cp{};
    cp.part_o = p.part_o, cp.part_ml = p.part_ml, cp.batch_info = batch_info;
    cp.out = out, cp.ob = ob, cp.oh = oh;
    cp.Hkv = p.Hkv, cp.G = p.G, cp.D = D, cp.dtype = p.dtype;
    B200KV_CUDA(launch_after_predecessor(combine_kernel, dim3(n_seqs, n_q_heads), dim3(D), 0, stream, cp, ib));
    return B200KV_OK;
}

// Pages per split of a decode call.
// (1) Few sequences (every (sequence, head group) pair fits the resident CTAs at once): one round of CTAs of nearly
//     equal size, the smallest run length for which all CTAs are resident together.  The kernel is bound by HBM, which
//     the resident CTAs share evenly whatever SM they sit on, so equal CTAs finish together; every further round would
//     pay the start-up of a CTA (page table, first tiles: ~2.5 us) again, with all its neighbours doing the same.
//     The 4-bit kernel is bound by instruction issue, where balance between SMs counts for more: two rounds when the
//     runs stay long.
// (2) Many sequences: 16 CTAs per SM over the run, so that the tail is short; small launches fill one round with up
//     to 8 pages per split instead of one page per CTA.
int64_t decode_pages_per_split(const b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int64_t window, bool use_mma, int nz) {
    const int Hkv = c->L.Hkv;
    auto pages_of = [&](int i) {
        const SeqState& s = c->seqs[seqs[i]];
        const int64_t first = std::max<int64_t>(s.start, window > 0 ? s.len - window : 0);
        return (s.len + PAGE_TOKENS - 1) / PAGE_TOKENS - first / PAGE_TOKENS;
    };
    int64_t total_pages = 0, max_pages = 1;
    for (int i = 0; i < n_seqs; i++) total_pages += pages_of(i), max_pages = std::max<int64_t>(max_pages, pages_of(i));
    const int64_t work = total_pages * Hkv * nz, target_ctas = 148 * 16, one_wave = 148 * 3;
    int64_t chunk = std::max<int64_t>((work + target_ctas - 1) / target_ctas, std::min<int64_t>((work + one_wave - 1) / one_wave, 8));
    int resident;
    if (use_mma) {
        resident = c->L.fmt == B200KV_FMT_Q4_0 ? 4 : (c->L.fmt == B200KV_FMT_Q8_1 ? 3 : 2);
    } else {  // the CUDA-core kernel: its ring of stages (Geo<FMT, D>) decides how many CTAs share an SM
        const int D = c->L.D, fmt = c->L.fmt;
        const int row = fmt == B200KV_FMT_F32 ? D * 4 : (fmt == B200KV_FMT_F16 || fmt == B200KV_FMT_BF16) ? D * 2 : fmt == B200KV_FMT_Q8_1 ? D : D / 2;
        const int scales = (fmt == B200KV_FMT_Q8_1 || fmt == B200KV_FMT_Q4_0) ? PAGE_TOKENS * (D / 32) * 2 : 0;
        const int stage = 2 * (PAGE_TOKENS * row + scales);
        const int ns = std::min(4, std::max(2, 98304 / stage));
        resident = std::max(1, std::min(4, (227 * 1024) / (ns * stage + 4096)));
    }
    int64_t slots = 148 * resident;
    if (use_mma && c->L.fmt == B200KV_FMT_Q4_0 && work >= 2 * slots * 16) slots *= 2;
    if ((int64_t)n_seqs * Hkv * nz <= slots) {
        int64_t cand = std::max<int64_t>(1, work / slots);
        for (; cand < max_pages; cand += std::max<int64_t>(1, cand / 32)) {  // the count falls as cand grows; at max_pages it is one CTA per pair
            int64_t n = 0;
            for (int i = 0; i < n_seqs; i++) n += std::min<int64_t>(MAX_SPLITS, (pages_of(i) + cand - 1) / cand);
            if (n * Hkv * nz <= slots) break;
        }
        chunk = std::min(cand, max_pages);
    }
    return std::max<int64_t>(chunk, 1);
}

int launch_decode(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, const void* q,
                  const int64_t* qs, void* out, const int64_t* os, int32_t dtype, float scale, cudaStream_t stream, int64_t window,
                  const QueryRope* rope) {
    const int Hkv = c->L.Hkv, D = c->L.D, G = n_q_heads / Hkv;
    const bool use_mma = decode_mma_supported(c->L.fmt, D, dtype) && !c->force_simt;
    const int GT = use_mma ? 8 : (G == 1 ? 1 : 4), nz = (G + GT - 1) / GT;
    // ---- work list: split every sequence into runs of pages so that the grid covers the GPU many times ----
    // first visible token of every sequence: the last `window` tokens (window > 0), never before what was trimmed away
    auto first_of = [&](const SeqState& s) { return std::max<int64_t>(s.start, window > 0 ? s.len - window : 0); };
    int64_t total_pages = 0;
    for (int i = 0; i < n_seqs; i++) {
        const SeqState& s = c->seqs[seqs[i]];
        if (s.len <= 0) return fail("sequence %d is empty: nothing to attend to", seqs[i]);
        total_pages += (s.len + PAGE_TOKENS - 1) / PAGE_TOKENS - first_of(s) / PAGE_TOKENS;
    }
    int64_t chunk = decode_pages_per_split(c, n_seqs, seqs, window, use_mma, nz);
    // one entry per sequence: {table row, length, first work item, splits}; the work items follow from it
    InlineBatch ib{};
    std::vector<int4> ent((size_t)n_seqs);
    std::vector<int32_t> first((size_t)n_seqs);
    int n_items = 0;
    size_t n_part = 0;
    for (;;) {
        n_items = 0;
        for (int i = 0; i < n_seqs; i++) {
            const SeqState& s = c->seqs[seqs[i]];
            first[i] = (int32_t)first_of(s);
            const int pages = (int)((s.len + PAGE_TOKENS - 1) / PAGE_TOKENS) - first[i] / PAGE_TOKENS;
            const int splits = (int)std::min<int64_t>(MAX_SPLITS, (pages + chunk - 1) / chunk);
            ent[i] = make_int4(seqs[i], (int)s.len, n_items, splits);
            n_items += splits;
        }
        n_part = (size_t)n_items * Hkv * G;
        // the workspace was sized once, at create: a call whose natural split does not fit takes longer runs instead
        if (n_part * (D + 2) * sizeof(float) <= c->ws_bytes) break;
        if (n_items == n_seqs)
            return fail("%d sequences x %d query heads need %zu bytes of split partials, the workspace holds %zu: create the cache "
                        "with max_q_heads >= %d", n_seqs, n_q_heads, n_part * (D + 2) * sizeof(float), c->ws_bytes, n_q_heads);
        chunk *= 2;
    }
    const bool inline_batch = n_seqs <= INLINE_BATCH;  // small batches travel as a kernel parameter: no copy, no slot
    int slot = -1;
    uint8_t *h = nullptr, *d = nullptr;
    size_t items_bytes = 0;
    if (inline_batch) {
        ib.n = n_seqs;
        memcpy(ib.ent, ent.data(), (size_t)n_seqs * sizeof(int4));
        memcpy(ib.first, first.data(), (size_t)n_seqs * sizeof(int32_t));
    } else {
        items_bytes = (size_t)n_items * sizeof(WorkItem);
        const size_t desc_bytes = items_bytes + (size_t)n_seqs * 8;
        if (staging_acquire(c, desc_bytes, &slot, &h, &d) != B200KV_OK) return B200KV_KO;
        WorkItem* items = (WorkItem*)h;
        int32_t* info = (int32_t*)(h + items_bytes);
        for (int i = 0; i < n_seqs; i++) {
            info[2 * i] = ent[i].z, info[2 * i + 1] = ent[i].w;
            for (int k = 0; k < ent[i].w; k++) items[ent[i].z + k] = make_work_item(ent[i], i, k, first[i]);
        }
        if (staging_upload(c, slot, desc_bytes, stream) != B200KV_OK) return B200KV_KO;
    }

    DecodeParams p{};
    p.pool = c->pool, p.table = c->d_table, p.items = (const WorkItem*)d, p.status = c->d_status;
    p.q = q, p.qb = qs[0], p.qh = qs[1];
    if (rope && rope->cos) p.q_cos = rope->cos, p.q_sin = rope->sin, p.rope_b = rope->stride_b;
    p.part_o = (float*)c->ws;
    p.part_ml = p.part_o + n_part * D;
    p.page_bytes = c->L.page_bytes, p.n_pages = (int32_t)c->n_pages, p.max_pages_per_seq = c->max_pages_per_seq;
    p.Hkv = Hkv, p.G = G, p.dtype = dtype, p.scale = scale;
    p.wait_ns = c->wait_ns;
    if (c->stall_next_decode) p.stall_item = 0, p.wait_ns = 1000000, c->stall_next_decode = false;  // one launch, 1 ms
    int rc;
    {
    ProfScope ps(c, K_DECODE, stream);
    if (decode_mma_supported(c->L.fmt, D, dtype) && !c->force_simt) {
        rc = launch_decode_mma(c->L.fmt, p, n_items, stream, &ib);
    } else
    switch (c->L.fmt) {
        case B200KV_FMT_F32: rc = launch_decode_f<B200KV_FMT_F32>(p, D, n_items, stream, ib); break;
        case B200KV_FMT_F16: rc = launch_decode_f<B200KV_FMT_F16>(p, D, n_items, stream, ib); break;
        case B200KV_FMT_BF16: rc = launch_decode_f<B200KV_FMT_BF16>(p, D, n_items, stream, ib); break;
        case B200KV_FMT_Q8_1: rc = launch_decode_f<B200KV_FMT_Q8_1>(p, D, n_items, stream, ib); break;
        case B200KV_FMT_Q4_0: rc = launch_decode_f<B200KV_FMT_Q4_0>(p, D, n_items, stream, ib); break;
        default: rc = fail("format %d has no decode kernel", c->L.fmt);
    }
    }
    if (rc == B200KV_OK) {
        ProfScope ps(c, K_COMBINE, stream);
        CombineParams cp{};
        cp.part_o = p.part_o, cp.part_ml = p.part_ml, cp.batch_info = (const int32_t*)(d + items_bytes);
        cp.out = out, cp.ob = os[0], cp.oh = os[1];
        cp.Hkv = Hkv, cp.G = G, cp.D = D, cp.dtype = dtype;
        if (rope && rope->act_scratch) cp.act = (uint8_t*)rope->act_scratch + Q_HEADER, cp.act_status = (int*)rope->act_scratch, cp.n_rows = n_seqs;
        const unsigned rows = cp.act ? (unsigned)((n_seqs + 7) / 8 * 8) : (unsigned)n_seqs;
        if (launch_after_predecessor(combine_kernel, dim3(rows, n_q_heads), dim3(D), 0, stream, cp, ib) != cudaSuccess)
            rc = fail("combine launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    if (slot >= 0) staging_release(c, slot, stream);
    return rc;
}

}  // namespace b200kv
