// Device form of tract's QuantizedDynKeyValueCache (transformers/src/ops/quant_dyn_kv_cache.rs): affine
// int8 / int4 storage quantisation of the KV cache, quantise-on-append, dequantise-on-read.
//
//   per-token store   (PerTokenStore :98-149, the Value layout): every token row gets its own (lo, scale)
//   per-channel store (BlockChannelStore :159-250, the Key layout): every channel gets a (lo, scale) per block
//                     of 32 tokens, computed when the block fills; the partial block stays in f32
//   both keep the first 4 tokens (attention sinks) in f32 (:92).
// The reference runs this on the CPU only and rebuilds the whole f32 cache every step (:432-449).  Here the
// stores live in HBM, appends touch only the new tokens (plus the block that completes), and the arithmetic
// uses explicitly rounded IEEE operations in the reference's order so that codes, lo and scale are
// bit-identical to the CPU's:  scale = (hi > lo) ? (hi - lo) / lv : 1 ;  code = clamp(round((x - lo) / scale), 0, lv)
// (round half away from zero, NaN -> 0) ;  dequant = lo + code * scale (multiply, then add).
#include <algorithm>
#include <cstring>

#include "kivi_common.cuh"

namespace b200kv {

__device__ inline float kivi_lv(int bits) { return bits == 8 ? 255.f : 15.f; }
__device__ inline float kivi_scale(float lo, float hi, float lv) { return hi > lo ? __fdiv_rn(__fsub_rn(hi, lo), lv) : 1.0f; }
__device__ inline uint32_t kivi_code(float x, float lo, float scale, float lv) {
    float r = roundf(__fdiv_rn(__fsub_rn(x, lo), scale));
    if (r < 0.f) r = 0.f;   // f32::clamp keeps NaN; the `as u8` cast then turns it into 0
    if (r > lv) r = lv;
    return (r != r) ? 0u : (uint32_t)r;
}

__device__ inline void kivi_store_code(const KiviView& v, int stream, int32_t pg, int h, int slot, int c, uint32_t code) {
    if (kivi_mma_layout(v.bits, v.D)) {
        uint8_t* at = v.codes[stream] + ((int64_t)pg * v.H + h) * PAGE_TOKENS * v.row_bytes + kivi_code_offset(v.bits, stream, slot, c);
        if (v.bits == 8) {
            *at = (uint8_t)code;
        } else {  // the channel that shares the byte is 16 (K rows) or 8 (permuted V rows) away: the low-nibble lane writes
            const uint32_t other = __shfl_xor_sync(0xffffffffu, code, stream == 0 ? 16 : 8);
            if (code_nibble(B200KV_FMT_Q4_0, 128, stream, c) == 0) *at = (uint8_t)((code & 0xf) | ((other & 0xf) << 4));
        }
        return;
    }
    uint8_t* row = v.codes[stream] + (((int64_t)pg * v.H + h) * PAGE_TOKENS + slot) * v.row_bytes;
    if (v.bits == 8) {
        row[c] = (uint8_t)code;
    } else {  // two codes per byte, even channel in the low nibble (:63-75); the even lane writes the byte
        uint32_t other = __shfl_down_sync(0xffffffffu, code, 1);
        if ((c & 1) == 0) row[c >> 1] = (uint8_t)((code & 0xf) | ((other & 0xf) << 4));
    }
}
struct KiviAppend {
    KiviView v;
    const int32_t* desc;  // per batch entry {sequence, length before the append, -, -}
    const void* src[2];
    int64_t sb[2], sh[2], ss[2];
    int32_t n_seqs, S, dtype;
    int* status;
};

// Pass 1: per-channel streams — every 32-token block that this append completes.  One CTA per (block, head,
// batch entry), one thread per channel.  Rows come from the f32 residual (tokens appended earlier) or from
// the input (tokens of this call).
__global__ void kivi_block_kernel(KiviAppend a, int stream) {
    const KiviView& v = a.v;
    const int b = blockIdx.z, h = blockIdx.y, c = threadIdx.x;
    const int32_t seq = a.desc[4 * b], len0 = a.desc[4 * b + 1];
    const int i_begin = max(len0 - SINK, 0), i_end = max(len0 + a.S - SINK, 0);
    const int j = i_begin / KBLOCK + blockIdx.x;  // block index
    if (j >= i_end / KBLOCK) return;              // not completed by this call
    const float lv = kivi_lv(v.bits);
    const float* res = v.residual + (((int64_t)seq * v.H + h) * 2 + stream) * KBLOCK * v.D;
    float x[KBLOCK];
    float lo = INFINITY, hi = -INFINITY;
#pragma unroll
    for (int ti = 0; ti < KBLOCK; ti++) {
        const int i = j * KBLOCK + ti;
        float val;
        if (i < i_begin) val = res[ti * v.D + c];
        else {
            const int s = i + SINK - len0;
            val = ld_as_f32(a.src[stream], a.dtype, b * a.sb[stream] + h * a.sh[stream] + s * a.ss[stream] + c);
        }
        x[ti] = val;
        lo = fminf(lo, val);   // f32::min / max ignore a NaN operand, like fminf / fmaxf
        hi = fmaxf(hi, val);
    }
    const float scale = kivi_scale(lo, hi, lv);
    const int32_t pg = v.table[(int64_t)seq * v.max_pages_per_seq + (j * KBLOCK) / PAGE_TOKENS];
    if (pg < 0 || pg >= v.n_pages) {
        if (c == 0) atomicOr(a.status, STATUS_PAGE_OOB);
        return;
    }
    const int blk_in_page = (j * KBLOCK % PAGE_TOKENS) / KBLOCK;
    float* par = v.params[stream] + (((int64_t)pg * v.H + h) * 2 + blk_in_page) * 2 * v.D;
    par[c] = lo;
    par[v.D + c] = scale;
#pragma unroll
    for (int ti = 0; ti < KBLOCK; ti++)
        kivi_store_code(v, stream, pg, h, blk_in_page * KBLOCK + ti, c, kivi_code(x[ti], lo, scale, lv));
}

// Pass 2: every new token row.  Sinks, per-token quantisation, and the f32 residual of per-channel streams.
// One CTA per (token, head, batch entry) and stream (grid.x = S * n_streams), one thread per channel.
__global__ void kivi_row_kernel(KiviAppend a) {
    const KiviView& v = a.v;
    const int stream = blockIdx.x / a.S, s = blockIdx.x % a.S;
    const int b = blockIdx.z, h = blockIdx.y, c = threadIdx.x;
    const int32_t seq = a.desc[4 * b], len0 = a.desc[4 * b + 1];
    const int t = len0 + s;
    const float x = ld_as_f32(a.src[stream], a.dtype, b * a.sb[stream] + h * a.sh[stream] + s * a.ss[stream] + c);
    if (t < SINK) {
        v.sinks[((((int64_t)seq * v.H + h) * 2 + stream) * SINK + t) * v.D + c] = x;
        return;
    }
    const int i = t - SINK;
    if (v.per_channel[stream]) {
        // stays in f32 until its block fills; rows of a block completed by this very call were consumed by pass 1
        const int i_end = max(len0 + a.S - SINK, 0);
        if (i >= (i_end / KBLOCK) * KBLOCK)
            v.residual[((((int64_t)seq * v.H + h) * 2 + stream) * KBLOCK + i % KBLOCK) * v.D + c] = x;
        return;
    }
    // per-token: min / max over the D channels of the row
    __shared__ float red_lo[4], red_hi[4];
    float lo = x, hi = x;
    // fold(INFINITY, f32::min) ignores NaN elements: feed +inf / -inf instead of NaN into the reduction
    if (x != x) lo = INFINITY, hi = -INFINITY;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if ((c & 31) == 0) red_lo[c >> 5] = lo, red_hi[c >> 5] = hi;
    __syncthreads();
    lo = red_lo[0], hi = red_hi[0];
    for (int w = 1; w < (int)blockDim.x / 32; w++) lo = fminf(lo, red_lo[w]), hi = fmaxf(hi, red_hi[w]);
    const float lv = kivi_lv(v.bits);
    const float scale = kivi_scale(lo, hi, lv);
    const int32_t pg = v.table[(int64_t)seq * v.max_pages_per_seq + i / PAGE_TOKENS];
    if (pg < 0 || pg >= v.n_pages) {
        if (c == 0) atomicOr(a.status, STATUS_PAGE_OOB);
        return;
    }
    const int slot = i % PAGE_TOKENS;
    kivi_store_code(v, stream, pg, h, slot, c, kivi_code(x, lo, scale, lv));
    if (c == 0) {
        float* par = v.params[stream] + (((int64_t)pg * v.H + h) * PAGE_TOKENS + slot) * 2;
        par[0] = lo, par[1] = scale;
    }
}

struct KiviExport {
    KiviView v;
    int32_t seq;
    int64_t len;
    void* dst[2];
    int64_t dh[2], dt[2];
    int32_t dtype;
};

// dequant_all (:132-148, :222-249): sinks, quantised rows as lo + code * scale, residual verbatim; cast to dtype.
__global__ void kivi_export_kernel(KiviExport e) {
    const KiviView& v = e.v;
    const int stream = blockIdx.z, h = blockIdx.y, c = threadIdx.x;
    const int64_t t = blockIdx.x;
    const float val = kivi_elem(v, e.seq, e.len, stream, h, t, c);
    st_from_f32(e.dst[stream], e.dtype, h * e.dh[stream] + t * e.dt[stream] + c, val);
}

struct KiviRaw {
    KiviView v;
    int32_t seq, stream;
    int64_t len;
    uint8_t* codes;   // [H][n_q][row_bytes]
    float* lo;        // per-token: [H][n_q] ; per-channel: [H][n_fin][D]
    float* scale;
    float* sink;      // [H][n_sink][D]
    float* residual;  // [H][n_res][D]
};

// Raw state in the order the reference holds it (packed codes, parameters, sinks, residual).
__global__ void kivi_raw_kernel(KiviRaw r) {
    const KiviView& v = r.v;
    const int h = blockIdx.y, c = threadIdx.x, s = r.stream;
    const int64_t t = blockIdx.x;
    const int64_t n_sink = r.len < SINK ? r.len : SINK;
    if (t < SINK) {
        r.sink[((int64_t)h * n_sink + t) * v.D + c] = v.sinks[((((int64_t)r.seq * v.H + h) * 2 + s) * SINK + t) * v.D + c];
        return;
    }
    const int64_t i = t - SINK, n_after = r.len - SINK;
    const int32_t pg = v.table[(int64_t)r.seq * v.max_pages_per_seq + i / PAGE_TOKENS];
    const int slot = (int)(i % PAGE_TOKENS);
    const int64_t n_fin = n_after / KBLOCK;
    const int64_t n_q = v.per_channel[s] ? n_fin * KBLOCK : n_after;
    if (i < n_q) {
        if (kivi_mma_layout(v.bits, v.D)) {
            if (v.bits == 8) r.codes[((int64_t)h * n_q + i) * v.row_bytes + c] = (uint8_t)kivi_load_code(v, s, pg, h, slot, c);
            else if (c < v.row_bytes)  // the reference's packing: even channel in the low nibble
                r.codes[((int64_t)h * n_q + i) * v.row_bytes + c] =
                    (uint8_t)(kivi_load_code(v, s, pg, h, slot, 2 * c) | (kivi_load_code(v, s, pg, h, slot, 2 * c + 1) << 4));
        }
        else if (c < v.row_bytes)
            r.codes[((int64_t)h * n_q + i) * v.row_bytes + c] =
                v.codes[s][(((int64_t)pg * v.H + h) * PAGE_TOKENS + slot) * v.row_bytes + c];
        if (v.per_channel[s]) {
            if (i % KBLOCK == 0) {
                const float* par = v.params[s] + (((int64_t)pg * v.H + h) * 2 + slot / KBLOCK) * 2 * v.D;
                r.lo[((int64_t)h * n_fin + i / KBLOCK) * v.D + c] = par[c];
                r.scale[((int64_t)h * n_fin + i / KBLOCK) * v.D + c] = par[v.D + c];
            }
        } else if (c == 0) {
            const float* par = v.params[s] + (((int64_t)pg * v.H + h) * PAGE_TOKENS + slot) * 2;
            r.lo[(int64_t)h * n_q + i] = par[0];
            r.scale[(int64_t)h * n_q + i] = par[1];
        }
    } else {  // residual rows of a per-channel stream
        const int64_t n_res = n_after - n_q;
        r.residual[((int64_t)h * n_res + (i - n_q)) * v.D + c] =
            v.residual[((((int64_t)r.seq * v.H + h) * 2 + s) * KBLOCK + i % KBLOCK) * v.D + c];
    }
}

// ---- host side ------------------------------------------------------------------------------------------

bool fmt_is_kivi(int fmt) { return fmt == B200KV_FMT_KIVI8 || fmt == B200KV_FMT_KIVI4; }

KiviView kivi_view(const b200kv_cache* c) {
    KiviView v{};
    const KiviStore& k = c->kivi;
    for (int s = 0; s < 2; s++) v.codes[s] = k.codes[s], v.params[s] = k.params[s], v.per_channel[s] = k.per_channel[s];
    v.sinks = k.sinks, v.residual = k.residual, v.table = c->d_table;
    v.max_pages_per_seq = c->max_pages_per_seq, v.n_pages = (int32_t)c->n_pages, v.H = c->cfg.n_kv_heads, v.D = c->cfg.head_dim;
    v.bits = k.bits, v.row_bytes = k.row_bytes, v.n_streams = k.n_streams;
    return v;
}

int kivi_create(b200kv_cache* c) {
    KiviStore& k = c->kivi;
    const int H = c->cfg.n_kv_heads, D = c->cfg.head_dim;
    k.bits = c->cfg.format == B200KV_FMT_KIVI8 ? 8 : 4;
    k.row_bytes = D * k.bits / 8;
    k.n_streams = c->cfg.has_values ? 2 : 1;
    // fused cache: Keys per channel, Values per token (the KIVI layout); a lone cache picks with flags bit 0
    k.per_channel[0] = c->cfg.has_values ? 1 : ((c->cfg.flags & 1) ? 0 : 1);
    k.per_channel[1] = 0;
    for (int s = 0; s < k.n_streams; s++) {
        const size_t codes = (size_t)c->n_pages * H * PAGE_TOKENS * k.row_bytes;
        const size_t par = k.per_channel[s] ? (size_t)c->n_pages * H * 2 * 2 * D * 4 : (size_t)c->n_pages * H * PAGE_TOKENS * 2 * 4;
        B200KV_CUDA(cudaMalloc(&k.codes[s], codes));
        B200KV_CUDA(cudaMemset(k.codes[s], 0, codes));
        B200KV_CUDA(cudaMalloc(&k.params[s], par));
        B200KV_CUDA(cudaMemset(k.params[s], 0, par));
    }
    const size_t per_seq = (size_t)c->cfg.max_seqs * H * 2 * D * 4;
    B200KV_CUDA(cudaMalloc(&k.sinks, per_seq * SINK));
    B200KV_CUDA(cudaMemset(k.sinks, 0, per_seq * SINK));
    B200KV_CUDA(cudaMalloc(&k.residual, per_seq * KBLOCK));
    B200KV_CUDA(cudaMemset(k.residual, 0, per_seq * KBLOCK));
    return B200KV_OK;
}

void kivi_destroy(b200kv_cache* c) {
    KiviStore& k = c->kivi;
    for (int s = 0; s < 2; s++) {
        if (k.codes[s]) cudaFree(k.codes[s]);
        if (k.params[s]) cudaFree(k.params[s]);
    }
    if (k.sinks) cudaFree(k.sinks);
    if (k.residual) cudaFree(k.residual);
}

int64_t kivi_page_bytes(const b200kv_cache* c) {
    const KiviStore& k = c->kivi;
    const int H = c->cfg.n_kv_heads, D = c->cfg.head_dim;
    int64_t b = 0;
    for (int s = 0; s < k.n_streams; s++)
        b += (int64_t)H * PAGE_TOKENS * k.row_bytes + (k.per_channel[s] ? (int64_t)H * 2 * 2 * D * 4 : (int64_t)H * PAGE_TOKENS * 8);
    return b;
}

// Pages a sequence of `len` tokens needs: the sinks live outside the pages.
int64_t kivi_pages_for(int64_t len) { return len <= SINK ? 0 : (len - SINK + PAGE_TOKENS - 1) / PAGE_TOKENS; }

int kivi_append(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_new, const void* k_new, const int64_t* ks,
                const void* v_new, const int64_t* vs, int32_t dtype, const int32_t* d_desc, cudaStream_t stream) {
    KiviAppend a{};
    a.v = kivi_view(c);
    a.desc = d_desc;
    a.src[0] = k_new, a.src[1] = v_new;
    a.sb[0] = ks[0], a.sh[0] = ks[1], a.ss[0] = ks[2];
    if (v_new) a.sb[1] = vs[0], a.sh[1] = vs[1], a.ss[1] = vs[2];
    a.n_seqs = n_seqs, a.S = n_new, a.dtype = dtype, a.status = c->d_status;
    const int H = c->cfg.n_kv_heads, D = c->cfg.head_dim;
    ProfScope ps(c, K_APPEND, stream);
    // blocks completed by this call (at most ceil(S / 32) + 1 per sequence), before the residual is overwritten
    const int max_blocks = n_new / KBLOCK + 1;
    for (int s = 0; s < a.v.n_streams; s++)
        if (a.v.per_channel[s]) kivi_block_kernel<<<dim3(max_blocks, H, n_seqs), D, 0, stream>>>(a, s);
    kivi_row_kernel<<<dim3(n_new * a.v.n_streams, H, n_seqs), D, 0, stream>>>(a);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

int kivi_export(b200kv_cache* c, int32_t seq, void* k_out, const int64_t* ks, void* v_out, const int64_t* vs, int32_t dtype,
                cudaStream_t stream) {
    const int64_t len = c->seqs[seq].len;
    if (len == 0) return B200KV_OK;
    KiviExport e{};
    e.v = kivi_view(c);
    e.seq = seq, e.len = len, e.dtype = dtype;
    e.dst[0] = k_out, e.dh[0] = ks[0], e.dt[0] = ks[1];
    if (v_out) e.dst[1] = v_out, e.dh[1] = vs[0], e.dt[1] = vs[1];
    ProfScope ps(c, K_EXPORT, stream);
    kivi_export_kernel<<<dim3((unsigned)len, c->cfg.n_kv_heads, v_out ? 2 : 1), c->cfg.head_dim, 0, stream>>>(e);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

int kivi_fork(b200kv_cache* c, int32_t src, int32_t dst, cudaStream_t stream) {
    KiviStore& k = c->kivi;
    const int H = c->cfg.n_kv_heads, D = c->cfg.head_dim;
    const SeqState &a = c->seqs[src], &b = c->seqs[dst];
    for (size_t i = 0; i < a.pages.size(); i++)
        for (int s = 0; s < k.n_streams; s++) {
            const size_t cb = (size_t)H * PAGE_TOKENS * k.row_bytes;
            const size_t pb = k.per_channel[s] ? (size_t)H * 2 * 2 * D * 4 : (size_t)H * PAGE_TOKENS * 8;
            B200KV_CUDA(cudaMemcpyAsync(k.codes[s] + b.pages[i] * cb, k.codes[s] + a.pages[i] * cb, cb, cudaMemcpyDeviceToDevice, stream));
            B200KV_CUDA(cudaMemcpyAsync((uint8_t*)k.params[s] + b.pages[i] * pb, (uint8_t*)k.params[s] + a.pages[i] * pb, pb,
                                        cudaMemcpyDeviceToDevice, stream));
        }
    const size_t sk = (size_t)H * 2 * SINK * D, rs = (size_t)H * 2 * KBLOCK * D;
    B200KV_CUDA(cudaMemcpyAsync(k.sinks + dst * sk, k.sinks + src * sk, sk * 4, cudaMemcpyDeviceToDevice, stream));
    B200KV_CUDA(cudaMemcpyAsync(k.residual + dst * rs, k.residual + src * rs, rs * 4, cudaMemcpyDeviceToDevice, stream));
    return B200KV_OK;
}

}  // namespace b200kv

using namespace b200kv;

extern "C" int b200kv_export_kivi(b200kv_cache* c, int32_t seq, int32_t which, void* codes, float* lo, float* scale, float* sink,
                                  float* residual, void* stream) {
    if (validate_seqs(c, 1, &seq) != B200KV_OK) return B200KV_KO;
    if (!fmt_is_kivi(c->cfg.format)) return fail("format %d is not a KIVI store", c->cfg.format);
    if (which < 0 || which >= c->kivi.n_streams) return fail("which = %d out of range", which);
    const int64_t len = c->seqs[seq].len;
    if (len == 0) return B200KV_OK;
    DeviceGuard guard(c->cfg.device);
    KiviRaw r{};
    r.v = kivi_view(c);
    r.seq = seq, r.stream = which, r.len = len;
    r.codes = (uint8_t*)codes, r.lo = lo, r.scale = scale, r.sink = sink, r.residual = residual;
    kivi_raw_kernel<<<dim3((unsigned)len, c->cfg.n_kv_heads), c->cfg.head_dim, 0, (cudaStream_t)stream>>>(r);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

// ---- decode attention over a KIVI cache ---------------------------------------------------------------
// Dequantise-inside-attention for the reference's own quantised layout (the CPU op rebuilds the whole f32
// cache every step, quant_dyn_kv_cache.rs:432-449, and hands it to Sdpa).  CUDA-core formulation: a CTA takes a
// run of 32-token tiles of one (sequence, kv head) for up to 4 query heads of the group, dequantises each tile
// into shared memory with exactly the reference's arithmetic (lo + code * scale), and runs the usual online
// softmax; splits are merged by the same combine pass as the other decode kernels.
#include "kivi_simt.cuh"

namespace b200kv {

// kivi_mma.cu
bool kivi_mma_supported(const b200kv_cache* c, int dtype);
int kivi_mma_ctas_per_sm(int bits);
int launch_kivi_mma(b200kv_cache* c, const void* q, const int64_t* qs, int n_seqs, int G, int dtype, float scale, int n_splits,
                    float* part_o, float* part_ml, const InlineBatch& ib, cudaStream_t stream);

int kivi_decode(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, const void* q, const int64_t* qs, void* out,
                const int64_t* os, int32_t dtype, float scale, cudaStream_t stream) {
    const int H = c->cfg.n_kv_heads, D = c->cfg.head_dim, G = n_q_heads / H;
    if (n_seqs > INLINE_BATCH) return fail("a KIVI decode call takes at most %d sequences", INLINE_BATCH);
    int64_t max_len = 0;
    for (int i = 0; i < n_seqs; i++) max_len = std::max<int64_t>(max_len, c->seqs[seqs[i]].len);
    const bool mma = !c->kivi_cuda_core && kivi_mma_supported(c, dtype);
    int ns, n_part_per_seq;
    if (mma) {
        // tensor-core kernel over the finalised blocks in `ns` splits (a few CTAs per SM, at least 4 pages each), plus one
        // partial from the CUDA-core kernel for the sinks and the residual block
        const int64_t pages = (std::max<int64_t>(max_len - SINK, 0) / KBLOCK + 1) / 2;
        const int nz = (G + 7) / 8;
        // pick the split count that fills whole waves of 148 x (CTAs per SM) best (the splits of a batch of
        // equally long sequences cost the same), with at least 4 pages per split and at most 4 waves
        const int64_t units = (int64_t)n_seqs * H * nz, slots = 148 * kivi_mma_ctas_per_sm(c->kivi.bits);
        // one slot of the combine pass goes to the partial of the sinks and the residual block
        const int ns_max = (int)std::max<int64_t>(1, std::min<int64_t>(MAX_SPLITS - 1, pages / 4));
        double best = -1.0;
        ns = 1;
        for (int cand = 1; cand <= ns_max; cand++) {
            const int64_t ctas = units * cand, waves = (ctas + slots - 1) / slots;
            if (waves > 4 && cand > 1) break;
            const double eff = (double)ctas / (double)(waves * slots);
            if (eff > best + 0.02) best = eff, ns = cand;
        }
        n_part_per_seq = ns + 1;
    } else {
        // enough splits to cover the GPU a few times, at least 8 tiles (256 tokens) each
        const int64_t tiles = (std::max<int64_t>(max_len - SINK, 0) + KTILE - 1) / KTILE + 1;
        const int nz = (G + KGT - 1) / KGT;
        ns = (int)std::min<int64_t>(MAX_SPLITS, std::max<int64_t>(1, (148 * 10 + (int64_t)n_seqs * H * nz - 1) / ((int64_t)n_seqs * H * nz)));
        ns = (int)std::max<int64_t>(1, std::min<int64_t>(ns, tiles / 8));
        n_part_per_seq = ns;
    }
    // the workspace was sized once, at create: a call whose natural split does not fit takes fewer, longer splits
    const size_t per_split = (size_t)n_seqs * H * G * (D + 2) * sizeof(float);
    while (ns > 1 && (size_t)(mma ? ns + 1 : ns) * per_split > c->ws_bytes) ns--;
    n_part_per_seq = mma ? ns + 1 : ns;
    if ((size_t)n_part_per_seq * per_split > c->ws_bytes)
        return fail("%d sequences x %d query heads need %zu bytes of split partials, the workspace holds %zu: create the cache with "
                    "max_q_heads >= %d", n_seqs, n_q_heads, (size_t)n_part_per_seq * per_split, c->ws_bytes, n_q_heads);
    InlineBatch ib{};
    ib.n = n_seqs;
    for (int i = 0; i < n_seqs; i++) ib.ent[i] = make_int4(seqs[i], (int)c->seqs[seqs[i]].len, i * n_part_per_seq, n_part_per_seq);
    const size_t n_part = (size_t)n_seqs * n_part_per_seq * H * G;
    KiviDecode p{};
    p.v = kivi_view(c);
    p.q = q, p.qb = qs[0], p.qh = qs[1];
    p.part_o = (float*)c->ws, p.part_ml = p.part_o + n_part * D;
    p.G = G, p.dtype = dtype, p.scale = scale;
    p.n_splits = mma ? 1 : ns, p.f32_only = mma ? 1 : 0, p.part_stride = n_part_per_seq, p.part_off = 0;
    {
        ProfScope ps(c, K_DECODE, stream);
        if (mma) {  // one launch: its extra CTAs run the CUDA-core formulation on the sinks and the residual block
            if (launch_kivi_mma(c, q, qs, n_seqs, G, dtype, scale, ns, p.part_o, p.part_ml, ib, stream) != B200KV_OK) return B200KV_KO;
        } else {
            dim3 grid(n_seqs * p.n_splits, H, (G + KGT - 1) / KGT);
            if (D == 128) kivi_decode_kernel<128><<<grid, 128, 0, stream>>>(p, ib);
            else kivi_decode_kernel<64><<<grid, 128, 0, stream>>>(p, ib);
            B200KV_CUDA(cudaGetLastError());
        }
    }
    DecodeParams dp{};
    dp.part_o = p.part_o, dp.part_ml = p.part_ml, dp.Hkv = H, dp.G = G, dp.dtype = dtype;
    ProfScope ps(c, K_COMBINE, stream);
    return launch_combine(dp, nullptr, out, os[0], os[1], n_seqs, n_q_heads, D, stream, &ib);
}

}  // namespace b200kv
