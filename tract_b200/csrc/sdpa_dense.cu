// Generic scaled-dot-product attention over dense, strided tensors: any head_dim <= 256, GQA,
// optional additive mask with broadcast, causal masking aligned bottom-right.
//
// This is the drop-in for a lone `Sdpa` node (transformers/src/ops/sdpa.rs:84-89), which tract-cuda
// lowers to CudaFlashAttention only for head_dim 64 / 128 in f16 (cuda/src/transform.rs:301-409) and
// otherwise runs on the CPU.  It favours generality over speed: one warp per query row, keys taken 32
// at a time (one per lane), f32 accumulation, online softmax.  The benchmark shapes go through the
// specialised decode / prefill kernels instead.
//
// The same kernel also serves b200kv_attend for the cases its specialised kernels leave out (several queries per
// sequence with f32 queries or an f32 cache): K and V are then read straight from the pages of one sequence, element
// by element, dequantised as the reference's dequantise-on-read does -- nothing is materialised.
#include <cmath>

#include "kivi_common.cuh"

namespace b200kv {

// K / V of one sequence as they lie in a cache (PAGED instantiation of the kernel).
struct PagedSrc {
    const uint8_t* pool;
    const int32_t* table_row;  // page ids of the sequence
    int64_t page_bytes, len;
    int32_t fmt, chunk_bytes, kivi, seq;
    KiviView kv;  // the KIVI stores, when kivi != 0
};

struct DenseParams {
    const void *q, *k, *v, *mask;
    void* out;
    int64_t qs[3], ks[3], vs[3], os[3], ms[4];
    int32_t B, Hq, Hkv, S, T, D;
    int32_t dtype, kv_dtype, mask_dtype, causal;
    float scale;
    PagedSrc src;
};

// Channel d of token j of kv head h, K (which = 0) or V (1), of the sequence behind `s`.
__device__ inline float paged_elem(const PagedSrc& s, int D, int which, int h, int j, int d) {
    if (s.kivi) return kivi_elem(s.kv, s.seq, s.len, which, h, j, d);
    const int32_t pg = s.table_row[j / PAGE_TOKENS];
    const uint8_t* chunk = s.pool + (int64_t)pg * s.page_bytes + (int64_t)(h * 2 + which) * s.chunk_bytes;
    return chunk_elem(chunk, s.fmt, D, which, j % PAGE_TOKENS, d);
}

constexpr int DENSE_WARPS = 4;
constexpr int DENSE_MAX_D = 256;

template <bool PAGED>
__global__ void __launch_bounds__(DENSE_WARPS * 32) sdpa_dense_kernel(DenseParams p) {
    __shared__ float q_s[DENSE_WARPS][DENSE_MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * DENSE_WARPS + warp;
    const int64_t n_rows = (int64_t)p.B * p.Hq * p.S;
    if (row >= n_rows) return;
    const int i = (int)(row % p.S);
    const int hq = (int)((row / p.S) % p.Hq);
    const int b = (int)(row / ((int64_t)p.S * p.Hq));
    const int kvh = hq / (p.Hq / p.Hkv);
    const int D = p.D;

    for (int d = lane; d < D; d += 32) q_s[warp][d] = ld_as_f32(p.q, p.dtype, b * p.qs[0] + hq * p.qs[1] + i * p.qs[2] + d);
    __syncwarp();

    // causal, bottom-right aligned: key j is visible to query i iff j <= i + (T - S)
    const int kv_hi = p.causal ? max(0, min(p.T, i + (p.T - p.S) + 1)) : p.T;
    const int64_t kbase = b * p.ks[0] + kvh * p.ks[1];
    const int64_t vbase = b * p.vs[0] + kvh * p.vs[1];
    int64_t mbase = 0;
    if (p.mask) mbase = b * p.ms[0] + hq * p.ms[1] + i * p.ms[2];

    float m = -INFINITY, l = 0.f;
    float acc[DENSE_MAX_D / 32];
#pragma unroll
    for (int r = 0; r < DENSE_MAX_D / 32; r++) acc[r] = 0.f;

    for (int c0 = 0; c0 < kv_hi; c0 += 32) {
        const int j = c0 + lane;
        float s = -INFINITY;
        if (j < kv_hi) {
            float dot = 0.f;
            const int64_t kr = kbase + j * p.ks[2];
            if (PAGED) {
                for (int d = 0; d < D; d++) dot = fmaf(q_s[warp][d], paged_elem(p.src, D, 0, kvh, j, d), dot);
            } else {
                for (int d = 0; d < D; d++) dot = fmaf(q_s[warp][d], ld_as_f32(p.k, p.kv_dtype, kr + d), dot);
            }
            s = dot * p.scale;
            if (p.mask) s += ld_as_f32(p.mask, p.mask_dtype, mbase + j * p.ms[3]);
        }
        float cm = s;
#pragma unroll
        for (int o = 16; o; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
        const float m_new = fmaxf(m, cm);
        if (m_new == -INFINITY) continue;  // every key so far is masked out
        const float alpha = expf(m - m_new);
        const float pj = (j < kv_hi) ? expf(s - m_new) : 0.f;
        float ps = pj;
#pragma unroll
        for (int o = 16; o; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l = l * alpha + ps;
        m = m_new;
#pragma unroll
        for (int r = 0; r < DENSE_MAX_D / 32; r++) acc[r] *= alpha;
        const int n_here = min(32, kv_hi - c0);
        for (int jj = 0; jj < n_here; jj++) {
            const float pw = __shfl_sync(0xffffffffu, pj, jj);
            const int64_t vr = vbase + (int64_t)(c0 + jj) * p.vs[2];
#pragma unroll
            for (int r = 0; r < DENSE_MAX_D / 32; r++) {
                const int d = lane + 32 * r;
                if (d < D) acc[r] = fmaf(pw, PAGED ? paged_elem(p.src, D, 1, kvh, c0 + jj, d) : ld_as_f32(p.v, p.kv_dtype, vr + d), acc[r]);
            }
        }
    }
    const int64_t obase = b * p.os[0] + hq * p.os[1] + i * p.os[2];
#pragma unroll
    for (int r = 0; r < DENSE_MAX_D / 32; r++) {
        const int d = lane + 32 * r;
        if (d < D) st_from_f32(p.out, p.dtype, obase + d, acc[r] / l);  // l == 0 (no visible key) gives NaN
    }
}

int launch_sdpa_dense(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                      const int64_t* vs, const void* mask, const int64_t* ms, int mask_dtype, void* out,
                      const int64_t* os, int B, int Hq, int Hkv, int S, int T, int D, int dtype, int kv_dtype,
                      float scale, int causal, cudaStream_t stream) {
    DenseParams p{};
    p.q = q, p.k = k, p.v = v, p.mask = mask, p.out = out;
    for (int i = 0; i < 3; i++) p.qs[i] = qs[i], p.ks[i] = ks[i], p.vs[i] = vs[i], p.os[i] = os[i];
    if (mask)
        for (int i = 0; i < 4; i++) p.ms[i] = ms[i];
    p.B = B, p.Hq = Hq, p.Hkv = Hkv, p.S = S, p.T = T, p.D = D;
    p.dtype = dtype, p.kv_dtype = kv_dtype, p.mask_dtype = mask_dtype, p.causal = causal, p.scale = scale;
    const int64_t rows = (int64_t)B * Hq * S;
    if (rows == 0) return B200KV_OK;
    sdpa_dense_kernel<false><<<(unsigned)((rows + DENSE_WARPS - 1) / DENSE_WARPS), DENSE_WARPS * 32, 0, stream>>>(p);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

// The S queries of one sequence (its last S cached positions) over its pages: q, out [Hq, S, D] with strides {-, head, row}.
int launch_sdpa_paged(b200kv_cache* c, int32_t seq, const void* q, const int64_t* qs, void* out, const int64_t* os, int Hq, int S,
                      int dtype, float scale, int causal, cudaStream_t stream) {
    DenseParams p{};
    p.q = q, p.out = out;
    for (int i = 0; i < 3; i++) p.qs[i] = qs[i], p.os[i] = os[i];
    p.B = 1, p.Hq = Hq, p.Hkv = c->L.Hkv, p.S = S, p.T = (int)c->seqs[seq].len, p.D = c->L.D;
    p.dtype = dtype, p.causal = causal, p.scale = scale;
    p.src.pool = c->pool, p.src.table_row = c->d_table + (int64_t)seq * c->max_pages_per_seq;
    p.src.page_bytes = c->L.page_bytes, p.src.len = c->seqs[seq].len, p.src.fmt = c->L.fmt, p.src.chunk_bytes = c->L.chunk_bytes;
    p.src.kivi = fmt_is_kivi(c->L.fmt) ? 1 : 0, p.src.seq = seq;
    if (p.src.kivi) p.src.kv = kivi_view(c);
    const int64_t rows = (int64_t)Hq * S;
    if (rows == 0) return B200KV_OK;
    sdpa_dense_kernel<true><<<(unsigned)((rows + DENSE_WARPS - 1) / DENSE_WARPS), DENSE_WARPS * 32, 0, stream>>>(p);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

}  // namespace b200kv

namespace b200kv {
// Status word of the tensor-core kernel when it runs without a cache handle (the lone Sdpa): one per device.
static __device__ int g_sdpa_status;
static int* sdpa_status_ptr() {
    static int* ptr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_sdpa_status) != cudaSuccess) return nullptr;
        ptr[dev] = (int*)p;
    }
    return ptr[dev];
}
}  // namespace b200kv

using namespace b200kv;

extern "C" int b200kv_sdpa_check(void* stream) {
    int* dptr = sdpa_status_ptr();
    if (!dptr) return fail("no CUDA device");
    int st = 0;
    B200KV_CUDA(cudaMemcpyAsync(&st, dptr, sizeof st, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    B200KV_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (st) {
        B200KV_CUDA(cudaMemsetAsync(dptr, 0, sizeof st, (cudaStream_t)stream));
        return fail("device status %d: a bounded wait of a b200kv_sdpa call expired", st);
    }
    return B200KV_OK;
}

extern "C" int b200kv_sdpa(const void* q, const int64_t q_strides[3], const void* k, const int64_t k_strides[3],
                           const void* v, const int64_t v_strides[3], const void* mask, const int64_t mask_strides[4],
                           int32_t mask_dtype, void* out, const int64_t out_strides[3], int32_t batch,
                           int32_t n_q_heads, int32_t n_kv_heads, int32_t q_len, int32_t kv_len, int32_t head_dim,
                           int32_t dtype, float scale, int32_t causal, void* stream) {
    if (!q || !k || !v || !out || !q_strides || !k_strides || !v_strides || !out_strides) return fail("null tensor or strides");
    if (batch < 0 || q_len < 0 || kv_len < 0) return fail("negative dimension");
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads != 0)
        return fail("n_q_heads (%d) must be a positive multiple of n_kv_heads (%d)", n_q_heads, n_kv_heads);
    if (head_dim <= 0 || head_dim > DENSE_MAX_D) return fail("head_dim %d not in 1..%d", head_dim, DENSE_MAX_D);
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if (mask && (!mask_strides || mask_dtype < B200KV_F32 || mask_dtype > B200KV_BF16)) return fail("mask needs strides and a dtype");
    if (mask && causal) return fail("a mask and is_causal are mutually exclusive");
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) return fail("no CUDA device: b200kv has no CPU fallback");
    if (scale <= 0.f) scale = 1.0f / sqrtf((float)head_dim);
    if (batch == 0 || q_len == 0) return B200KV_OK;
    // f16 / bf16 at head_dim 64 / 128 with 16-byte aligned rows: the tensor-core kernel; everything else the generic one
    if (attn_tc_dense_supported(q, q_strides, k, k_strides, v, v_strides, mask, mask_dtype, out, out_strides, batch, n_q_heads, n_kv_heads,
                                q_len, kv_len, head_dim, dtype, causal)) {
        int* status = sdpa_status_ptr();
        if (status)
            return launch_attn_tc_dense(q, q_strides, k, k_strides, v, v_strides, mask, mask_strides, mask_dtype, out, out_strides, batch,
                                        n_q_heads, n_kv_heads, q_len, kv_len, head_dim, dtype, scale, causal, status, (cudaStream_t)stream);
    }
    return launch_sdpa_dense(q, q_strides, k, k_strides, v, v_strides, mask, mask_strides, mask_dtype, out, out_strides,
                             batch, n_q_heads, n_kv_heads, q_len, kv_len, head_dim, dtype, dtype, scale, causal,
                             (cudaStream_t)stream);
}
