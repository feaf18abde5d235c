// b200kv_attend: attention of the newest tokens of each sequence over its paged cache.
//
// The fused "cache + Sdpa" op of the reference (InPlaceKvSdpa, transformers/src/ops/inplace_kv_cache.rs:135-216)
// appends and then attends; here the two halves are b200kv_append and b200kv_attend, enqueued back to back.
#include <cmath>

#include "internal.h"

using namespace b200kv;

extern "C" int b200kv_attend(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, int32_t n_new,
                             const void* q, const int64_t q_strides[3], void* out, const int64_t out_strides[3],
                             int32_t dtype, float scale, int32_t causal, void* stream_) {
    if (validate_seqs(c, n_seqs, seqs) != B200KV_OK) return B200KV_KO;
    if (!c->L.has_v) return fail("this cache holds one tensor only: attention needs K and V");
    if (!q || !out || !q_strides || !out_strides) return fail("null tensor or strides");
    if (n_new <= 0) return fail("n_new must be positive");
    if (n_q_heads <= 0 || n_q_heads % c->L.Hkv != 0)
        return fail("n_q_heads (%d) must be a positive multiple of n_kv_heads (%d)", n_q_heads, c->L.Hkv);
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    for (int i = 0; i < n_seqs; i++)
        if (c->seqs[seqs[i]].len < n_new)
            return fail("sequence %d holds %lld tokens, fewer than the %d queries: append before attending", seqs[i],
                        (long long)c->seqs[seqs[i]].len, n_new);
    if (scale <= 0.f) scale = 1.0f / sqrtf((float)c->L.D);
    cudaStream_t stream = (cudaStream_t)stream_;
    DeviceGuard guard(c->cfg.device);

    const bool kivi = fmt_is_kivi(c->L.fmt);
    if (n_new == 1 && kivi && !c->force_simt && n_seqs <= 256)
        return kivi_decode(c, n_seqs, seqs, n_q_heads, q, q_strides, out, out_strides, dtype, scale, stream);
    if (n_new == 1 && !kivi) return launch_decode(c, n_seqs, seqs, n_q_heads, q, q_strides, out, out_strides, dtype, scale, stream);
    for (int i = 0; i < n_seqs; i++)
        if (c->seqs[seqs[i]].start > 0) return fail("sequence %d was trimmed: only one query per sequence can attend over it", seqs[i]);

    if (!kivi && !c->force_simt && prefill_tc_supported(c, n_q_heads, dtype, q, q_strides, out, out_strides))
        return launch_prefill_tc(c, n_seqs, seqs, n_q_heads, n_new, q, q_strides, out, out_strides, dtype, scale, causal, stream);
    // block-quantised pages, KIVI stores and head_dim 64: the same pipeline, with the operand tiles rebuilt in shared memory
    if (!c->force_simt && attn_tc_supported(c, n_q_heads, dtype, q, q_strides, out, out_strides))
        return launch_attn_tc_paged(c, n_seqs, seqs, n_q_heads, n_new, q, q_strides, out, out_strides, dtype, scale, causal, stream);

    // otherwise (f32 queries, f32 caches, KIVI stores, unaligned tensors): the generic kernel, one sequence at a time, reading the pages in place
    for (int i = 0; i < n_seqs; i++) {
        const int esz = dtype_size(dtype);
        const void* qi = (const uint8_t*)q + (int64_t)i * q_strides[0] * esz;
        void* oi = (uint8_t*)out + (int64_t)i * out_strides[0] * esz;
        ProfScope ps(c, K_DENSE, stream);
        if (launch_sdpa_paged(c, seqs[i], qi, q_strides, oi, out_strides, n_q_heads, n_new, dtype, scale, causal, stream) != B200KV_OK)
            return B200KV_KO;
    }
    return B200KV_OK;
}

// Sliding-window decode attention: the one query of every sequence attends over its last `window` cached tokens.
// The fused op of transformers/src/ops/window_kv_cache.rs:160-228 (WindowKvSdpa: push K_new / V_new into ring buffers of
// `window` slots, then attend over the valid slots, no mask) is b200kv_append + this call (+ b200kv_trim to bound memory).
extern "C" int b200kv_attend_window(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, const void* q,
                                    const int64_t q_strides[3], void* out, const int64_t out_strides[3], int32_t dtype, float scale,
                                    int64_t window, void* stream_) {
    if (validate_seqs(c, n_seqs, seqs) != B200KV_OK) return B200KV_KO;
    if (!c->L.has_v) return fail("this cache holds one tensor only: attention needs K and V");
    if (fmt_is_kivi(c->L.fmt)) return fail("a KIVI cache has no sliding-window attention");
    if (!q || !out || !q_strides || !out_strides) return fail("null tensor or strides");
    if (window <= 0) return fail("window must be positive");
    if (n_q_heads <= 0 || n_q_heads % c->L.Hkv != 0)
        return fail("n_q_heads (%d) must be a positive multiple of n_kv_heads (%d)", n_q_heads, c->L.Hkv);
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if (scale <= 0.f) scale = 1.0f / sqrtf((float)c->L.D);
    DeviceGuard guard(c->cfg.device);
    return launch_decode(c, n_seqs, seqs, n_q_heads, q, q_strides, out, out_strides, dtype, scale, (cudaStream_t)stream_, window);
}

// Decode attention with ApplyRope (transformers/src/ops/apply_rope.rs:143-176) folded into the query load: what
// b200kv_rope on q followed by b200kv_attend would give, bit for bit, in one launch less.  cos / sin hold one row of D
// values of type `dtype` per sequence (the position of its newest token); rope_stride is the distance between rows.
extern "C" int b200kv_attend_rope(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, const void* q,
                                  const int64_t q_strides[3], const void* cos, const void* sin, int64_t rope_stride, void* out,
                                  const int64_t out_strides[3], int32_t dtype, float scale, void* stream_) {
    if (validate_seqs(c, n_seqs, seqs) != B200KV_OK) return B200KV_KO;
    if (!c->L.has_v) return fail("this cache holds one tensor only: attention needs K and V");
    if (fmt_is_kivi(c->L.fmt)) return fail("a KIVI cache takes its query already rotated: b200kv_rope, then b200kv_attend");
    if (!q || !out || !cos || !sin || !q_strides || !out_strides) return fail("null tensor or strides");
    if (n_q_heads <= 0 || n_q_heads % c->L.Hkv != 0)
        return fail("n_q_heads (%d) must be a positive multiple of n_kv_heads (%d)", n_q_heads, c->L.Hkv);
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if (c->L.D % 2 != 0) return fail("ApplyRope needs an even head_dim");
    if (scale <= 0.f) scale = 1.0f / sqrtf((float)c->L.D);
    DeviceGuard guard(c->cfg.device);
    const QueryRope rope{cos, sin, rope_stride, nullptr};
    return launch_decode(c, n_seqs, seqs, n_q_heads, q, q_strides, out, out_strides, dtype, scale, (cudaStream_t)stream_, 0, &rope);
}

// Decode attention whose result lands as the quantised activation of the W4A8 GEMM that follows it (the o-projection of a
// decoder block): b200kv_attend (or b200kv_attend_rope, when cos / sin are given) followed by b200kv_q40_quantize of the
// [n_seqs, n_q_heads * D] result, bit for bit, without the quantiser launch.  `out` may be null when only the GEMM reads
// the result.  `scratch`: b200kv_q40_scratch_bytes(n_q_heads * D, n_seqs) bytes; then b200kv_q40_gemm_quantized with m = n_seqs.
extern "C" int b200kv_attend_q40(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, const void* q,
                                 const int64_t q_strides[3], const void* cos, const void* sin, int64_t rope_stride, void* out,
                                 const int64_t out_strides[3], void* scratch, int32_t dtype, float scale, void* stream_) {
    if (validate_seqs(c, n_seqs, seqs) != B200KV_OK) return B200KV_KO;
    if (!c->L.has_v) return fail("this cache holds one tensor only: attention needs K and V");
    if (fmt_is_kivi(c->L.fmt)) return fail("a KIVI cache has no fused epilogue: b200kv_attend, then b200kv_q40_quantize");
    if (!q || !q_strides || !scratch || (out && !out_strides)) return fail("null tensor or strides");
    if ((cos == nullptr) != (sin == nullptr)) return fail("cos and sin come together");
    if ((uintptr_t)scratch % 16) return fail("scratch must be 16-byte aligned");
    if (n_q_heads <= 0 || n_q_heads % c->L.Hkv != 0)
        return fail("n_q_heads (%d) must be a positive multiple of n_kv_heads (%d)", n_q_heads, c->L.Hkv);
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if (c->L.D % 32 != 0) return fail("the quantised epilogue needs head_dim a multiple of 32");
    if (scale <= 0.f) scale = 1.0f / sqrtf((float)c->L.D);
    DeviceGuard guard(c->cfg.device);
    const QueryRope ends{cos, sin, rope_stride, scratch};
    const int64_t no_strides[3] = {0, 0, 0};
    return launch_decode(c, n_seqs, seqs, n_q_heads, q, q_strides, out, out ? out_strides : no_strides, dtype, scale, (cudaStream_t)stream_, 0, &ends);
}

// The fused cache + attention op as one call (InPlaceKvSdpa::eval, transformers/src/ops/inplace_kv_cache.rs:190-216: push
// K_new / V_new, then Sdpa of Q over the accumulated cache): b200kv_append followed by b200kv_attend, one transition
// from the host instead of two.
extern "C" int b200kv_append_attend(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_new, const void* k_new,
                                    const int64_t k_strides[3], const void* v_new, const int64_t v_strides[3], int32_t n_q_heads,
                                    const void* q, const int64_t q_strides[3], void* out, const int64_t out_strides[3], int32_t dtype,
                                    float scale, int32_t causal, void* stream) {
    if (!q || !out || !q_strides || !out_strides) return fail("null tensor or strides");  // before anything is appended
    if (b200kv_append(c, n_seqs, seqs, n_new, k_new, k_strides, v_new, v_strides, dtype, stream) != B200KV_OK) return B200KV_KO;
    return b200kv_attend(c, n_seqs, seqs, n_q_heads, n_new, q, q_strides, out, out_strides, dtype, scale, causal, stream);
}
