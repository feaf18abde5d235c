// Host-side mirror, in C++, of the tract operator interface for the KV-cache + attention path, on top of
// the C ABI of include/b200kv.h.  tract's host code is Rust; where no Rust toolchain is available this
// header plays the part of the ops a maintainer would add to tract-cuda, with the same names, argument
// meaning and error behaviour:
//
//   DynKeyValueCache / DynKeyValueCacheState   transformers/src/ops/dyn_kv_cache.rs:69-239 (GPU twin
//                                              gpu/src/ops/dyn_kv_cache.rs:58-259): a stateful op whose eval()
//                                              appends its input along the sequence axis and returns the whole
//                                              cache; load_from / save_to / resolve_symbols / truncate / freeze
//   QuantizedDynKeyValueCache                  transformers/src/ops/quant_dyn_kv_cache.rs:286-495: the same with
//                                              quantised storage; eval() returns the dequantised cache
//   Sdpa                                       transformers/src/ops/sdpa.rs:84-89: stateless attention
//   PagedKvSdpa                                the fused {cache K, cache V, Sdpa} op, the pattern of
//                                              InPlaceKvSdpa (transformers/src/ops/inplace_kv_cache.rs:135-216):
//                                              inputs [Q, K_new, V_new], output = attention over the accumulated cache
//
// Errors are exceptions carrying the library's last-error text (tract: TractResult / anyhow).  Tensors are
// device pointers with shape and strides in elements, the innermost axis contiguous — what a DeviceTensor
// hands out (gpu/src/tensor/mod.rs:113-146).  Nothing here computes on the host.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>

#include "../../include/b200kv.h"

namespace tract_b200 {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};
inline void ck(int rc) {
    if (rc != B200KV_OK) throw Error(b200kv_last_error());
}

enum class DatumType { F32 = B200KV_F32, F16 = B200KV_F16, BF16 = B200KV_BF16 };
inline int size_of(DatumType dt) { return dt == DatumType::F32 ? 4 : 2; }

// A rank-4 [B, H, S, D] device tensor view (rank-3 callers insert H = 1, as FlashSdpaOp::eval does).
struct DeviceTensor {
    void* ptr = nullptr;
    DatumType dt = DatumType::F32;
    int64_t shape[4] = {0, 0, 0, 0};
    int64_t strides[4] = {0, 0, 0, 1};
    static DeviceTensor contiguous(void* p, DatumType dt, int64_t b, int64_t h, int64_t s, int64_t d) {
        DeviceTensor t;
        t.ptr = p, t.dt = dt;
        t.shape[0] = b, t.shape[1] = h, t.shape[2] = s, t.shape[3] = d;
        t.strides[3] = 1, t.strides[2] = d, t.strides[1] = s * d, t.strides[0] = h * s * d;
        return t;
    }
};

// ---- stateless attention ------------------------------------------------------------------------------
struct Sdpa {
    float scale = 0.f;  // 0: 1/sqrt(D), the op's default when `scale` is None
    DatumType datum_type = DatumType::F32;
    bool is_causal = false;

    // inputs [q, k, v] (+ optional additive mask [Mb, Mh, S, T]); output has q's shape and type.
    void eval(const DeviceTensor& q, const DeviceTensor& k, const DeviceTensor& v, const DeviceTensor* mask, const DeviceTensor& out,
              void* stream) const {
        if (q.shape[0] != k.shape[0] || q.shape[3] != k.shape[3]) throw Error("Batch / head dim mismatch between Q and K");
        if (k.shape[1] != v.shape[1] || k.shape[2] != v.shape[2]) throw Error("K/V shape mismatch");
        int64_t ms[4] = {0, 0, 0, 0};
        if (mask) {
            for (int i = 0; i < 4; i++) ms[i] = mask->strides[i];
            if (mask->shape[0] == 1) ms[0] = 0;  // broadcast over batch / heads
            if (mask->shape[1] == 1) ms[1] = 0;
        }
        ck(b200kv_sdpa(q.ptr, q.strides, k.ptr, k.strides, v.ptr, v.strides, mask ? mask->ptr : nullptr, mask ? ms : nullptr,
                       mask ? (int)mask->dt : 0, out.ptr, out.strides, (int32_t)q.shape[0], (int32_t)q.shape[1], (int32_t)k.shape[1],
                       (int32_t)q.shape[2], (int32_t)k.shape[2], (int32_t)q.shape[3], (int)q.dt, scale, is_causal ? 1 : 0, stream));
    }
};

// ---- cache ops ------------------------------------------------------------------------------------------
struct CacheSpec {
    std::string name;
    int axis = 2;  // the sequence axis of [B, H, S, D]; the only one the paged store supports
    int format = B200KV_FMT_F16;
    int n_kv_heads = 0, head_dim = 0;
    int64_t capacity_tokens = 0;  // what tract's memory-sizing hints would give (transformers/src/lib.rs:107-116)
    bool per_token = false;       // a lone quantised cache: Value layout instead of Key layout
};

// One (node, State) pair: owns a handle with a single sequence, like an OpState owns its cache tensor.
class KvState {
  public:
    KvState(const CacheSpec& spec, bool has_values, int device) : spec_(spec), has_values_(has_values) {
        if (spec.axis != 2) throw Error("seq axis must be 2 ([B, H, S, D])");
        b200kv_config cfg{};
        cfg.device = device, cfg.format = spec.format, cfg.n_kv_heads = spec.n_kv_heads, cfg.head_dim = spec.head_dim;
        cfg.has_values = has_values ? 1 : 0, cfg.max_seqs = 2;  // the live state + one frozen copy
        cfg.max_seq_tokens = spec.capacity_tokens, cfg.pool_tokens = 2 * spec.capacity_tokens;
        cfg.flags = spec.per_token ? 1 : 0;
        ck(b200kv_create(&cfg, &cache_));
        try {
            ck(b200kv_seq_new(cache_, &seq_));
        } catch (...) {
            b200kv_destroy(cache_);
            throw;
        }
    }
    ~KvState() {
        if (cache_) b200kv_destroy(cache_);
    }
    KvState(const KvState&) = delete;
    KvState& operator=(const KvState&) = delete;

    // OpState::resolve_symbols: the value the past-length symbol is bound to.
    int64_t past_len() const {
        int64_t n = b200kv_seq_len(cache_, seq_);
        if (n < 0) throw Error(b200kv_last_error());
        return n;
    }
    // OpState::load_from: the initial cache tensor(s) [1, H, P, D] are ingested like any input (the quantised
    // formats re-quantise them token by token, as QuantizedDynKvCacheState::load_from does).
    void load_from(const DeviceTensor& k, const DeviceTensor* v, void* stream) {
        if (past_len() != 0) throw Error("KV cache " + spec_.name + " was already initialized");
        append(k, v, stream);
    }
    // OpState::save_to: the cache as contiguous [H, len, D] tensors of type dt.
    void save_to(void* k_out, void* v_out, DatumType dt, void* stream) const {
        if (past_len() == 0) throw Error("KV cache " + spec_.name + " was never initialized");
        const int64_t st[2] = {past_len() * spec_.head_dim, spec_.head_dim};
        ck(b200kv_export(cache_, seq_, k_out, st, v_out, v_out ? st : nullptr, (int)dt, stream));
    }
    void truncate(int64_t len) {
        if (past_len() == 0) throw Error("Can not truncate a zero-len kv-cache value");
        ck(b200kv_truncate(cache_, seq_, len));
    }
    // OpStateFreeze::freeze / FrozenOpState::unfreeze: the frozen state is a device-side copy.
    int32_t freeze(void* stream) {
        int32_t f;
        ck(b200kv_fork(cache_, seq_, &f, stream));
        return f;
    }
    void unfreeze(int32_t frozen) {
        ck(b200kv_seq_free(cache_, seq_));
        seq_ = frozen;
    }
    void append(const DeviceTensor& k, const DeviceTensor* v, void* stream) {
        if (k.shape[0] != 1) throw Error("one State holds one sequence: batch must be 1");
        ck(b200kv_append(cache_, 1, &seq_, (int32_t)k.shape[2], k.ptr, k.strides, v ? v->ptr : nullptr, v ? v->strides : nullptr,
                         (int)k.dt, stream));
    }
    // push K_new / V_new, then attend: InPlaceKvSdpa::eval as one call into the library
    void append_attend(const DeviceTensor& k, const DeviceTensor& v, const DeviceTensor& q, const DeviceTensor& out, float scale, bool causal,
                       void* stream) {
        if (k.shape[0] != 1) throw Error("one State holds one sequence: batch must be 1");
        ck(b200kv_append_attend(cache_, 1, &seq_, (int32_t)k.shape[2], k.ptr, k.strides, v.ptr, v.strides, (int32_t)q.shape[1], q.ptr,
                                q.strides, out.ptr, out.strides, (int)q.dt, scale, causal ? 1 : 0, stream));
    }
    void attend(const DeviceTensor& q, const DeviceTensor& out, float scale, bool causal, void* stream) {
        ck(b200kv_attend(cache_, 1, &seq_, (int32_t)q.shape[1], (int32_t)q.shape[2], q.ptr, q.strides, out.ptr, out.strides, (int)q.dt,
                         scale, causal ? 1 : 0, stream));
    }
    // WindowKvSdpa (transformers/src/ops/window_kv_cache.rs:160-228): decode attention over the last `window` tokens, then the
    // pages before the window go back to the pool, as the reference's ring buffer forgets them.
    void attend_window(const DeviceTensor& q, const DeviceTensor& out, float scale, int64_t window, void* stream) {
        ck(b200kv_attend_window(cache_, 1, &seq_, (int32_t)q.shape[1], q.ptr, q.strides, out.ptr, out.strides, (int)q.dt, scale, window, stream));
        ck(b200kv_trim(cache_, seq_, window));
    }
    // ApplyRope (transformers/src/ops/apply_rope.rs:143-176) on the query, then Sdpa over the cache, as one launch:
    // cos / sin are the [1, 1, D] rows of the newest position.
    void attend_rope(const DeviceTensor& q, const DeviceTensor& cos, const DeviceTensor& sin, const DeviceTensor& out, float scale,
                     void* stream) {
        ck(b200kv_attend_rope(cache_, 1, &seq_, (int32_t)q.shape[1], q.ptr, q.strides, cos.ptr, sin.ptr, 0, out.ptr, out.strides,
                              (int)q.dt, scale, stream));
    }
    // Sdpa at S = 1 whose only consumer is a Q4_0 MatMul: the result lands in `scratch` as that MatMul's quantised activation
    // (Q40MatMul::eval_quantized with m = 1 follows).  cos / sin (ApplyRope on q) and out are optional.
    void attend_q40(const DeviceTensor& q, const void* cos, const void* sin, void* out, const int64_t* out_strides, void* scratch,
                    float scale, void* stream) {
        ck(b200kv_attend_q40(cache_, 1, &seq_, (int32_t)q.shape[1], q.ptr, q.strides, cos, sin, 0, out, out_strides, scratch, (int)q.dt,
                             scale, stream));
    }
    void check(void* stream) { ck(b200kv_check(cache_, stream)); }
    const CacheSpec& spec() const { return spec_; }

  private:
    CacheSpec spec_;
    bool has_values_;
    b200kv_cache* cache_ = nullptr;
    int32_t seq_ = -1;
};

// DynKeyValueCache (and, with a quantised format, QuantizedDynKeyValueCache) as a lone node: eval() appends
// the input and writes the whole cache, [1, H, P + S, D] in the input's type, into `out`.
struct DynKeyValueCache {
    CacheSpec spec;
    KvState* state(int device) const { return new KvState(spec, /*has_values=*/false, device); }
    // Returns the new length (the axis dim of the op's output fact, P + S).
    static int64_t eval(KvState& st, const DeviceTensor& input, void* out, void* stream) {
        st.append(input, nullptr, stream);
        st.save_to(out, nullptr, input.dt, stream);
        return st.past_len();
    }
};

// The fused op: inputs [Q, K_new, V_new]; output = Sdpa(Q, cache(K), cache(V)).
struct PagedKvSdpa {
    CacheSpec spec;
    float scale = 0.f;
    bool is_causal = true;
    KvState* state(int device) const { return new KvState(spec, /*has_values=*/true, device); }
    void eval(KvState& st, const DeviceTensor& q, const DeviceTensor& k_new, const DeviceTensor& v_new, const DeviceTensor& out,
              void* stream) const {
        st.append_attend(k_new, v_new, q, out, scale, is_causal, stream);
    }
};

// ---- the ops either side of the cache path ---------------------------------------------------------------
// A Q4_0 weight constant [n, k] applied with the arithmetic of Q4_0::w4a8_gemm (linalg/src/frame/block_quant/q4_0.rs:260-310);
// what dispatch_ggml_matvec_q40 (cuda/src/kernels/matmul/mod.rs:481-520) does today.  `packed` and `scratch` are device
// buffers the caller owns (sizes from packed_bytes / scratch_bytes): nothing is allocated here.
struct Q40MatMul {
    int64_t n = 0, k = 0;
    const void* packed = nullptr;
    static int64_t packed_bytes(int64_t n, int64_t k) { return b200kv_q40_packed_bytes(n, k); }
    static int64_t scratch_bytes(int64_t k, int32_t m) { return b200kv_q40_scratch_bytes(k, m); }
    // once per weight: `blocks` is the reference's storage, n rows of k / 32 blocks of 18 bytes
    void pack(const void* blocks, void* packed_out, void* stream) {
        ck(b200kv_q40_pack(blocks, n, k, packed_out, stream));
        packed = packed_out;
    }
    // out[m, n] (f32) = a[m, k] . W^T
    void eval(const void* a, int64_t a_stride, int32_t m, DatumType dt, void* scratch, float* out, int64_t out_stride, void* stream) const {
        if (!packed) throw Error("Q4_0 weights were not packed");
        ck(b200kv_q40_gemm(packed, n, k, a, a_stride, m, (int)dt, scratch, out, out_stride, stream));
    }
    // The product with the m activation rows `scratch` already holds in quantised form (one of the producers below ran on
    // the same stream); `out` is of type out_dt: the Cast that follows the MatMul in the graph, folded into the store.
    void eval_quantized(int32_t m, void* scratch, void* out, int64_t out_stride, DatumType out_dt, void* stream) const {
        if (!packed) throw Error("Q4_0 weights were not packed");
        ck(b200kv_q40_gemm_quantized_as(packed, n, k, m, scratch, out, out_stride, (int)out_dt, stream));
    }
};

// Producers of the quantised activation of a Q40MatMul (Q4_0::quantize_row_q8, linalg/src/frame/block_quant/q4_0.rs:199-222),
// alone or fused with the nodes before the MatMul; each gives the bits of the separate nodes run one after the other.
inline void q40_quantize(const void* a, int64_t a_stride, int32_t m, DatumType dt, int64_t k, void* scratch, void* stream) {
    ck(b200kv_q40_quantize(a, a_stride, m, (int)dt, k, scratch, stream));
}
// Silu(gate) * up -> quantise
inline void q40_silu_mul_quantize(const void* gate, int64_t gate_stride, const void* up, int64_t up_stride, int32_t m, DatumType dt, int64_t k,
                                  void* scratch, void* stream) {
    ck(b200kv_q40_silu_mul_quantize(gate, gate_stride, up, up_stride, m, (int)dt, k, scratch, stream));
}
// v = x + residual (residual may be null; v stored to x_out when given) -> RmsNorm(v, eps) * weight -> quantise; f32
inline void q40_add_rms_norm_quantize(const float* x, int64_t x_stride, const float* residual, int64_t residual_stride, const float* weight,
                                      float eps, float* x_out, int64_t x_out_stride, int32_t m, int64_t k, void* scratch, void* stream) {
    ck(b200kv_q40_add_rms_norm_quantize(x, x_stride, residual, residual_stride, weight, eps, x_out, x_out_stride, m, k, scratch, stream));
}

// RmsNorm over the last axis (core/src/ops/nn/rms_norm.rs), optionally fused with the Mul by a weight vector that follows it.
struct RmsNorm {
    float eps = 1e-5f;
    void eval(const void* x, int64_t x_stride, const void* weight, void* out, int64_t out_stride, int64_t rows, int32_t d, DatumType dt,
              void* stream) const {
        ck(b200kv_rms_norm(x, x_stride, weight, out, out_stride, rows, d, eps, (int)dt, stream));
    }
};

// Silu (and the Mul that follows it in a gated FFN), Add, Cast, ArgMax, Gather on axis 0: the element-wise nodes of a decoder block.
inline void silu_mul(const void* gate, const void* up, void* out, int64_t n, DatumType dt, void* stream) {
    ck(b200kv_silu_mul(gate, up, out, n, (int)dt, stream));
}
inline void add(const void* a, const void* b, void* out, int64_t n, DatumType dt, void* stream) { ck(b200kv_add(a, b, out, n, (int)dt, stream)); }
inline void cast(const void* src, int64_t src_stride, DatumType src_dt, void* dst, int64_t dst_stride, DatumType dst_dt, int64_t rows,
                 int64_t cols, void* stream) {
    ck(b200kv_cast(src, src_stride, (int)src_dt, dst, dst_stride, (int)dst_dt, rows, cols, stream));
}
inline void argmax(const float* x, int64_t stride, int64_t rows, int32_t n, int32_t* out, void* stream) {
    ck(b200kv_argmax(x, stride, rows, n, out, stream));
}
inline void gather_rows(const void* table, int64_t n_rows, int64_t row_bytes, const int32_t* ids, int64_t n_ids, void* out, void* stream) {
    ck(b200kv_gather_rows(table, n_rows, row_bytes, ids, n_ids, out, stream));
}

}  // namespace tract_b200
