/* b200kv — C ABI of the B200 (sm_100a) KV-cache + attention library.
 *
 * This is the boundary a tract maintainer binds from Rust (extern "C" + raw device
 * pointers): the functions below replace, on the "cuda" runtime, what tract does in
 *   gpu/src/ops/dyn_kv_cache.rs            (GpuDynKVCache: alloc + copy_nd the whole past each step)
 *   cuda/src/ops/flash_attn.rs             (CudaFlashAttention op)
 *   cuda/src/kernels/flash_attn.rs:82-189  (CudaFlashAttn::dispatch_eval launcher)
 *   cuda/src/transform.rs:301-409          (convert_sdpa_to_cuda_flash_attn)
 * and give the CPU-only ops of transformers/src/ops/quant_dyn_kv_cache.rs a device form.
 *
 * Conventions (they mirror tract's own, api/ffi/src/lib.rs:16-60):
 *   - every function returns B200KV_OK or B200KV_KO; after KO, b200kv_last_error() returns a
 *     thread-local message.  All shape / dtype / capacity validation happens on the host
 *     before anything is enqueued; a failed call enqueues nothing and changes no state.
 *   - calls only ENQUEUE work on the given stream (a cudaStream_t / CUstream passed as void*);
 *     there is no hidden device synchronisation.  Host-side bookkeeping (sequence lengths,
 *     page tables) is updated at enqueue time, so the calls on one cache must be issued in
 *     program order on streams the caller keeps ordered — one thread at a time per cache,
 *     like an OpState.  Distinct caches are independent.
 *   - tensors are raw device pointers plus strides in ELEMENTS; the innermost (head_dim) axis
 *     must be contiguous.  The library never allocates caller-visible outputs.
 *   - there is no CPU fallback: without a CUDA device every entry point fails.
 */
#ifndef B200KV_H
#define B200KV_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200KV_OK 0
#define B200KV_KO 1

/* element type of caller tensors (tract DatumType F32 / F16; BF16 is an extension) */
typedef enum { B200KV_F32 = 0, B200KV_F16 = 1, B200KV_BF16 = 2 } b200kv_dtype;

/* storage format of the cache pages */
typedef enum {
    B200KV_FMT_F32 = 0,  /* bit copy of f32 input  (DynKeyValueCache, transformers/src/ops/dyn_kv_cache.rs) */
    B200KV_FMT_F16 = 1,  /* bit copy of f16 input */
    B200KV_FMT_BF16 = 2, /* bit copy of bf16 input */
    B200KV_FMT_Q8_1 = 3, /* blocks of 32 along head_dim: f16 scale + 32 int8 codes, arithmetic of
                            linalg/src/frame/block_quant/q8_1.rs:20-63 (the unused f16 sum is not stored) */
    B200KV_FMT_Q4_0 = 4, /* blocks of 32 along head_dim: f16 scale + 16 bytes of nibbles,
                            linalg/src/frame/block_quant/q4_0.rs:19-95 */
    B200KV_FMT_KIVI8 = 5, /* QuantizedDynKeyValueCache, bits = 8 (transformers/src/ops/quant_dyn_kv_cache.rs) */
    B200KV_FMT_KIVI4 = 6  /* QuantizedDynKeyValueCache, bits = 4 */
} b200kv_format;

typedef struct b200kv_cache b200kv_cache; /* opaque: page pool + page tables of one layer's K (and V) */

typedef struct {
    int32_t device;         /* CUDA device ordinal */
    int32_t format;         /* b200kv_format */
    int32_t n_kv_heads;     /* Hkv */
    int32_t head_dim;       /* D: 64 or 128 */
    int32_t has_values;     /* 1: the cache holds K and V (fused cache + attention); 0: one tensor only
                               (a lone DynKeyValueCache node) */
    int32_t max_seqs;       /* sequences that can be live at once */
    int64_t max_seq_tokens; /* longest sequence (sizes the page table rows) */
    int64_t pool_tokens;    /* capacity of the page pool in tokens, summed over sequences */
    int32_t flags;          /* bit 0: a lone (has_values == 0) KIVI cache quantises per token (the Value layout of
                               QuantizedDynKeyValueCache, per_channel = false) instead of per channel */
    int32_t max_q_heads;    /* most query heads an attention call on this cache will bring (sizes the split-KV workspace,
                               which is allocated once, here); 0 selects 8 * n_kv_heads */
} b200kv_config;

/* Thread-local message of the last failed call on this thread (tract_get_last_error analogue). */
const char* b200kv_last_error(void);

/* Library / build information: "b200kv <version> sm_100a". */
const char* b200kv_version(void);

/* ---- cache life cycle (the OpState of DynKeyValueCache / the fused cache+attention op) ---- */

/* Allocates the page pool and page tables on cfg->device.  Replaces the per-step cuMemAlloc of
 * GpuDynKVCacheState::eval (gpu/src/ops/dyn_kv_cache.rs:88-108). */
int b200kv_create(const b200kv_config* cfg, b200kv_cache** out);
int b200kv_destroy(b200kv_cache* cache);

/* Bytes of the split-KV workspace b200kv_create allocates for this configuration, beside the page pool: the partial
 * outputs of decode attention (one (head_dim + 2)-float record per page run, kv head and query head of the group).  It is
 * sized once from max_seqs and max_q_heads (the reference takes such buffers from the session arena,
 * gpu/src/session_handler.rs:35-46); no call made after b200kv_create allocates or frees device memory: a decode call
 * whose natural split would need more records than the workspace holds cuts its sequences into fewer, longer runs
 * instead.  Returns -1 for a configuration b200kv_create would refuse. */
int64_t b200kv_workspace_bytes(const b200kv_config* cfg);

/* A sequence is one independent state (one tract `State`); ids are small integers reused after free. */
int b200kv_seq_new(b200kv_cache* cache, int32_t* seq_out);
int b200kv_seq_free(b200kv_cache* cache, int32_t seq);

/* Cached length of a sequence: what OpState::resolve_symbols binds the past-length symbol to
 * (transformers/src/ops/dyn_kv_cache.rs:153-156).  Returns -1 on error. */
int64_t b200kv_seq_len(b200kv_cache* cache, int32_t seq);

/* Pages currently unused in the pool, and bytes one page holds (introspection for sizing). */
int64_t b200kv_free_pages(b200kv_cache* cache);
int64_t b200kv_page_bytes(b200kv_cache* cache);

/* ---- append (DynKeyValueCacheState::eval, transformers/src/ops/dyn_kv_cache.rs:158-174;
 *              QuantizedDynKvCacheState::ingest, quant_dyn_kv_cache.rs:403-430) ----
 * Appends n_new tokens to each of n_seqs sequences.  k_new / v_new are [n_seqs, Hkv, n_new, D]
 * with strides {batch, head, token} in elements (D contiguous).  For the bit-copy formats `dtype`
 * must equal the storage type; the quantised formats take f32 / f16 / bf16 input and quantise on
 * append after casting to f32, as the reference does.  v_new must be NULL iff has_values == 0. */
int b200kv_append(b200kv_cache* cache, int32_t n_seqs, const int32_t* seqs, int32_t n_new, const void* k_new,
                  const int64_t k_strides[3], const void* v_new, const int64_t v_strides[3], int32_t dtype,
                  void* stream);

/* b200kv_append with the rotary position embedding of the keys fused in: K_new goes through ApplyRope
 * (transformers/src/ops/apply_rope.rs:143-176, x * cos + rotate_half(x) * sin, each operation rounded to `dtype`) on its
 * way into the pages, which saves the separate pass over K that the graph `ApplyRope -> DynKeyValueCache` makes.
 * cos / sin are [n_seqs, n_new, D] of type `dtype` (the same for every head), strides {batch, token} in elements
 * (0 to broadcast over the batch).  V is stored as given.  Not available for the KIVI formats. */
int b200kv_append_rope(b200kv_cache* cache, int32_t n_seqs, const int32_t* seqs, int32_t n_new, const void* k_new,
                       const int64_t k_strides[3], const void* v_new, const int64_t v_strides[3], const void* cos,
                       const void* sin, const int64_t rope_strides[2], int32_t dtype, void* stream);

/* Stand-alone ApplyRope for the query side (replaces cuda/src/kernels/cu/nn.cu `apply_rope_nd*`): x and out are
 * [batch, n_heads, n_tokens, head_dim] with strides {batch, head, token}; cos / sin as above.  Not in place. */
int b200kv_rope(const void* x, const int64_t x_strides[3], const void* cos, const void* sin, const int64_t rope_strides[2],
                void* out, const int64_t out_strides[3], int32_t batch, int32_t n_heads, int32_t n_tokens, int32_t head_dim,
                int32_t dtype, void* stream);

/* ---- attention over the cache (Sdpa over the accumulated K/V: the fused form of
 *      transformers/src/ops/inplace_kv_cache.rs:135-216; kernels replace cuda/src/kernels/cu/flash_attn.cu) ----
 * q and out are [n_seqs, n_q_heads, n_new, D]; the n_new queries of sequence i are its LAST n_new
 * cached positions (call after b200kv_append), so `causal` masks key j for query r iff
 * j > len_i - n_new + r (bottom-right aligned, transformers/src/ops/flash_sdpa.rs:285-294).
 * n_new == 1 runs the split-KV decode kernel, n_new > 1 the prefill kernel.  scale <= 0 selects
 * 1/sqrt(D).  Quantised pages are dequantised on the fly. */
int b200kv_attend(b200kv_cache* cache, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, int32_t n_new,
                  const void* q, const int64_t q_strides[3], void* out, const int64_t out_strides[3], int32_t dtype,
                  float scale, int32_t causal, void* stream);

/* ---- state access (OpState::save_to / load_from, truncate, freeze:
 *      gpu/src/ops/dyn_kv_cache.rs:18-40,116-125,136-168) ---- */

/* Writes the cached K (and V) of one sequence as contiguous-in-D tensors [Hkv, len, D] with strides
 * {head, token}; quantised formats are dequantised (f32 arithmetic, then cast to `dtype`).  This is the
 * tensor DynKeyValueCache returns to a consumer that is not the fused attention, and what save_to stores.
 * v_out may be NULL. */
int b200kv_export(b200kv_cache* cache, int32_t seq, void* k_out, const int64_t k_strides[2], void* v_out,
                  const int64_t v_strides[2], int32_t dtype, void* stream);

/* Raw quantised state of one sequence, in token order, for bit-exact checks and fast freeze:
 *   Q8_1: codes int8 [Hkv, len, D],        scales f16 [Hkv, len, D/32]
 *   Q4_0: codes uint8 [Hkv, len, D/2] (byte j of a block = element j | element j+16 << 4), scales as above
 * which = 0 for K, 1 for V.  Fails for the bit-copy formats (use b200kv_export). */
int b200kv_export_codes(b200kv_cache* cache, int32_t seq, int32_t which, void* codes, void* scales, void* stream);

/* Raw state of one stream (which = 0: K, 1: V) of a KIVI cache, in the order the reference's stores hold it
 * (transformers/src/ops/quant_dyn_kv_cache.rs:98-116,159-180), for bit-exact checks:
 *   sink      f32 [Hkv, min(len, 4), D]                     the first tokens, never quantised
 *   codes     u8  [Hkv, n_q, D * bits / 8]                  packed codes of the n_q quantised tokens
 *   lo, scale f32 [Hkv, n_q] (per-token stream) or [Hkv, n_q / 32, D] (per-channel stream)
 *   residual  f32 [Hkv, n_res, D]                           per-channel stream: the partial block
 * with n_q = len - 4 (per token) or 32 * ((len - 4) / 32) (per channel), n_res = (len - 4) % 32. */
int b200kv_export_kivi(b200kv_cache* cache, int32_t seq, int32_t which, void* codes, float* lo, float* scale,
                       float* sink, float* residual, void* stream);

/* The fused cache + attention op as one call (InPlaceKvSdpa::eval, transformers/src/ops/inplace_kv_cache.rs:190-216: push
 * K_new / V_new, then Sdpa of Q over the accumulated cache): b200kv_append followed by b200kv_attend with the same n_new,
 * one transition from the host instead of two.  If the attention is refused after the append went through, the appended
 * tokens stay (b200kv_truncate takes them back). */
int b200kv_append_attend(b200kv_cache* cache, int32_t n_seqs, const int32_t* seqs, int32_t n_new, const void* k_new,
                         const int64_t k_strides[3], const void* v_new, const int64_t v_strides[3], int32_t n_q_heads,
                         const void* q, const int64_t q_strides[3], void* out, const int64_t out_strides[3], int32_t dtype,
                         float scale, int32_t causal, void* stream);

/* Sliding-window decode attention (WindowKvSdpa, transformers/src/ops/window_kv_cache.rs:160-228: K / V ring buffers of
 * `window` slots, attention over the valid slots without a mask): the one query of every sequence (q, out:
 * [n_seqs, n_q_heads, 1, D]) attends over its last `window` cached tokens.  Call after b200kv_append, like b200kv_attend.
 * Not available for the KIVI formats. */
int b200kv_attend_window(b200kv_cache* cache, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, const void* q,
                         const int64_t q_strides[3], void* out, const int64_t out_strides[3], int32_t dtype, float scale,
                         int64_t window, void* stream);

/* Decode attention with ApplyRope (transformers/src/ops/apply_rope.rs:143-176) folded into the query load: the result of
 * b200kv_rope on q followed by b200kv_attend with n_new = 1, bit for bit, without the intermediate tensor.  q, out:
 * [n_seqs, n_q_heads, 1, D]; cos / sin: one row of D values of type `dtype` per sequence, `rope_stride` elements apart.
 * Not available for the KIVI formats. */
int b200kv_attend_rope(b200kv_cache* cache, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, const void* q,
                       const int64_t q_strides[3], const void* cos, const void* sin, int64_t rope_stride, void* out,
                       const int64_t out_strides[3], int32_t dtype, float scale, void* stream);

/* Decode attention whose result lands as the quantised activation of the W4A8 GEMM that follows it (the o-projection of
 * a decoder block): b200kv_attend with n_new = 1 (b200kv_attend_rope when cos / sin are given) followed by
 * b200kv_q40_quantize of the [n_seqs, n_q_heads * D] result, bit for bit, without the quantiser launch.  `out` may be null
 * when only the GEMM reads the result.  `scratch`: b200kv_q40_scratch_bytes(n_q_heads * D, n_seqs) bytes, 16-byte aligned;
 * follow with b200kv_q40_gemm_quantized(.., m = n_seqs, scratch, ..) on the same stream.  Not for the KIVI formats. */
int b200kv_attend_q40(b200kv_cache* cache, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, const void* q,
                      const int64_t q_strides[3], const void* cos, const void* sin, int64_t rope_stride, void* out,
                      const int64_t out_strides[3], void* scratch, int32_t dtype, float scale, void* stream);

/* Gives the pages that lie wholly before the last `keep_last` tokens of a sequence back to the pool: the bounded memory of
 * the reference's ring buffer (window_kv_cache.rs:77-137) on the paged store.  The sequence keeps its length (positions go
 * on counting); from now on attention sees at most the tokens from len - keep_last on, export / fork / truncation below
 * that point / multi-query attention fail. */
int b200kv_trim(b200kv_cache* cache, int32_t seq, int64_t keep_last);

/* Drops the tail of a sequence (speculative-decoding rollback; DynKeyValueCacheState::truncate,
 * transformers/src/ops/dyn_kv_cache.rs:112-119 — on device, without the host round trip of
 * gpu/src/ops/dyn_kv_cache.rs:116-125).  Fails if len exceeds the current length. */
int b200kv_truncate(b200kv_cache* cache, int32_t seq, int64_t len);
/* The same for the sequences of a batch in one call (a decode loop rolls every sequence of a step back together, as
 * examples/causal_llm/src/lib.rs:383-408 truncates every cache state of the model): lens[i] is the new length of seqs[i].
 * All sequences are checked first; on KO none has changed. */
int b200kv_truncate_many(b200kv_cache* cache, int32_t n_seqs, const int32_t* seqs, const int64_t* lens);

/* Device-side copy of a sequence into a new one (OpStateFreeze::freeze / unfreeze keep the cache on
 * device, gpu/src/ops/dyn_kv_cache.rs:136-168). */
int b200kv_fork(b200kv_cache* cache, int32_t seq, int32_t* new_seq_out, void* stream);

/* Device status word: 0 unless a kernel recorded a problem (page index out of range, a bounded wait
 * that expired).  Synchronises the stream.  Returns KO and sets the message if the word is non-zero. */
int b200kv_check(b200kv_cache* cache, void* stream);

/* Decode attention (one query per sequence: the n_new == 1 case of b200kv_attend, same arguments and
 * result) whose split-KV partials live in no allocation at all, for callers that cannot allocate device
 * memory for them: a server that has given every free byte of HBM to page pools it made itself before it
 * loaded this library, a runtime whose device arena was sized once and whose allocator hook refuses
 * anything else, or a latency-critical loop in which the device-wide synchronisation implied by
 * cudaMalloc / cudaFree would stall the other streams.  b200kv_attend keeps the partials in the workspace
 * b200kv_create allocates; this entry point keeps them in a fixed 8 MiB device array inside the library
 * (held by every GPU that loads the library, from load to exit) and calls neither cudaMalloc nor cudaFree
 * nor any allocating library routine.
 *   - Limit: page runs x n_kv_heads x (n_q_heads / n_kv_heads) x (head_dim + 2) floats <= 2 Mi floats, where
 *     page runs is the number of splits of the batch (at most 64 per sequence).  A call beyond the limit
 *     fails with a message that states both numbers; nothing is enqueued.
 *   - Not served (refused during validation, nothing enqueued): KIVI caches, which have decode kernels of
 *     their own, and sequences whose front pages b200kv_trim gave back.  b200kv_attend serves both.
 *   - The first call on a device looks up the device address of the array (cudaGetSymbolAddress, with that
 *     device current); make that first call before any stream capture begins.
 *   - All calls on one device share the array, and a call leaves its partials behind; each call overwrites
 *     every slot it reads, so nothing needs clearing, but two calls whose kernels overlap on the GPU
 *     (different streams, or different caches, without an ordering between them) race on it.
 * This entry point has no counterpart in the reference. */
int b200kv_attend_static_scratch(b200kv_cache* cache, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads,
                                 const void* q, const int64_t q_strides[3], void* out, const int64_t out_strides[3],
                                 int32_t dtype, float scale, void* stream);

/* ---- Q4_0 weights x activations: the decode-time linear layers either side of the cache path ----
 * Arithmetic of Q4_0::w4a8_gemm / w4a8_gemv (linalg/src/frame/block_quant/q4_0.rs:199-310), bit for bit: activations
 * quantised per block of 32 to int8 with an f32 scale, exact int32 block dot products, contributions added in
 * ascending block order.  Replaces cuda/src/kernels/cu/mm_mv_q.cu (`mul_vec_q40_m_*`) and cu/quantize.cu behind
 * dispatch_ggml_matvec_q40 (cuda/src/kernels/matmul/mod.rs:481-520). */

/* Bytes of the packed form of an [n, k] Q4_0 matrix (k a multiple of 32), or -1. */
int64_t b200kv_q40_packed_bytes(int64_t n, int64_t k);
/* Repacks `blocks` (device memory; the reference's storage: n rows of k/32 blocks of 18 bytes, f16 scale then 16
 * nibble bytes, cuda/src/rewrite_rules/pad_q40_weights.rs does the reference's own repacking) into `packed`
 * (device memory, 16-byte aligned, b200kv_q40_packed_bytes long).  Done once per weight matrix. */
int b200kv_q40_pack(const void* blocks, int64_t n, int64_t k, void* packed, void* stream);
/* Bytes of device scratch a GEMM with up to m activation rows needs (quantised activations + a status word), or -1.
 * The producers lay the activations out for the kernel that a call with that many rows runs (records of 8 rows below 128
 * rows, tensor-core operand tiles of 128 rows from there on): a producer and the GEMM that reads it are given the same m. */
int64_t b200kv_q40_scratch_bytes(int64_t k, int32_t m);
/* out[m, n] = a[m, k] . W[n, k]^T.  `a` is device memory of type `dtype` (cast to f32 first, as the reference's callers
 * do), rows a_stride elements apart; `out` is f32, rows out_stride elements apart; `scratch` is caller-provided device
 * memory (16-byte aligned) that must not be shared by two calls in flight.  Allocates nothing. */
int b200kv_q40_gemm(const void* packed, int64_t n, int64_t k, const void* a, int64_t a_stride, int32_t m, int32_t dtype,
                    void* scratch, float* out, int64_t out_stride, void* stream);
/* The two halves of b200kv_q40_gemm, for callers that feed several matrices from one activation (the gate and up
 * projections of a gated FFN) or that produce the activation with one of the fused calls below.
 * b200kv_q40_quantize is Q4_0::quantize_row_q8 (q4_0.rs:199-222) for m rows into `scratch`; b200kv_q40_gemm_quantized
 * multiplies what `scratch` holds (m rows of k values) with a packed matrix.  Same stream, same scratch. */
int b200kv_q40_quantize(const void* a, int64_t a_stride, int32_t m, int32_t dtype, int64_t k, void* scratch, void* stream);
int b200kv_q40_gemm_quantized(const void* packed, int64_t n, int64_t k, int32_t m, void* scratch, float* out, int64_t out_stride,
                              void* stream);
/* b200kv_q40_gemm_quantized with the result stored as `out_dtype` (the f32 result rounded once: the Cast that follows
 * the MatMul in the graph, core/src/ops/cast.rs, folded into the store). */
int b200kv_q40_gemm_quantized_as(const void* packed, int64_t n, int64_t k, int32_t m, void* scratch, void* out, int64_t out_stride,
                                 int32_t out_dtype, void* stream);
/* Producers fused with the quantiser: the activation never visits HBM as floats.  Each gives the bits of the separate
 * calls run one after the other.
 *   silu_mul:      scratch <- quantise(Silu(gate) * up)            (b200kv_silu_mul, then b200kv_q40_quantize)
 *   add_rms_norm:  v = x + residual (residual may be null); x_out <- v when x_out is given (it may be x or residual);
 *                  scratch <- quantise(RmsNorm(v, eps) * weight)   (b200kv_add, b200kv_rms_norm, b200kv_q40_quantize); f32 only */
int b200kv_q40_silu_mul_quantize(const void* gate, int64_t gate_stride, const void* up, int64_t up_stride, int32_t m, int32_t dtype,
                                 int64_t k, void* scratch, void* stream);
int b200kv_q40_add_rms_norm_quantize(const float* x, int64_t x_stride, const float* residual, int64_t residual_stride,
                                     const float* weight, float eps, float* x_out, int64_t x_out_stride, int32_t m, int64_t k,
                                     void* scratch, void* stream);
/* Ordering on the stream.  The GEMM and the producers are scheduled behind the kernel before them with a programmatic
 * dependency: they read activations, residuals and scratch only after that kernel has finished, but the packed weights
 * and the norm `weight` vector are fetched earlier.  Those two are constants of the model: they must be complete before
 * the kernel that precedes the call was enqueued (b200kv_q40_pack takes care of this for the matrix it packs). */
/* Synchronises `stream` and reports (once) whether a bounded wait of any GEMM that used `scratch` since the last check expired. */
int b200kv_q40_check(const void* scratch, void* stream);

/* ---- decoder glue between the linear layers and the attention ----
 * RmsNorm over the last axis of [rows, d] (core/src/ops/nn/rms_norm.rs:28-66; kernel rms_norm_f32,
 * linalg/src/generic/rms_norm.rs:7-18; replaces cuda/src/kernels/cu/nn.cu `rms_norm_*`): f32 arithmetic, result cast to `dtype`.
 * `weight` ([d], type `dtype`, may be NULL) is the Mul that follows RmsNorm in the graph, fused.  Strides in elements. */
int b200kv_rms_norm(const void* x, int64_t x_stride, const void* weight, void* out, int64_t out_stride, int64_t rows, int32_t d,
                    float eps, int32_t dtype, void* stream);
/* out = silu(gate) * up over n elements (up may be NULL: plain Silu).  Silu is x * sigmoid(x) with tract-linalg's generic
 * rational sigmoid (linalg/src/generic/sigmoid.rs:11-45, silu.rs:26-30), bit for bit in f32; its result is rounded to `dtype`
 * before the product, as the graph's Silu -> Mul does.  May run in place. */
int b200kv_silu_mul(const void* gate, const void* up, void* out, int64_t n, int32_t dtype, void* stream);
/* out = a + b over n elements (the residual connections; cuda/src/kernels/cu/binary.cu).  May run in place. */
int b200kv_add(const void* a, const void* b, void* out, int64_t n, int32_t dtype, void* stream);
/* out[r] = index of the first maximum of row r of the f32 matrix [rows, n] (ArgMax over the logits: greedy decoding). */
int b200kv_argmax(const float* x, int64_t stride, int64_t rows, int32_t n, int32_t* out, void* stream);
/* out[i] = table[ids[i]]: rows of row_bytes bytes (a multiple of 16); the embedding lookup (core Gather on axis 0). */
int b200kv_gather_rows(const void* table, int64_t n_rows_table, int64_t row_bytes, const int32_t* ids, int64_t n_ids, void* out,
                       void* stream);

/* dst[r, c] = (dst_dtype) src[r, c] through f32 (core Cast; cuda/src/kernels/cu/array.cu `cast_*`): [rows, cols] windows of row-major
 * matrices, strides in elements.  The same types both sides make it a strided copy. */
int b200kv_cast(const void* src, int64_t src_stride, int32_t src_dtype, void* dst, int64_t dst_stride, int32_t dst_dtype,
                int64_t rows, int64_t cols, void* stream);

/* Per-launch timing, off by default.  When enabled, every kernel launched for this cache is bracketed by a
 * CUDA event pair on the caller's stream (what tract-cuda's TractCudaStream does for its profiler,
 * cuda/src/context.rs:364-453).  b200kv_profile_read waits for the recorded launches, returns up to
 * max_records (kernel id, milliseconds) pairs in launch order and clears the log.  Kernel ids:
 * 0 page-table update, 1 append, 2 decode, 3 split combine, 4 export, 5 generic sdpa, 6 prefill.
 * `enable` is a bit set: bit 0 turns the timing on; bit 1 (a test hook) routes decode attention through the
 * CUDA-core kernel even where the tensor-core kernel applies (KIVI caches: through export + the generic kernel), so
 * the two can be checked against each other; bit 2 (a test hook) keeps KIVI decode attention on its CUDA-core
 * kernel alone; bit 3 (a test hook, consumed by the next decode launch of a non-KIVI cache) exercises the give-up path of
 * the bounded waits without any fault: one CTA of that launch issues no copies, its first wait runs out after 1 ms, it
 * sets the status word, publishes an empty partial and returns -- b200kv_check then reports the expired wait, the
 * output of that call is not meaningful, and the cache is usable as before. */
int b200kv_profile(b200kv_cache* cache, int32_t enable);
int b200kv_profile_read(b200kv_cache* cache, int32_t max_records, int32_t* kernel_ids, float* ms, int32_t* n_out);

/* ---- lone Sdpa (transformers/src/ops/sdpa.rs:84-89; replaces convert_sdpa_to_cuda_flash_attn +
 *      CudaFlashAttention for an Sdpa node that is not fused with a cache) ----
 * q [B, Hq, S, D], k / v [B, Hkv, T, D], out [B, Hq, S, D]; strides {batch, head, row} in elements.
 * mask (may be NULL) is additive, [Mb, Mh, S, T] with Mb in {1, B} and Mh in {1, Hq}, strides
 * {batch, head, row, col} (0 to broadcast), element type mask_dtype.  Any D <= 256.  f16 / bf16 tensors at head_dim 64 or 128
 * whose rows start on 16-byte boundaries run on the tensor cores (tcgen05); everything else on a generic CUDA-core kernel. */
int b200kv_sdpa(const void* q, const int64_t q_strides[3], const void* k, const int64_t k_strides[3], const void* v,
                const int64_t v_strides[3], const void* mask, const int64_t mask_strides[4], int32_t mask_dtype,
                void* out, const int64_t out_strides[3], int32_t batch, int32_t n_q_heads, int32_t n_kv_heads,
                int32_t q_len, int32_t kv_len, int32_t head_dim, int32_t dtype, float scale, int32_t causal,
                void* stream);

/* b200kv_sdpa has no cache handle to carry a status word: this synchronises `stream` and reports (once) whether a bounded
 * wait of a b200kv_sdpa call on the current device expired (the analogue of b200kv_check). */
int b200kv_sdpa_check(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200KV_H */
