//! Raw FFI declarations of `libb200kv.so`: one item per symbol of `include/b200kv.h`, same order, same
//! argument lists.  Drop into `cuda/src/b200kv_sys.rs` of tract-cuda behind the `b200kv` feature.
//!
//! Conventions of the library: every call returns `B200KV_OK` (0) or `B200KV_KO` (1) and leaves a
//! thread-local message behind on KO (`b200kv_last_error`), validates on the host before it enqueues
//! anything, and only ENQUEUES on the `CUstream` it is given.  Tensors are raw device pointers plus
//! strides in ELEMENTS; the head_dim axis must be contiguous.
#![allow(non_camel_case_types, clippy::too_many_arguments)]

use std::os::raw::{c_char, c_float, c_int, c_void};

pub const B200KV_OK: c_int = 0;
pub const B200KV_KO: c_int = 1;

/// `b200kv_dtype`: element type of caller tensors.
pub const B200KV_F32: i32 = 0;
pub const B200KV_F16: i32 = 1;
pub const B200KV_BF16: i32 = 2;

/// `b200kv_format`: storage format of the cache pages.
pub const B200KV_FMT_F32: i32 = 0;
pub const B200KV_FMT_F16: i32 = 1;
pub const B200KV_FMT_BF16: i32 = 2;
pub const B200KV_FMT_Q8_1: i32 = 3;
pub const B200KV_FMT_Q4_0: i32 = 4;
pub const B200KV_FMT_KIVI8: i32 = 5;
pub const B200KV_FMT_KIVI4: i32 = 6;

/// Opaque handle: page pool, page tables and split-KV workspace of one layer's K (and V).
#[repr(C)]
pub struct b200kv_cache {
    _private: [u8; 0],
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct b200kv_config {
    pub device: i32,
    pub format: i32,
    pub n_kv_heads: i32,
    pub head_dim: i32,
    pub has_values: i32,
    pub max_seqs: i32,
    pub max_seq_tokens: i64,
    pub pool_tokens: i64,
    /// bit 0: a lone KIVI cache quantises per token (the Value layout) instead of per channel
    pub flags: i32,
    /// most query heads an attention call will bring (sizes the split-KV workspace); 0 = 8 * n_kv_heads
    pub max_q_heads: i32,
}

extern "C" {
    pub fn b200kv_last_error() -> *const c_char;
    pub fn b200kv_version() -> *const c_char;

    // ---- cache life cycle ----
    pub fn b200kv_create(cfg: *const b200kv_config, out: *mut *mut b200kv_cache) -> c_int;
    pub fn b200kv_workspace_bytes(cfg: *const b200kv_config) -> i64;
    pub fn b200kv_destroy(cache: *mut b200kv_cache) -> c_int;
    pub fn b200kv_seq_new(cache: *mut b200kv_cache, seq_out: *mut i32) -> c_int;
    pub fn b200kv_seq_free(cache: *mut b200kv_cache, seq: i32) -> c_int;
    pub fn b200kv_seq_len(cache: *mut b200kv_cache, seq: i32) -> i64;
    pub fn b200kv_free_pages(cache: *mut b200kv_cache) -> i64;
    pub fn b200kv_page_bytes(cache: *mut b200kv_cache) -> i64;

    // ---- append ----
    pub fn b200kv_append(
        cache: *mut b200kv_cache, n_seqs: i32, seqs: *const i32, n_new: i32,
        k_new: *const c_void, k_strides: *const i64, v_new: *const c_void, v_strides: *const i64,
        dtype: i32, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_append_rope(
        cache: *mut b200kv_cache, n_seqs: i32, seqs: *const i32, n_new: i32,
        k_new: *const c_void, k_strides: *const i64, v_new: *const c_void, v_strides: *const i64,
        cos: *const c_void, sin: *const c_void, rope_strides: *const i64, dtype: i32, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_rope(
        x: *const c_void, x_strides: *const i64, cos: *const c_void, sin: *const c_void, rope_strides: *const i64,
        out: *mut c_void, out_strides: *const i64, batch: i32, n_heads: i32, n_tokens: i32, head_dim: i32,
        dtype: i32, stream: *mut c_void,
    ) -> c_int;

    // ---- attention over the cache ----
    pub fn b200kv_attend(
        cache: *mut b200kv_cache, n_seqs: i32, seqs: *const i32, n_q_heads: i32, n_new: i32,
        q: *const c_void, q_strides: *const i64, out: *mut c_void, out_strides: *const i64,
        dtype: i32, scale: c_float, causal: i32, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_append_attend(
        cache: *mut b200kv_cache, n_seqs: i32, seqs: *const i32, n_new: i32,
        k_new: *const c_void, k_strides: *const i64, v_new: *const c_void, v_strides: *const i64,
        n_q_heads: i32, q: *const c_void, q_strides: *const i64, out: *mut c_void, out_strides: *const i64,
        dtype: i32, scale: c_float, causal: i32, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_attend_window(
        cache: *mut b200kv_cache, n_seqs: i32, seqs: *const i32, n_q_heads: i32,
        q: *const c_void, q_strides: *const i64, out: *mut c_void, out_strides: *const i64,
        dtype: i32, scale: c_float, window: i64, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_attend_rope(
        cache: *mut b200kv_cache, n_seqs: i32, seqs: *const i32, n_q_heads: i32,
        q: *const c_void, q_strides: *const i64, cos: *const c_void, sin: *const c_void, rope_stride: i64,
        out: *mut c_void, out_strides: *const i64, dtype: i32, scale: c_float, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_attend_q40(
        cache: *mut b200kv_cache, n_seqs: i32, seqs: *const i32, n_q_heads: i32,
        q: *const c_void, q_strides: *const i64, cos: *const c_void, sin: *const c_void, rope_stride: i64,
        out: *mut c_void, out_strides: *const i64, scratch: *mut c_void, dtype: i32, scale: c_float,
        stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_attend_static_scratch(
        cache: *mut b200kv_cache, n_seqs: i32, seqs: *const i32, n_q_heads: i32,
        q: *const c_void, q_strides: *const i64, out: *mut c_void, out_strides: *const i64,
        dtype: i32, scale: c_float, stream: *mut c_void,
    ) -> c_int;

    // ---- state access ----
    pub fn b200kv_export(
        cache: *mut b200kv_cache, seq: i32, k_out: *mut c_void, k_strides: *const i64,
        v_out: *mut c_void, v_strides: *const i64, dtype: i32, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_export_codes(
        cache: *mut b200kv_cache, seq: i32, which: i32, codes: *mut c_void, scales: *mut c_void, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_export_kivi(
        cache: *mut b200kv_cache, seq: i32, which: i32, codes: *mut c_void, lo: *mut c_float, scale: *mut c_float,
        sink: *mut c_float, residual: *mut c_float, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_trim(cache: *mut b200kv_cache, seq: i32, keep_last: i64) -> c_int;
    pub fn b200kv_truncate(cache: *mut b200kv_cache, seq: i32, len: i64) -> c_int;
    pub fn b200kv_truncate_many(cache: *mut b200kv_cache, n_seqs: i32, seqs: *const i32, lens: *const i64) -> c_int;
    pub fn b200kv_fork(cache: *mut b200kv_cache, seq: i32, new_seq_out: *mut i32, stream: *mut c_void) -> c_int;
    pub fn b200kv_check(cache: *mut b200kv_cache, stream: *mut c_void) -> c_int;
    pub fn b200kv_profile(cache: *mut b200kv_cache, enable: i32) -> c_int;
    pub fn b200kv_profile_read(
        cache: *mut b200kv_cache, max_records: i32, kernel_ids: *mut i32, ms: *mut c_float, n_out: *mut i32,
    ) -> c_int;

    // ---- Q4_0 weights x activations ----
    pub fn b200kv_q40_packed_bytes(n: i64, k: i64) -> i64;
    pub fn b200kv_q40_pack(blocks: *const c_void, n: i64, k: i64, packed: *mut c_void, stream: *mut c_void) -> c_int;
    pub fn b200kv_q40_scratch_bytes(k: i64, m: i32) -> i64;
    pub fn b200kv_q40_gemm(
        packed: *const c_void, n: i64, k: i64, a: *const c_void, a_stride: i64, m: i32, dtype: i32,
        scratch: *mut c_void, out: *mut c_float, out_stride: i64, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_q40_quantize(
        a: *const c_void, a_stride: i64, m: i32, dtype: i32, k: i64, scratch: *mut c_void, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_q40_gemm_quantized(
        packed: *const c_void, n: i64, k: i64, m: i32, scratch: *mut c_void, out: *mut c_float, out_stride: i64,
        stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_q40_gemm_quantized_as(
        packed: *const c_void, n: i64, k: i64, m: i32, scratch: *mut c_void, out: *mut c_void, out_stride: i64,
        out_dtype: i32, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_q40_silu_mul_quantize(
        gate: *const c_void, gate_stride: i64, up: *const c_void, up_stride: i64, m: i32, dtype: i32, k: i64,
        scratch: *mut c_void, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_q40_add_rms_norm_quantize(
        x: *const c_float, x_stride: i64, residual: *const c_float, residual_stride: i64, weight: *const c_float,
        eps: c_float, x_out: *mut c_float, x_out_stride: i64, m: i32, k: i64, scratch: *mut c_void, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_q40_check(scratch: *const c_void, stream: *mut c_void) -> c_int;

    // ---- decoder glue ----
    pub fn b200kv_rms_norm(
        x: *const c_void, x_stride: i64, weight: *const c_void, out: *mut c_void, out_stride: i64, rows: i64, d: i32,
        eps: c_float, dtype: i32, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_silu_mul(gate: *const c_void, up: *const c_void, out: *mut c_void, n: i64, dtype: i32, stream: *mut c_void) -> c_int;
    pub fn b200kv_add(a: *const c_void, b: *const c_void, out: *mut c_void, n: i64, dtype: i32, stream: *mut c_void) -> c_int;
    pub fn b200kv_argmax(x: *const c_float, stride: i64, rows: i64, n: i32, out: *mut i32, stream: *mut c_void) -> c_int;
    pub fn b200kv_gather_rows(
        table: *const c_void, n_rows_table: i64, row_bytes: i64, ids: *const i32, n_ids: i64, out: *mut c_void,
        stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_cast(
        src: *const c_void, src_stride: i64, src_dtype: i32, dst: *mut c_void, dst_stride: i64, dst_dtype: i32,
        rows: i64, cols: i64, stream: *mut c_void,
    ) -> c_int;

    // ---- lone Sdpa ----
    pub fn b200kv_sdpa(
        q: *const c_void, q_strides: *const i64, k: *const c_void, k_strides: *const i64,
        v: *const c_void, v_strides: *const i64, mask: *const c_void, mask_strides: *const i64, mask_dtype: i32,
        out: *mut c_void, out_strides: *const i64, batch: i32, n_q_heads: i32, n_kv_heads: i32,
        q_len: i32, kv_len: i32, head_dim: i32, dtype: i32, scale: c_float, causal: i32, stream: *mut c_void,
    ) -> c_int;
    pub fn b200kv_sdpa_check(stream: *mut c_void) -> c_int;
}

/// Turns a status code into a `TractResult`, carrying the library's thread-local message.
pub fn ck(rc: c_int) -> tract_core::internal::TractResult<()> {
    if rc == B200KV_OK {
        return Ok(());
    }
    let msg = unsafe { std::ffi::CStr::from_ptr(b200kv_last_error()) }.to_string_lossy().into_owned();
    tract_core::internal::bail!("b200kv: {msg}")
}
