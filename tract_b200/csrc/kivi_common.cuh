// Geometry of the device form of tract's QuantizedDynKeyValueCache stores, shared by the append / export kernels
// and the two decode kernels.
#pragma once
#include "internal.h"

namespace b200kv {

constexpr int SINK = 4;     // SINK_TOKENS
constexpr int KBLOCK = 32;  // KEY_BLOCK

struct KiviView {  // device pointers + geometry, passed by value to the kernels
    uint8_t* codes[2];   // [n_pages][H][64][row_bytes] per stream
    float* params[2];    // per-token stream: [n_pages][H][64][2] ; per-channel stream: [n_pages][H][2 blocks][2][D]
    float* sinks;        // [max_seqs][H][2 streams][SINK][D]
    float* residual;     // [max_seqs][H][2 streams][KBLOCK][D]  (used by per-channel streams)
    const int32_t* table;
    int32_t max_pages_per_seq, n_pages, H, D, bits, row_bytes, n_streams;
    int32_t per_channel[2];
};


// At head_dim 128 the codes of a (page, head) lie exactly like the data region of a block-quantised chunk (common.cuh):
// int8 like Q8_1, int4 like Q4_0 -- 16-byte units XOR-swizzled per 128-byte line, V rows in the permuted channel order,
// int4 nibbles paired as that format pairs them -- so that the tensor-core decode kernel builds its fragments from
// contiguous bytes without bank conflicts.  The order the reference packs (quant_dyn_kv_cache.rs:63-75) is restored by
// the export kernels.  head_dim 64 keeps natural rows.
__host__ __device__ inline bool kivi_mma_layout(int bits, int D) { return D == 128 && (bits == 8 || bits == 4); }
__host__ __device__ constexpr int kivi_layout_fmt(int bits) { return bits == 8 ? B200KV_FMT_Q8_1 : B200KV_FMT_Q4_0; }
__device__ inline uint32_t kivi_code_offset(int bits, int stream, int slot, int c) {
    const int fmt = kivi_layout_fmt(bits);
    return chunk_addr(fmt, 128, stream, slot, code_pos(fmt, 128, stream, c));
}

// A code (below 2^23) as f32, exactly, without the conversion unit: 0x4B000000 | code is the float 2^23 + code.
__device__ inline float kivi_code_f32(uint32_t code) { return __fsub_rn(__uint_as_float(0x4B000000u | code), 8388608.f); }
// lo + code * scale, multiply then add (quant_dyn_kv_cache.rs:141-146, :231-240)
__device__ inline float kivi_dequant(uint32_t code, float lo, float scale) { return __fadd_rn(lo, __fmul_rn(kivi_code_f32(code), scale)); }

__device__ inline uint32_t kivi_load_code(const KiviView& v, int stream, int32_t pg, int h, int slot, int c) {
    if (kivi_mma_layout(v.bits, v.D)) {
        const uint32_t b = v.codes[stream][((int64_t)pg * v.H + h) * PAGE_TOKENS * v.row_bytes + kivi_code_offset(v.bits, stream, slot, c)];
        if (v.bits == 8) return b;
        return code_nibble(B200KV_FMT_Q4_0, 128, stream, c) ? (b >> 4) : (b & 0xf);
    }
    const uint8_t* row = v.codes[stream] + (((int64_t)pg * v.H + h) * PAGE_TOKENS + slot) * v.row_bytes;
    if (v.bits == 8) return row[c];
    const uint32_t b = row[c >> 1];
    return (c & 1) ? (b >> 4) : (b & 0xf);
}

// Element c of token t (0 .. len-1) of head h of one stream, as dequant_all gives it (quant_dyn_kv_cache.rs:132-148,
// :222-249): the f32 sinks, quantised rows as lo + code * scale, the f32 residual rows of a per-channel stream verbatim.
__device__ inline float kivi_elem(const KiviView& v, int32_t seq, int64_t len, int stream, int h, int64_t t, int c) {
    if (t < SINK) return v.sinks[((((int64_t)seq * v.H + h) * 2 + stream) * SINK + t) * v.D + c];
    const int64_t i = t - SINK;
    const int32_t pg = v.table[(int64_t)seq * v.max_pages_per_seq + i / PAGE_TOKENS];
    const int slot = (int)(i % PAGE_TOKENS);
    if (v.per_channel[stream]) {
        const int64_t n_fin = (len - SINK) / KBLOCK;
        if (i >= n_fin * KBLOCK) return v.residual[((((int64_t)seq * v.H + h) * 2 + stream) * KBLOCK + i % KBLOCK) * v.D + c];
        const float* par = v.params[stream] + (((int64_t)pg * v.H + h) * 2 + slot / KBLOCK) * 2 * v.D;
        return kivi_dequant(kivi_load_code(v, stream, pg, h, slot, c), par[c], par[v.D + c]);
    }
    const float* par = v.params[stream] + (((int64_t)pg * v.H + h) * PAGE_TOKENS + slot) * 2;
    return kivi_dequant(kivi_load_code(v, stream, pg, h, slot, c), par[0], par[1]);
}

KiviView kivi_view(const b200kv_cache* c);

}  // namespace b200kv
