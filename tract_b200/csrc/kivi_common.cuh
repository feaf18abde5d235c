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

// lo + code * scale, multiply then add (quant_dyn_kv_cache.rs:141-146, :231-240)
__device__ inline float kivi_dequant(uint32_t code, float lo, float scale) { return __fadd_rn(lo, __fmul_rn((float)code, scale)); }

KiviView kivi_view(const b200kv_cache* c);

}  // namespace b200kv
