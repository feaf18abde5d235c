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


// int8 codes at head_dim 128 lie in the (page, head) region exactly like the data region of a Q8_1 chunk
// (common.cuh: 16-byte units XOR-swizzled per 128-byte token line, V rows in the permuted channel order), so that the
// tensor-core decode kernel builds its fragments from contiguous bytes without bank conflicts.  Everything else
// keeps natural rows.
__host__ __device__ inline bool kivi_mma_layout(int bits, int D) { return bits == 8 && D == 128; }
__device__ inline uint32_t kivi_code_offset(int stream, int slot, int c) {
    return chunk_addr(B200KV_FMT_Q8_1, 128, stream, slot, code_pos(B200KV_FMT_Q8_1, 128, stream, c));
}

KiviView kivi_view(const b200kv_cache* c);

}  // namespace b200kv
