// Launch parameters shared by the two decode kernels (CUDA-core and tensor-core formulations).
#pragma once
#include "internal.h"

namespace b200kv {

struct WorkItem {
    int32_t trow;        // page-table row of the sequence
    int32_t len;         // cached length of the sequence
    int32_t page_begin;  // first page of this split
    int32_t n_pages;     // pages in this split
    int32_t batch;       // batch entry
    int32_t split;       // split index inside the batch entry
    int32_t pad0, pad1;
};

struct DecodeParams {
    const uint8_t* pool;
    const int32_t* table;
    const WorkItem* items;
    int* status;
    const void* q;
    int64_t qb, qh;  // q strides {batch, head} in elements
    float* part_o;   // [item][Hkv][G][D]   unnormalised partial outputs
    float* part_ml;  // [item][Hkv][G][2]   running max (natural-log units), running sum
    int64_t page_bytes;
    int32_t n_pages, max_pages_per_seq, Hkv, G, dtype;
    float scale;
};

// decode.cu
int launch_decode_simt(int fmt, int D, const DecodeParams& p, int n_items, cudaStream_t stream);
int launch_combine(const DecodeParams& p, const int32_t* batch_info, void* out, int64_t ob, int64_t oh, int n_seqs,
                   int n_q_heads, int D, cudaStream_t stream);
// decode_mma.cu
bool decode_mma_supported(int fmt, int D, int dtype);
int launch_decode_mma(int fmt, const DecodeParams& p, int n_items, cudaStream_t stream);

}  // namespace b200kv
