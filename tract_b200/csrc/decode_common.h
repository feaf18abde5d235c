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
    int32_t first;       // first visible token: a sliding window, or a sequence whose front pages were given back (0: all)
    int32_t pad1;
};

struct DecodeParams {
    const uint8_t* pool;
    const int32_t* table;
    const WorkItem* items;
    int* status;
    const void* q;
    int64_t qb, qh;  // q strides {batch, head} in elements
    // ApplyRope on the query as it is loaded (null: q is used as it is): rows of D values of type dtype, one per batch entry
    const void* q_cos;
    const void* q_sin;
    int64_t rope_b;  // cos / sin stride between batch entries, in elements
    float* part_o;   // [item][Hkv][G][D]   unnormalised partial outputs
    float* part_ml;  // [item][Hkv][G][2]   running max (natural-log units), running sum
    int64_t page_bytes;
    int32_t n_pages, max_pages_per_seq, Hkv, G, dtype;
    float scale;
    uint64_t wait_ns = 1000000000ull;  // limit of each bounded barrier wait
    int32_t stall_item = -1;  // -1, or (a test hook) the work item whose CTA of kv head 0 never issues its copies: its first wait
                         // runs out, it flags STATUS_WAIT_EXPIRED, publishes an empty partial and returns
    int32_t pad0 = 0;
};

// Per-call batch description small enough to travel as a kernel parameter (no host-to-device copy, no
// staging slot): one entry per sequence of the call, {page-table row, cached length, first work item,
// number of splits}.  The work items are a pure function of it: split k of a sequence with `pages` pages
// covers pages [k * base + min(k, rem), ...) where base = pages / splits, rem = pages % splits.
constexpr int INLINE_BATCH = 256;
constexpr int MAX_SPLITS = 64;  // most partials per sequence the combine pass merges
struct InlineBatch {
    int32_t n;  // entries in use; 0 = the kernels read p.items / batch_info from device memory instead
    int32_t pad[3];
    int4 ent[INLINE_BATCH];
    int32_t first[INLINE_BATCH];  // first visible token of each entry (0: the whole sequence)
};

// Channel `ch` of the query row of (batch, head), after ApplyRope when the call carries cos / sin.  The rotated value is
// rounded to dtype after every operation, so it equals what a separate rope kernel would have stored and this load
// would have read back.
__device__ inline float load_query(const DecodeParams& p, int D, int batch, int head, int ch) {
    const int64_t row = (int64_t)batch * p.qb + (int64_t)head * p.qh;
    if (!p.q_cos) return ld_as_f32(p.q, p.dtype, row + ch);
    const int esz = p.dtype == B200KV_F32 ? 4 : 2;
    return rope_row_elem((const uint8_t*)p.q + row * esz, (const uint8_t*)p.q_cos + (int64_t)batch * p.rope_b * esz,
                         (const uint8_t*)p.q_sin + (int64_t)batch * p.rope_b * esz, p.dtype, D, ch);
}

__host__ __device__ inline WorkItem make_work_item(const int4& e, int batch, int k, int first = 0) {
    const int p0 = first / PAGE_TOKENS;  // pages before the first visible token are not walked (they may have been freed)
    const int pages = (e.y + PAGE_TOKENS - 1) / PAGE_TOKENS - p0;
    const int base = pages / e.w, rem = pages % e.w;
    WorkItem w;
    w.trow = e.x, w.len = e.y;
    w.page_begin = p0 + k * base + (k < rem ? k : rem);
    w.n_pages = base + (k < rem ? 1 : 0);
    w.batch = batch, w.split = k, w.first = first, w.pad1 = 0;
    return w;
}
// Work item `item` of an inline batch: binary search for the sequence that owns it.
__device__ inline WorkItem resolve_work_item(const InlineBatch& ib, int item) {
    int lo = 0, hi = ib.n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (ib.ent[mid].z <= item) lo = mid;
        else hi = mid - 1;
    }
    return make_work_item(ib.ent[lo], lo, item - ib.ent[lo].z, ib.first[lo]);
}

// decode.cu
int launch_decode_simt(int fmt, int D, const DecodeParams& p, int n_items, cudaStream_t stream, const InlineBatch* ib = nullptr);
int launch_combine(const DecodeParams& p, const int32_t* batch_info, void* out, int64_t ob, int64_t oh, int n_seqs,
                   int n_q_heads, int D, cudaStream_t stream, const InlineBatch* ib = nullptr);
// decode_mma.cu
bool decode_mma_supported(int fmt, int D, int dtype);
int launch_decode_mma(int fmt, const DecodeParams& p, int n_items, cudaStream_t stream, const InlineBatch* ib = nullptr);
// An InlineBatch with n = 0, for launches that read their batch from device memory.
const InlineBatch& empty_inline_batch();

}  // namespace b200kv
