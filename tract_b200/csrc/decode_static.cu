// b200kv_attend_static_scratch: decode attention whose split-KV partials live in a fixed device array
// instead of the cache's growable workspace.
//
// Some callers must not trigger a device allocation while they run a step: a serving loop that has
// handed all free HBM to its page pools, a plan whose device arena was sized once up front and that
// treats any later cudaMalloc as a bug, or code that runs where an implicit device synchronisation
// (which cudaMalloc / cudaFree imply) would stall every other stream.  b200kv_attend keeps its split
// partials in a workspace that b200kv_create allocates; this entry point needs no device memory of
// the cache's own beyond the pages: it runs the same kernels, only the partials go to
// g_decode_scratch below, which every GPU that loads this library holds from load until exit.
#include <cmath>
#include <cstring>
#include <mutex>

#include "decode_common.h"

namespace b200kv {

// 8 MiB per GPU.  One partial is (head_dim + 2) floats; a call needs items x n_kv_heads x group of them,
// where items = total number of page runs of the batch (at most 64 per sequence).
constexpr size_t STATIC_SCRATCH_FLOATS = 2u << 20;
static __device__ __align__(256) float g_decode_scratch[STATIC_SCRATCH_FLOATS];

// Device address of g_decode_scratch per device ordinal.  In host code the symbol's name is only a
// stand-in; the address a kernel can use comes from cudaGetSymbolAddress, asked once per device with
// that device current.
constexpr int MAX_DEVICES = 64;
static float* g_scratch_ptr[MAX_DEVICES];
static std::mutex g_scratch_mu;

static int static_scratch(int device, float** out) {
    if (device < 0 || device >= MAX_DEVICES) return fail("device ordinal %d out of range", device);
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (!g_scratch_ptr[device]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_decode_scratch);  // the cache's device is current here
        if (e != cudaSuccess || !ptr) return fail("cudaGetSymbolAddress(g_decode_scratch) failed: %s", cudaGetErrorString(e));
        g_scratch_ptr[device] = (float*)ptr;
    }
    *out = g_scratch_ptr[device];
    return B200KV_OK;
}

}  // namespace b200kv

using namespace b200kv;

extern "C" int b200kv_attend_static_scratch(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads,
                                            const void* q, const int64_t q_strides[3], void* out,
                                            const int64_t out_strides[3], int32_t dtype, float scale, void* stream_) {
    if (validate_seqs(c, n_seqs, seqs) != B200KV_OK) return B200KV_KO;
    if (!c->L.has_v) return fail("this cache holds one tensor only: attention needs K and V");
    if (fmt_is_kivi(c->L.fmt))
        return fail("a KIVI cache (format %d) has decode kernels of its own, which this entry point does not run: use b200kv_attend", c->L.fmt);
    if (!q || !out || !q_strides || !out_strides) return fail("null tensor or strides");
    if (n_q_heads <= 0 || n_q_heads % c->L.Hkv != 0)
        return fail("n_q_heads (%d) must be a positive multiple of n_kv_heads (%d)", n_q_heads, c->L.Hkv);
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if (scale <= 0.f) scale = 1.0f / sqrtf((float)c->L.D);
    cudaStream_t stream = (cudaStream_t)stream_;
    DeviceGuard guard(c->cfg.device);

    const int Hkv = c->L.Hkv, D = c->L.D, G = n_q_heads / Hkv;
    const bool use_mma = decode_mma_supported(c->L.fmt, D, dtype) && !c->force_simt;
    const int GT = use_mma ? 8 : (G == 1 ? 1 : 4), nz = (G + GT - 1) / GT;
    int64_t total_pages = 0;
    for (int i = 0; i < n_seqs; i++) {
        if (c->seqs[seqs[i]].start > 0) return fail("sequence %d was trimmed: use b200kv_attend or b200kv_attend_window", seqs[i]);
        const int64_t len = c->seqs[seqs[i]].len;
        if (len <= 0) return fail("sequence %d is empty: nothing to attend to", seqs[i]);
        total_pages += (len + PAGE_TOKENS - 1) / PAGE_TOKENS;
    }
    int64_t chunk = decode_pages_per_split(c, n_seqs, seqs, 0, use_mma, nz);
    // size the work list first, so that nothing is enqueued when the fixed array is too small
    size_t n_items = 0;
    for (int i = 0; i < n_seqs; i++) {
        const int64_t pages = (c->seqs[seqs[i]].len + PAGE_TOKENS - 1) / PAGE_TOKENS;
        int64_t splits = (pages + chunk - 1) / chunk;
        n_items += (size_t)(splits > 64 ? 64 : splits);
    }
    const size_t n_part = n_items * (size_t)Hkv * G;
    const size_t need = n_part * (size_t)(D + 2);
    if (need > STATIC_SCRATCH_FLOATS)
        return fail("this call needs %zu floats of split partials (%zu page runs x %d kv heads x %d q heads per kv head x "
                    "(%d + 2)); the fixed scratch array holds %zu: use b200kv_attend, or fewer sequences per call",
                    need, n_items, Hkv, G, D, (size_t)STATIC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (static_scratch(c->cfg.device, &scratch) != B200KV_OK) return B200KV_KO;

    // work list written straight into the pinned descriptor slot (no host containers)
    const size_t items_bytes = n_items * sizeof(WorkItem);
    const size_t desc_bytes = items_bytes + (size_t)n_seqs * 8;
    int slot;
    uint8_t *h, *d;
    if (staging_acquire(c, desc_bytes, &slot, &h, &d) != B200KV_OK) return B200KV_KO;
    WorkItem* items = (WorkItem*)h;
    int32_t* info = (int32_t*)(h + items_bytes);
    size_t at = 0;
    for (int i = 0; i < n_seqs; i++) {
        const SeqState& s = c->seqs[seqs[i]];
        const int pages = (int)((s.len + PAGE_TOKENS - 1) / PAGE_TOKENS);
        int64_t sp = (pages + chunk - 1) / chunk;
        const int splits = (int)(sp > 64 ? 64 : sp);
        info[2 * i] = (int32_t)at;
        info[2 * i + 1] = splits;
        int begin = 0;
        for (int k = 0; k < splits; k++) {
            const int n = (pages - begin + (splits - k) - 1) / (splits - k);
            items[at++] = WorkItem{seqs[i], (int32_t)s.len, begin, n, i, k, 0, 0};
            begin += n;
        }
    }
    if (staging_upload(c, slot, desc_bytes, stream) != B200KV_OK) {
        staging_release(c, slot, stream);  // the slot goes back to the ring; nothing that reads it was enqueued
        return B200KV_KO;
    }

    DecodeParams p{};
    p.pool = c->pool, p.table = c->d_table, p.items = (const WorkItem*)d, p.status = c->d_status;
    p.q = q, p.qb = q_strides[0], p.qh = q_strides[1];
    // every partial slot of this call is written by the decode kernel before the combine pass reads it,
    // so nothing has to be cleared: whatever the previous call left in the array is simply overwritten
    p.part_o = scratch;
    p.part_ml = scratch + n_part * D;
    p.page_bytes = c->L.page_bytes, p.n_pages = (int32_t)c->n_pages, p.max_pages_per_seq = c->max_pages_per_seq;
    p.Hkv = Hkv, p.G = G, p.dtype = dtype, p.scale = scale;
    p.wait_ns = c->wait_ns;
    int rc = use_mma ? launch_decode_mma(c->L.fmt, p, (int)n_items, stream)
                     : launch_decode_simt(c->L.fmt, D, p, (int)n_items, stream);
    if (rc == B200KV_OK)
        rc = launch_combine(p, (const int32_t*)(d + items_bytes), out, out_strides[0], out_strides[1], n_seqs, n_q_heads, D, stream);
    staging_release(c, slot, stream);
    return rc;
}
