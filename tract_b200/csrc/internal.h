// Host-side state of a cache handle and helpers shared by the translation units.
#pragma once
#include <cstdarg>
#include <cstdio>
#include <string>
#include <vector>

#include "common.cuh"

namespace b200kv {

// Thread-local message of the last failure (the analogue of tract's LAST_ERROR, api/ffi/src/lib.rs:27-60).
std::string& last_error();
int fail(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

#define B200KV_CUDA(call)                                                                          \
    do {                                                                                           \
        cudaError_t e__ = (call);                                                                  \
        if (e__ != cudaSuccess) return ::b200kv::fail("%s failed: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

struct SeqState {
    bool live = false;
    int64_t len = 0;
    int64_t start = 0;  // first token still held: the pages before start / 64 were given back by b200kv_trim (entries -1)
    std::vector<int32_t> pages;
};

// Ring of descriptor slots: each call that needs per-call metadata on the device writes it into a
// pinned host slot, enqueues one H2D copy into the matching device slot and records an event after
// the kernels that read it, so a slot is never rewritten while the GPU may still use it.
struct Staging {
    static constexpr int SLOTS = 16;
    size_t slot_bytes = 0;
    uint8_t* host = nullptr;
    uint8_t* dev = nullptr;
    cudaEvent_t ev[SLOTS] = {};
    bool used[SLOTS] = {};
    int next = 0;
};

}  // namespace b200kv

namespace b200kv {
// Stores of the KIVI formats (kivi.cu); null for every other format.
struct KiviStore {
    uint8_t* codes[2] = {nullptr, nullptr};
    float* params[2] = {nullptr, nullptr};
    float* sinks = nullptr;
    float* residual = nullptr;
    int bits = 0, row_bytes = 0, n_streams = 0;
    int per_channel[2] = {0, 0};
};
}  // namespace b200kv

struct b200kv_cache {
    b200kv_config cfg;
    b200kv::KiviStore kivi;
    b200kv::Layout L;
    int64_t n_pages = 0;
    int max_pages_per_seq = 0;
    uint8_t* pool = nullptr;
    int32_t* d_table = nullptr;  // [max_seqs][max_pages_per_seq] page ids
    int* d_status = nullptr;
    std::vector<int32_t> free_pages;
    std::vector<b200kv::SeqState> seqs;
    b200kv::Staging st;
    uint8_t* ws = nullptr;  // split-KV partials: allocated once at create, never grown
    size_t ws_bytes = 0;
    uint64_t wait_ns = 1000000000ull;  // limit of every bounded barrier wait of the decode kernels
    bool stall_next_decode = false;    // test hook: the next decode launch leaves one CTA waiting for a copy nobody issued
    // optional per-launch timing (the analogue of tract-cuda's event pairs around every launch,
    // cuda/src/context.rs:364-453): off by default
    bool kivi_cuda_core = false;  // test hook: KIVI decode through the CUDA-core kernel alone
    bool force_simt = false;  // test hook: route decode through the CUDA-core kernel even where the tensor-core one applies
    bool prof_on = false;
    struct ProfRec {
        int id;
        cudaEvent_t a, b;
    };
    std::vector<ProfRec> prof;
};

namespace b200kv {

// Reserves a descriptor slot (blocking only if the ring wrapped onto a slot still in flight).
int staging_acquire(b200kv_cache* c, size_t bytes, int* slot, uint8_t** host, uint8_t** dev);
// Copies the first `bytes` of the slot to the device on `stream`.
int staging_upload(b200kv_cache* c, int slot, size_t bytes, cudaStream_t stream);
// Marks the slot as consumed by everything enqueued on `stream` so far.
int staging_release(b200kv_cache* c, int slot, cudaStream_t stream);
// Partial records the split-KV workspace of a configuration holds (it is allocated once, by b200kv_create).
int64_t workspace_records(const b200kv_config& cfg);

int validate_seqs(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs);

// Kernel ids reported by b200kv_profile_read.
enum { K_SCATTER = 0, K_APPEND = 1, K_DECODE = 2, K_COMBINE = 3, K_EXPORT = 4, K_DENSE = 5, K_PREFILL = 6 };

// Brackets the launches made during its lifetime with an event pair when profiling is on.
struct ProfScope {
    b200kv_cache* c;
    cudaStream_t stream;
    b200kv_cache::ProfRec rec{};
    bool live = false;
    ProfScope(b200kv_cache* c_, int id, cudaStream_t s) : c(c_), stream(s) {
        if (!c || !c->prof_on) return;
        if (cudaEventCreate(&rec.a) != cudaSuccess || cudaEventCreate(&rec.b) != cudaSuccess) return;
        rec.id = id;
        cudaEventRecord(rec.a, stream);
        live = true;
    }
    ~ProfScope() {
        if (!live) return;
        cudaEventRecord(rec.b, stream);
        c->prof.push_back(rec);
    }
};

// decode.cu
struct QueryRope {  // what a decode call may fold in at its two ends
    const void* cos;   // ApplyRope of the query inside the decode kernels: one cos / sin row of D values per batch entry, or null
    const void* sin;
    int64_t stride_b;  // elements
    void* act_scratch; // the result also (or only) as the quantised activation of a W4A8 GEMM, or null
};
int64_t decode_pages_per_split(const b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int64_t window, bool use_mma, int nz);
int launch_decode(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, const void* q,
                  const int64_t* q_strides, void* out, const int64_t* out_strides, int32_t dtype, float scale,
                  cudaStream_t stream, int64_t window = 0, const QueryRope* rope = nullptr);
// sdpa_dense.cu
int launch_sdpa_dense(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                      const int64_t* vs, const void* mask, const int64_t* ms, int mask_dtype, void* out,
                      const int64_t* os, int B, int Hq, int Hkv, int S, int T, int D, int dtype, int kv_dtype,
                      float scale, int causal, cudaStream_t stream);
int launch_sdpa_paged(b200kv_cache* c, int32_t seq, const void* q, const int64_t* qs, void* out, const int64_t* os, int Hq, int S,
                      int dtype, float scale, int causal, cudaStream_t stream);
// kivi.cu
bool fmt_is_kivi(int fmt);
int kivi_create(b200kv_cache* c);
void kivi_destroy(b200kv_cache* c);
int64_t kivi_page_bytes(const b200kv_cache* c);
int64_t kivi_pages_for(int64_t len);
int kivi_append(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_new, const void* k_new, const int64_t* ks,
                const void* v_new, const int64_t* vs, int32_t dtype, const int32_t* d_desc, cudaStream_t stream);
int kivi_export(b200kv_cache* c, int32_t seq, void* k_out, const int64_t* ks, void* v_out, const int64_t* vs, int32_t dtype,
                cudaStream_t stream);
int kivi_fork(b200kv_cache* c, int32_t src, int32_t dst, cudaStream_t stream);
int kivi_decode(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, const void* q, const int64_t* qs, void* out,
                const int64_t* os, int32_t dtype, float scale, cudaStream_t stream);
// prefill_tc.cu
bool prefill_tc_supported(const b200kv_cache* c, int n_q_heads, int dtype, const void* q, const int64_t* qs, const void* out,
                          const int64_t* os);
int launch_prefill_tc(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, int32_t n_new, const void* q,
                      const int64_t* qs, void* out, const int64_t* os, int32_t dtype, float scale, int causal,
                      cudaStream_t stream);
// attn_tc.cu
bool attn_tc_supported(const b200kv_cache* c, int n_q_heads, int dtype, const void* q, const int64_t* qs, const void* out, const int64_t* os);
int launch_attn_tc_paged(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_q_heads, int32_t n_new, const void* q, const int64_t* qs,
                         void* out, const int64_t* os, int32_t dtype, float scale, int causal, cudaStream_t stream);
bool attn_tc_dense_supported(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v, const int64_t* vs,
                             const void* mask, int mask_dtype, const void* out, const int64_t* os, int B, int Hq, int Hkv, int S, int T, int D,
                             int dtype, int causal);
int launch_attn_tc_dense(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v, const int64_t* vs, const void* mask,
                         const int64_t* ms, int mask_dtype, void* out, const int64_t* os, int B, int Hq, int Hkv, int S, int T, int D, int dtype,
                         float scale, int causal, int* status, cudaStream_t stream);
// cache.cu
int launch_export(b200kv_cache* c, int32_t seq, void* k_out, const int64_t* ks, void* v_out, const int64_t* vs,
                  int32_t dtype, cudaStream_t stream);

// q40_tc.cu: the W4A8 GEMM for Q_TC_MIN_ROWS activation rows and more, on tcgen05
int launch_q40_gemm_tc(const void* packed, const void* act, void* out, int* status, int64_t n, int64_t nb, int64_t out_stride, int32_t m,
                       int32_t out_dtype, cudaStream_t stream);

}  // namespace b200kv
