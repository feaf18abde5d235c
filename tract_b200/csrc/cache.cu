// Cache handle (page pool, page tables, descriptor ring) and the append / export kernels.
//
// Replaces GpuDynKVCacheState::eval (gpu/src/ops/dyn_kv_cache.rs:58-113), which allocates a fresh
// [.., P+S, ..] tensor and copies the whole past every step, by an in-place paged append that
// touches only the S new tokens; and gives QuantizedDynKvCacheState::ingest
// (transformers/src/ops/quant_dyn_kv_cache.rs:403-430) a device form for the block-32 formats,
// with the arithmetic of linalg/src/frame/block_quant/{q8_1.rs:20-48, q4_0.rs:19-45} done with
// explicitly rounded IEEE operations so that codes and scales are bit-identical to the CPU's.
#include <algorithm>
#include <cstring>

#include "internal.h"

namespace b200kv {

std::string& last_error() {
    static thread_local std::string e;
    return e;
}
int fail(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    last_error() = buf;
    return B200KV_KO;
}

// ---- descriptor ring ---------------------------------------------------------------------------
int staging_acquire(b200kv_cache* c, size_t bytes, int* slot, uint8_t** host, uint8_t** dev) {
    Staging& s = c->st;
    if (bytes > s.slot_bytes) return fail("call descriptor of %zu bytes exceeds the %zu-byte slot", bytes, s.slot_bytes);
    int i = s.next;
    s.next = (s.next + 1) % Staging::SLOTS;
    if (s.used[i]) B200KV_CUDA(cudaEventSynchronize(s.ev[i]));
    s.used[i] = false;
    *slot = i;
    *host = s.host + (size_t)i * s.slot_bytes;
    *dev = s.dev + (size_t)i * s.slot_bytes;
    return B200KV_OK;
}
int staging_upload(b200kv_cache* c, int slot, size_t bytes, cudaStream_t stream) {
    Staging& s = c->st;
    B200KV_CUDA(cudaMemcpyAsync(s.dev + (size_t)slot * s.slot_bytes, s.host + (size_t)slot * s.slot_bytes, bytes,
                                cudaMemcpyHostToDevice, stream));
    return B200KV_OK;
}
int staging_release(b200kv_cache* c, int slot, cudaStream_t stream) {
    B200KV_CUDA(cudaEventRecord(c->st.ev[slot], stream));
    c->st.used[slot] = true;
    return B200KV_OK;
}
// Partial records (one per page run, kv head and query head of its group) the split-KV workspace is sized for.
// A decode launch aims at 148 x 16 CTAs, each of which publishes at most 8 records (decode_pages_per_split), and every
// sequence adds at most one run of its own to that: 148 * 16 * 8 + max_seqs * max_q_heads covers the natural split of
// every call; a call that would need more (more query heads than announced) takes longer runs instead.
int64_t workspace_records(const b200kv_config& cfg) {
    const int64_t hq = cfg.max_q_heads > 0 ? cfg.max_q_heads : 8 * (int64_t)cfg.n_kv_heads;
    return 148 * 16 * 8 + 2 * (int64_t)cfg.max_seqs * ((hq + 7) / 8 * 8);
}
int validate_seqs(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs) {
    if (!c) return fail("null cache");
    if (n_seqs <= 0 || !seqs) return fail("need at least one sequence");
    for (int i = 0; i < n_seqs; i++) {
        int s = seqs[i];
        if (s < 0 || s >= (int)c->seqs.size() || !c->seqs[s].live) return fail("sequence %d is not live", s);
        for (int j = 0; j < i; j++)
            if (seqs[j] == s) return fail("sequence %d appears twice in one call", s);
    }
    return B200KV_OK;
}

// ---- kernels ---------------------------------------------------------------------------------------

__global__ void table_scatter_kernel(int32_t* table, const int32_t* upd, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) table[upd[2 * i]] = upd[2 * i + 1];
}

struct AppendParams {
    uint8_t* pool;
    int32_t* table;
    const int32_t* desc;  // per batch entry: {table row, length before the append, offset of its first new page in
                          // `upd` (or -1), page number of that first new page}
    const int32_t* upd;   // (page-table index, page id) pairs of the pages this call allocated
    int32_t n_upd;
    int* status;
    const void* src[2];
    int64_t sb[2], sh[2], ss[2];
    int64_t page_bytes;
    int32_t n_pages, max_pages_per_seq;
    int32_t n_seqs, H, S, D;
    int32_t chunk_bytes, data_bytes, plane_w, units;  // units = 16-byte units per row
    int32_t dtype, vec_ok, has_v;
    // optional rotary embedding applied to K on the way in: cos / sin [n_seqs, S, D], strides {batch, token}
    const void* rope_cos;
    const void* rope_sin;
    int64_t rope_b, rope_s;
};

// Batch description of an append small enough to travel as a kernel parameter (no copy, no staging slot).
constexpr int INLINE_APPEND = 256;
struct InlineAppend {
    int32_t n;  // entries in use; 0 = read p.desc / p.upd from device memory
    int32_t pad[3];
    int4 ent[INLINE_APPEND];  // {table row, length before the append, offset of the first new page in upd or -1, its page number}
    int2 upd[INLINE_APPEND];  // (page-table index, page id) pairs
};

// Rust `x as i8` after f32::round / truncation: saturating, NaN -> 0.
__device__ inline int sat_i8_rz(float x) {
    int i = __float2int_rz(x);  // saturates to int32, NaN -> 0
    return max(-128, min(127, i));
}

// One thread per 16-byte unit of a token-head row.  grid.z = 2 * batch entry + (K or V); grid.x walks the (head, token,
// unit) triples of that entry, so that the index arithmetic is three 32-bit divisions and no 64-bit one.
template <int FMT>
__global__ void __launch_bounds__(256) append_kernel(AppendParams p, const __grid_constant__ InlineAppend ia) {
    constexpr int EPU = elems_in_bytes<FMT>(16);  // elements per unit
    const int kv = p.has_v ? (int)(blockIdx.z & 1) : 0;
    grid_launch_dependents();  // a decode launch that follows may be scheduled now; it waits for this grid before reading pages
    grid_dependency_wait();    // the kernel before has written k_new / v_new, and is done with the pages and the table
    if (blockIdx.x == 0 && blockIdx.z == 0)  // publish the new page-table entries (replaces a separate launch)
        for (int i = threadIdx.x; i < p.n_upd; i += blockDim.x) {
            const int2 u = ia.n ? ia.upd[i] : ((const int2*)p.upd)[i];
            p.table[u.x] = u.y;
        }
    const int b = p.has_v ? (int)(blockIdx.z >> 1) : (int)blockIdx.z;
    const uint32_t per_head = (uint32_t)p.S * (uint32_t)p.units, idx = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t hq = idx / per_head, rem = idx - hq * per_head;
    const bool valid = hq < (uint32_t)p.H;
    // lanes past the end stay alive for the shuffles below (their partner lanes are past the end as well): point them at the last row
    const int h = valid ? (int)hq : p.H - 1, s = valid ? (int)(rem / (uint32_t)p.units) : p.S - 1, u = (int)(idx % (uint32_t)p.units);
    const int c0 = u * EPU;

    // ---- load EPU input elements --------------------------------------------------------------
    const int esz = dtype_size(p.dtype);
    const uint8_t* src = (const uint8_t*)p.src[kv] + (b * p.sb[kv] + h * p.sh[kv] + s * p.ss[kv] + c0) * esz;
    uint4 out16 = make_uint4(0, 0, 0, 0);  // bit-copy formats: the 16 bytes this thread stores
    uint8_t codes[EPU > 16 ? EPU : 16];      // quantised formats: one code per element of the unit
    float scale_f = 0.f;
    bool write_scale = false;

    const bool rope = p.rope_cos != nullptr && kv == 0;
    const uint8_t* row0 = (const uint8_t*)p.src[kv] + (b * p.sb[kv] + h * p.sh[kv] + s * p.ss[kv]) * esz;  // channel 0 of the row
    const uint8_t* cos_row = (const uint8_t*)p.rope_cos + (b * p.rope_b + s * p.rope_s) * esz;
    const uint8_t* sin_row = (const uint8_t*)p.rope_sin + (b * p.rope_b + s * p.rope_s) * esz;
    if constexpr (FMT == B200KV_FMT_F32 || FMT == B200KV_FMT_F16 || FMT == B200KV_FMT_BF16) {
        // bit copy: storage type == input type (checked on the host)
        if (rope) {
            uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
            for (int i = 0; i < EPU; i++) {
                const float r = rope_row_elem(row0, cos_row, sin_row, p.dtype, p.D, c0 + i);
                if (FMT == B200KV_FMT_F32) w[i % 4] = __float_as_uint(r);
                else if (FMT == B200KV_FMT_F16) w[(i / 2) % 4] |= (uint32_t)__half_as_ushort(__float2half_rn(r)) << (16 * (i & 1));
                else w[(i / 2) % 4] |= (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(r)) << (16 * (i & 1));
            }
            out16 = make_uint4(w[0], w[1], w[2], w[3]);
        } else if (p.vec_ok) {
            out16 = *(const uint4*)src;
        } else {
            uint8_t tmp[16];
            for (int i = 0; i < 16; i += esz)
                for (int j = 0; j < esz; j++) tmp[i + j] = src[i + j];
            memcpy(&out16, tmp, 16);
        }
    } else {
        float v[EPU];
        if (rope) {
#pragma unroll
            for (int i = 0; i < EPU; i++) v[i] = rope_row_elem(row0, cos_row, sin_row, p.dtype, p.D, c0 + i);
        } else if (p.dtype == B200KV_F32) {
            if (p.vec_ok) {
#pragma unroll
                for (int i = 0; i < EPU / 4; i++) {
                    float4 f = ((const float4*)src)[i];
                    v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < EPU; i++) v[i] = ((const float*)src)[i];
            }
        } else if (p.vec_ok) {  // 16-bit input: 8 elements per 128-bit load
#pragma unroll
            for (int i = 0; i < EPU / 8; i++) {
                const uint4 w = ((const uint4*)src)[i];
                const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (p.dtype == B200KV_F16) {
                        const float2 f = __half22float2(*(const __half2*)&ws[j]);
                        v[8 * i + 2 * j] = f.x, v[8 * i + 2 * j + 1] = f.y;
                    } else {  // bf16 -> f32 is a shift
                        v[8 * i + 2 * j] = __uint_as_float(ws[j] << 16), v[8 * i + 2 * j + 1] = __uint_as_float(ws[j] & 0xffff0000u);
                    }
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < EPU; i++) v[i] = ld_as_f32(src, p.dtype, i);
        }
        // signed value of largest magnitude, first occurrence wins (strict <); NaN never wins
        float amax = 0.f, mx = 0.f;
#pragma unroll
        for (int i = 0; i < EPU; i++) {
            float a = fabsf(v[i]);
            if (amax < a) {
                amax = a;
                mx = v[i];
            }
        }
        if constexpr (FMT == B200KV_FMT_Q8_1) {
            // a block of 32 spans two units: combine with the neighbour lane, lower channels win ties
            float o_amax = __shfl_xor_sync(0xffffffffu, amax, 1);
            float o_mx = __shfl_xor_sync(0xffffffffu, mx, 1);
            bool take_other = (u & 1) ? !(o_amax < amax) : (amax < o_amax);
            if (take_other) mx = o_mx;
            float scale = __fdiv_rn(mx, 127.0f);
            float r = (scale == 0.f) ? 0.f : __fdiv_rn(1.0f, scale);
            // codes are stored offset-binary (code + 128) so that the decode kernel can widen them to
            // f16 with byte permutes only; b200kv_export_codes returns the two's-complement int8
#pragma unroll
            for (int i = 0; i < 16; i++)
                codes[i] = (uint8_t)((sat_i8_rz(roundf(__fmul_rn(v[i], r))) + 128) & 0xff);
            scale_f = scale;
            write_scale = (u & 1) == 0;
        } else {  // Q4_0: the unit is the whole block
            float scale = __fdiv_rn(mx, -8.0f);
            float r = (scale == 0.f) ? 0.f : __fdiv_rn(1.0f, scale);
#pragma unroll
            for (int j = 0; j < 16; j++) {
                int lo = min(sat_i8_rz(__fadd_rn(__fmul_rn(v[j], r), 8.5f)), 15);
                int hi = min(sat_i8_rz(__fadd_rn(__fmul_rn(v[j + 16], r), 8.5f)), 15);
                // The reference writes `lo as u8 | (hi as u8) << 4` without masking (helpers.rs:57-68): a
                // negative lo code (reachable only through an infinite reciprocal) spills its upper bits
                // into the high nibble.  Store the nibbles that byte would hold.
                codes[j] = (uint8_t)(lo & 0xf);
                codes[j + 16] = (uint8_t)((hi | (lo >> 4)) & 0xf);
            }
            scale_f = scale;
            write_scale = true;
        }
    }
    if (!valid) return;

    // ---- locate the page slot and store --------------------------------------------------------------
    const int4 ent = ia.n ? ia.ent[b] : ((const int4*)p.desc)[b];
    const int32_t trow = ent.x, len0 = ent.y, upd_off = ent.z, new_pn = ent.w;
    const int64_t pos = (int64_t)len0 + s;
    const int32_t pn = (int32_t)(pos / PAGE_TOKENS);
    // pages allocated by this very call are taken from the call descriptor: the table entries are written by
    // block 0 of this launch (above) for the kernels that follow, not for this one
    const int32_t pg = (upd_off >= 0 && pn >= new_pn)
                           ? (ia.n ? ia.upd[upd_off + pn - new_pn].y : p.upd[2 * (upd_off + pn - new_pn) + 1])
                           : p.table[(int64_t)trow * p.max_pages_per_seq + pn];
    if (pg < 0 || pg >= p.n_pages) {
        atomicOr(p.status, STATUS_PAGE_OOB);
        return;
    }
    const int t = (int)(pos % PAGE_TOKENS);
    uint8_t* chunk = p.pool + (int64_t)pg * p.page_bytes + (int64_t)(h * (p.has_v ? 2 : 1) + kv) * p.chunk_bytes;
    uint8_t* data = chunk;
    if constexpr (FMT == B200KV_FMT_F32 || FMT == B200KV_FMT_F16 || FMT == B200KV_FMT_BF16) {
        *(uint4*)(data + chunk_addr(FMT, p.D, kv, t, u * 16)) = out16;
    } else if constexpr (FMT == B200KV_FMT_Q8_1) {
        if (v_permuted(FMT, p.D, kv)) {
            // channels 16u + r and 16u + r + 8 sit side by side at position 16r + 2u
#pragma unroll
            for (int r = 0; r < 8; r++)
                *(uint16_t*)(data + chunk_addr(FMT, p.D, kv, t, r * 16) + 2 * u) =
                    (uint16_t)(codes[r] | ((uint16_t)codes[r + 8] << 8));
        } else {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++)
                w[i] = codes[4 * i] | (codes[4 * i + 1] << 8) | (codes[4 * i + 2] << 16) | ((uint32_t)codes[4 * i + 3] << 24);
            *(uint4*)(data + chunk_addr(FMT, p.D, kv, t, u * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {  // Q4_0, codes[i] = nibble of channel 32u + i
        if (v_permuted(FMT, p.D, kv)) {
            // byte 8r + j = channel 16j + r | channel 16j + r + 8 << 4 ; this block covers j = 2u, 2u + 1
#pragma unroll
            for (int r = 0; r < 8; r++) {
                uint32_t b0 = codes[r] | (codes[r + 8] << 4), b1 = codes[16 + r] | (codes[24 + r] << 4);
                *(uint16_t*)(data + chunk_addr(FMT, p.D, kv, t, r * 8) + 2 * u) = (uint16_t)(b0 | (b1 << 8));
            }
        } else {
            uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 16; j++) w[j / 4] |= (uint32_t)(codes[j] | (codes[j + 16] << 4)) << (8 * (j % 4));
            *(uint4*)(data + chunk_addr(FMT, p.D, kv, t, u * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    if (write_scale) {
        int blk = (FMT == B200KV_FMT_Q8_1) ? u / 2 : u;
        ((__half*)(chunk + p.data_bytes))[scale_index(FMT, p.D, kv, t, blk)] = __float2half_rn(scale_f);
    }
}

// The bit-copy formats without rotary embedding, aligned input: four units per thread, the four 16-byte loads issued
// before the first store so that a thread keeps 64 bytes in flight.  Same indexing as append_kernel.
template <int FMT>
__global__ void __launch_bounds__(256) append_copy_kernel(AppendParams p, const __grid_constant__ InlineAppend ia) {
    constexpr int REP = 4;
    const int kv = p.has_v ? (int)(blockIdx.z & 1) : 0;
    grid_launch_dependents();
    if (blockIdx.x == 0 && blockIdx.z == 0)
        for (int i = threadIdx.x; i < p.n_upd; i += blockDim.x) {
            const int2 u = ia.n ? ia.upd[i] : ((const int2*)p.upd)[i];
            p.table[u.x] = u.y;
        }
    const int b = p.has_v ? (int)(blockIdx.z >> 1) : (int)blockIdx.z;
    const uint32_t units = (uint32_t)p.units, per_head = (uint32_t)p.S * units;
    const int esz = dtype_size(p.dtype);
    const int4 ent = ia.n ? ia.ent[b] : ((const int4*)p.desc)[b];
    const int32_t trow = ent.x, len0 = ent.y, upd_off = ent.z, new_pn = ent.w;
    uint4 val[REP];
    int hh[REP], ss[REP], uu[REP];
    bool ok[REP];
#pragma unroll
    for (int r = 0; r < REP; r++) {
        const uint32_t idx = (blockIdx.x * REP + r) * blockDim.x + threadIdx.x;
        const uint32_t hq = idx / per_head, rem = idx - hq * per_head;
        ok[r] = hq < (uint32_t)p.H;
        hh[r] = (int)hq, ss[r] = (int)(rem / units), uu[r] = (int)(rem % units);
        if (ok[r])
            val[r] = *(const uint4*)((const uint8_t*)p.src[kv] + (b * p.sb[kv] + hh[r] * p.sh[kv] + ss[r] * p.ss[kv]) * esz + uu[r] * 16);
    }
#pragma unroll
    for (int r = 0; r < REP; r++) {
        if (!ok[r]) continue;
        const int64_t pos = (int64_t)len0 + ss[r];
        const int32_t pn = (int32_t)(pos / PAGE_TOKENS);
        const int32_t pg = (upd_off >= 0 && pn >= new_pn)
                               ? (ia.n ? ia.upd[upd_off + pn - new_pn].y : p.upd[2 * (upd_off + pn - new_pn) + 1])
                               : p.table[(int64_t)trow * p.max_pages_per_seq + pn];
        if (pg < 0 || pg >= p.n_pages) {
            atomicOr(p.status, STATUS_PAGE_OOB);
            continue;
        }
        uint8_t* chunk = p.pool + (int64_t)pg * p.page_bytes + (int64_t)(hh[r] * (p.has_v ? 2 : 1) + kv) * p.chunk_bytes;
        *(uint4*)(chunk + chunk_addr(FMT, p.D, kv, (int)(pos % PAGE_TOKENS), uu[r] * 16)) = val[r];
    }
}

struct ExportParams {
    const uint8_t* pool;
    const int32_t* table_row;  // page ids of the sequence
    void* dst[2];
    int64_t dh[2], dt[2];  // strides {head, token} in elements
    void* codes;           // raw export: codes / scales destinations (one of K, V)
    void* scales;
    int64_t page_bytes, len;
    int32_t H, D, chunk_bytes, data_bytes, plane_w, units, row_bytes;
    int32_t dtype, has_v, which;
};

// One thread per 16 bytes of the natural row; mode 0: dequantised / bit-copied elements,
// mode 1: raw codes (int8 two's complement / GGML nibble bytes) + scales.
template <int FMT, int MODE>
__global__ void __launch_bounds__(256) export_kernel(ExportParams p) {
    constexpr int EPU = elems_in_bytes<FMT>(16);
    const int kv = MODE == 1 ? p.which : blockIdx.y;
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t row = gid / p.units;
    const int u = (int)(gid % p.units);
    if (row >= (int64_t)p.H * p.len) return;
    const int h = (int)(row / p.len);
    const int64_t tok = row % p.len;
    const int32_t pg = p.table_row[tok / PAGE_TOKENS];
    const int t = (int)(tok % PAGE_TOKENS);
    const uint8_t* chunk = p.pool + (int64_t)pg * p.page_bytes + (int64_t)(h * (p.has_v ? 2 : 1) + kv) * p.chunk_bytes;
    const int64_t base = h * p.dh[kv] + tok * p.dt[kv];
    if (FMT == B200KV_FMT_F32 || FMT == B200KV_FMT_F16 || FMT == B200KV_FMT_BF16) {
        // bit copy (the destination has the storage element type): no conversion, NaN payloads survive
        const uint4 raw = *(const uint4*)(chunk + chunk_addr(FMT, p.D, kv, t, u * 16));
        if (FMT == B200KV_FMT_F32) {
            uint32_t* d = (uint32_t*)p.dst[kv] + base + u * EPU;
            d[0] = raw.x, d[1] = raw.y, d[2] = raw.z, d[3] = raw.w;
        } else {
            uint16_t* d = (uint16_t*)p.dst[kv] + base + u * EPU;
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; i++) d[2 * i] = (uint16_t)w[i], d[2 * i + 1] = (uint16_t)(w[i] >> 16);
        }
        return;
    }
    const int nb = p.D / 32;
    const __half* scales = (const __half*)(chunk + p.data_bytes);
    const int c0 = u * EPU;  // first channel of this thread (Q8_1: 16 channels, Q4_0: one block of 32)
    if (MODE == 1) {
        uint8_t out[16];
        if (FMT == B200KV_FMT_Q8_1) {
#pragma unroll
            for (int i = 0; i < 16; i++) out[i] = (uint8_t)(load_code<FMT>(chunk, p.D, kv, t, c0 + i) & 0xff);
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++)
                out[i] = (uint8_t)(load_code<FMT>(chunk, p.D, kv, t, c0 + i) | (load_code<FMT>(chunk, p.D, kv, t, c0 + 16 + i) << 4));
        }
        uint8_t* dst = (uint8_t*)p.codes + ((int64_t)h * p.len + tok) * p.row_bytes + u * 16;
#pragma unroll
        for (int i = 0; i < 16; i++) dst[i] = out[i];
        if (u < nb) ((__half*)p.scales)[((int64_t)h * p.len + tok) * nb + u] = scales[scale_index(FMT, p.D, kv, t, u)];
        return;
    }
#pragma unroll
    for (int i = 0; i < EPU; i++) {
        const int ch = c0 + i;
        const int code = load_code<FMT>(chunk, p.D, kv, t, ch) - (FMT == B200KV_FMT_Q4_0 ? 8 : 0);
        // code * f32(f16 scale): exact in f32 (q8_1.rs:50-63, q4_0.rs:82-95)
        st_from_f32(p.dst[kv], p.dtype, base + ch, __fmul_rn((float)code, __half2float(scales[scale_index(FMT, p.D, kv, t, ch / 32)])));
    }
}

// ---- host side --------------------------------------------------------------------------------------

static int alloc_pages(b200kv_cache* c, SeqState& s, int64_t new_len, std::vector<int32_t>& upd, int row) {
    int64_t need = fmt_is_kivi(c->cfg.format) ? kivi_pages_for(new_len) : (new_len + PAGE_TOKENS - 1) / PAGE_TOKENS;
    int64_t have = (int64_t)s.pages.size();
    if (need > c->max_pages_per_seq) return fail("sequence would exceed max_seq_tokens (%lld)", (long long)c->cfg.max_seq_tokens);
    if (need - have > (int64_t)c->free_pages.size())
        return fail("page pool exhausted: need %lld more pages, %zu free", (long long)(need - have), c->free_pages.size());
    for (int64_t i = have; i < need; i++) {
        int32_t pg = c->free_pages.back();
        c->free_pages.pop_back();
        s.pages.push_back(pg);
        upd.push_back((int32_t)((int64_t)row * c->max_pages_per_seq + i));
        upd.push_back(pg);
    }
    return B200KV_OK;
}

template <int FMT>
static void launch_append_fmt(const AppendParams& p, const InlineAppend& ia, int n_kv, cudaStream_t stream) {
    const int64_t per_entry = (int64_t)p.H * p.S * p.units;  // < 2^31: checked by the caller
    if constexpr (FMT == B200KV_FMT_F32 || FMT == B200KV_FMT_F16 || FMT == B200KV_FMT_BF16) {
        if (p.vec_ok && !p.rope_cos && per_entry >= 4096) {  // bulk appends (prompt chunks): four units per thread
            dim3 grid((unsigned)((per_entry + 1023) / 1024), 1, (unsigned)(p.n_seqs * n_kv));
            append_copy_kernel<FMT><<<grid, 256, 0, stream>>>(p, ia);
            return;
        }
    }
    dim3 grid((unsigned)((per_entry + 255) / 256), 1, (unsigned)(p.n_seqs * n_kv));
    (void)launch_after_predecessor(append_kernel<FMT>, grid, dim3(256), 0, stream, p, ia);  // the caller reads cudaGetLastError
}

int launch_export(b200kv_cache* c, int32_t seq, void* k_out, const int64_t* ks, void* v_out, const int64_t* vs,
                  int32_t dtype, cudaStream_t stream) {
    const SeqState& s = c->seqs[seq];
    if (s.len == 0) return B200KV_OK;
    ExportParams p{};
    p.pool = c->pool;
    p.table_row = c->d_table + (int64_t)seq * c->max_pages_per_seq;
    p.dst[0] = k_out, p.dst[1] = v_out;
    p.dh[0] = ks[0], p.dt[0] = ks[1];
    if (v_out) p.dh[1] = vs[0], p.dt[1] = vs[1];
    p.page_bytes = c->L.page_bytes, p.len = s.len;
    p.H = c->L.Hkv, p.D = c->L.D, p.chunk_bytes = c->L.chunk_bytes, p.data_bytes = c->L.data_bytes;
    p.plane_w = c->L.plane_w, p.units = c->L.row_bytes / 16, p.row_bytes = c->L.row_bytes;
    p.dtype = dtype, p.has_v = c->L.has_v;
    int64_t threads = (int64_t)p.H * p.len * p.units;
    dim3 grid((unsigned)((threads + 255) / 256), v_out ? 2 : 1);
    ProfScope ps(c, K_EXPORT, stream);
    switch (c->L.fmt) {
        case B200KV_FMT_F32: export_kernel<B200KV_FMT_F32, 0><<<grid, 256, 0, stream>>>(p); break;
        case B200KV_FMT_F16: export_kernel<B200KV_FMT_F16, 0><<<grid, 256, 0, stream>>>(p); break;
        case B200KV_FMT_BF16: export_kernel<B200KV_FMT_BF16, 0><<<grid, 256, 0, stream>>>(p); break;
        case B200KV_FMT_Q8_1: export_kernel<B200KV_FMT_Q8_1, 0><<<grid, 256, 0, stream>>>(p); break;
        case B200KV_FMT_Q4_0: export_kernel<B200KV_FMT_Q4_0, 0><<<grid, 256, 0, stream>>>(p); break;
        default: return fail("format %d cannot be exported", c->L.fmt);
    }
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

}  // namespace b200kv

using namespace b200kv;

extern "C" {

const char* b200kv_last_error(void) { return last_error().c_str(); }
const char* b200kv_version(void) { return "b200kv 0.1 sm_100a"; }

int b200kv_create(const b200kv_config* cfg, b200kv_cache** out) {
    if (!cfg || !out) return fail("null argument");
    *out = nullptr;
    if (cfg->format < B200KV_FMT_F32 || cfg->format > B200KV_FMT_KIVI4)
        return fail("storage format %d is not available in this build", cfg->format);
    if (cfg->head_dim != 64 && cfg->head_dim != 128) return fail("head_dim must be 64 or 128, got %d", cfg->head_dim);
    if (cfg->n_kv_heads <= 0 || cfg->max_seqs <= 0 || cfg->max_seq_tokens <= 0 || cfg->pool_tokens <= 0)
        return fail("n_kv_heads, max_seqs, max_seq_tokens and pool_tokens must be positive");
    if (cfg->max_q_heads < 0 || (cfg->max_q_heads > 0 && cfg->max_q_heads % cfg->n_kv_heads != 0))
        return fail("max_q_heads (%d) must be 0 or a multiple of n_kv_heads (%d)", cfg->max_q_heads, cfg->n_kv_heads);
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0)
        return fail("no CUDA device: b200kv has no CPU fallback");
    if (cfg->device < 0 || cfg->device >= n_dev) return fail("device %d out of range (%d devices)", cfg->device, n_dev);
    cudaDeviceProp prop;
    B200KV_CUDA(cudaGetDeviceProperties(&prop, cfg->device));
    if (prop.major != 10) return fail("device %d is sm_%d%d; this library is built for sm_100a only", cfg->device, prop.major, prop.minor);
    DeviceGuard guard(cfg->device);

    b200kv_cache* c = new b200kv_cache();
    c->cfg = *cfg;
    c->L = make_layout(cfg->format, cfg->head_dim, cfg->n_kv_heads, cfg->has_values ? 1 : 0);
    c->max_pages_per_seq = (int)((cfg->max_seq_tokens + PAGE_TOKENS - 1) / PAGE_TOKENS);
    // every live sequence may hold one partly filled page
    c->n_pages = (cfg->pool_tokens + PAGE_TOKENS - 1) / PAGE_TOKENS + cfg->max_seqs;
    c->seqs.resize(cfg->max_seqs);
    auto cleanup = [&](int rc) {
        b200kv_destroy(c);
        return rc;
    };
    if (fmt_is_kivi(cfg->format)) {
        if (kivi_create(c) != B200KV_OK) return cleanup(B200KV_KO);
    } else {
        size_t pool_bytes = (size_t)c->n_pages * c->L.page_bytes;
        if (cudaMalloc(&c->pool, pool_bytes) != cudaSuccess)
            return cleanup(fail("cannot allocate a %zu-byte page pool: %s", pool_bytes, cudaGetErrorString(cudaGetLastError())));
        // zero the pool once: unused token slots of a partly filled page are read (and masked) by the
        // attention kernels and must hold finite values
        if (cudaMemset(c->pool, 0, pool_bytes) != cudaSuccess) return cleanup(fail("cudaMemset failed"));
    }
    size_t table_bytes = (size_t)cfg->max_seqs * c->max_pages_per_seq * sizeof(int32_t);
    if (cudaMalloc(&c->d_table, table_bytes) != cudaSuccess || cudaMemset(c->d_table, 0xff, table_bytes) != cudaSuccess)
        return cleanup(fail("cannot allocate the page tables"));
    if (cudaMalloc(&c->d_status, sizeof(int)) != cudaSuccess || cudaMemset(c->d_status, 0, sizeof(int)) != cudaSuccess)
        return cleanup(fail("cannot allocate the status word"));
    c->free_pages.resize(c->n_pages);
    for (int64_t i = 0; i < c->n_pages; i++) c->free_pages[i] = (int32_t)(c->n_pages - 1 - i);
    // descriptor slots: the largest descriptor is a decode work list (64 splits per sequence at most)
    c->st.slot_bytes = std::max<size_t>(64 << 10, (size_t)cfg->max_seqs * (16 + 64 * 32) + 4096);
    if (cudaMallocHost(&c->st.host, c->st.slot_bytes * Staging::SLOTS) != cudaSuccess ||
        cudaMalloc(&c->st.dev, c->st.slot_bytes * Staging::SLOTS) != cudaSuccess)
        return cleanup(fail("cannot allocate the descriptor ring"));
    for (int i = 0; i < Staging::SLOTS; i++)
        if (cudaEventCreateWithFlags(&c->st.ev[i], cudaEventDisableTiming) != cudaSuccess)
            return cleanup(fail("cannot create events"));
    // the only scratch the attention calls use: split-KV partials, sized once (no call after this one allocates)
    c->ws_bytes = (size_t)workspace_records(*cfg) * (cfg->head_dim + 2) * sizeof(float);
    if (cudaMalloc(&c->ws, c->ws_bytes) != cudaSuccess) return cleanup(fail("cannot allocate the %zu-byte split-KV workspace", c->ws_bytes));
    if (cudaDeviceSynchronize() != cudaSuccess) return cleanup(fail("device error during creation"));
    *out = c;
    return B200KV_OK;
}

int64_t b200kv_workspace_bytes(const b200kv_config* cfg) {
    if (!cfg || cfg->n_kv_heads <= 0 || cfg->max_seqs <= 0 || (cfg->head_dim != 64 && cfg->head_dim != 128) || cfg->max_q_heads < 0) {
        fail("configuration b200kv_create would refuse");
        return -1;
    }
    return workspace_records(*cfg) * (cfg->head_dim + 2) * (int64_t)sizeof(float);
}

int b200kv_destroy(b200kv_cache* c) {
    if (!c) return B200KV_OK;
    DeviceGuard guard(c->cfg.device);
    cudaDeviceSynchronize();
    for (auto& r : c->prof) cudaEventDestroy(r.a), cudaEventDestroy(r.b);
    for (int i = 0; i < Staging::SLOTS; i++)
        if (c->st.ev[i]) cudaEventDestroy(c->st.ev[i]);
    if (c->st.host) cudaFreeHost(c->st.host);
    if (c->st.dev) cudaFree(c->st.dev);
    if (c->ws) cudaFree(c->ws);
    if (c->d_status) cudaFree(c->d_status);
    if (c->d_table) cudaFree(c->d_table);
    if (c->pool) cudaFree(c->pool);
    kivi_destroy(c);
    delete c;
    return B200KV_OK;
}

int b200kv_seq_new(b200kv_cache* c, int32_t* seq_out) {
    if (!c || !seq_out) return fail("null argument");
    for (size_t i = 0; i < c->seqs.size(); i++)
        if (!c->seqs[i].live) {
            c->seqs[i].live = true;
            c->seqs[i].len = 0;
            c->seqs[i].start = 0;
            c->seqs[i].pages.clear();
            *seq_out = (int32_t)i;
            return B200KV_OK;
        }
    return fail("all %zu sequence slots are in use", c->seqs.size());
}

int b200kv_seq_free(b200kv_cache* c, int32_t seq) {
    if (!c || seq < 0 || seq >= (int)c->seqs.size() || !c->seqs[seq].live) return fail("sequence %d is not live", seq);
    SeqState& s = c->seqs[seq];
    for (int32_t pg : s.pages)
        if (pg >= 0) c->free_pages.push_back(pg);  // trimmed entries are -1
    s.pages.clear();
    s.len = 0;
    s.start = 0;
    s.live = false;
    return B200KV_OK;
}

int64_t b200kv_seq_len(b200kv_cache* c, int32_t seq) {
    if (!c || seq < 0 || seq >= (int)c->seqs.size() || !c->seqs[seq].live) {
        fail("sequence %d is not live", seq);
        return -1;
    }
    return c->seqs[seq].len;
}

int64_t b200kv_free_pages(b200kv_cache* c) { return c ? (int64_t)c->free_pages.size() : -1; }
int64_t b200kv_page_bytes(b200kv_cache* c) {
    if (!c) return -1;
    return fmt_is_kivi(c->cfg.format) ? kivi_page_bytes(c) : c->L.page_bytes;
}

static int append_impl(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_new, const void* k_new,
                       const int64_t k_strides[3], const void* v_new, const int64_t v_strides[3], const void* rope_cos,
                       const void* rope_sin, const int64_t* rope_strides, int32_t dtype, void* stream_) {
    if (validate_seqs(c, n_seqs, seqs) != B200KV_OK) return B200KV_KO;
    if ((rope_cos != nullptr) != (rope_sin != nullptr) || (rope_cos && !rope_strides)) return fail("cos, sin and their strides come together");
    if (rope_cos && fmt_is_kivi(c->L.fmt)) return fail("the fused rotary embedding is not available for KIVI caches: apply b200kv_rope first");
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_new < 0) return fail("n_new must be >= 0");
    if (n_new == 0) return B200KV_OK;
    if (!k_new || !k_strides) return fail("k_new and its strides are required");
    if (c->L.has_v ? (!v_new || !v_strides) : (v_new != nullptr))
        return fail(c->L.has_v ? "this cache holds K and V: v_new is required" : "this cache holds one tensor: v_new must be NULL");
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if (!fmt_is_block_quant(c->L.fmt) && !fmt_is_kivi(c->L.fmt) && dtype != c->L.fmt)
        return fail("a bit-copy cache of format %d takes input of the same type, got dtype %d", c->L.fmt, dtype);
    if (!fmt_is_kivi(c->L.fmt) && ((int64_t)n_seqs * (c->L.has_v ? 2 : 1) > 65535 ||
                                   (int64_t)c->L.Hkv * n_new * (c->L.row_bytes / 16) >= (1ll << 31)))
        return fail("append of %d sequences x %d tokens exceeds the launch geometry: split the call", n_seqs, n_new);
    DeviceGuard guard(c->cfg.device);

    // host bookkeeping first, committed only if everything can be enqueued
    std::vector<int32_t> upd;
    std::vector<size_t> old_pages(n_seqs);
    auto rollback = [&](int upto) {
        for (int i = 0; i < upto; i++) {
            SeqState& s = c->seqs[seqs[i]];
            while (s.pages.size() > old_pages[i]) {
                c->free_pages.push_back(s.pages.back());
                s.pages.pop_back();
            }
        }
    };
    for (int i = 0; i < n_seqs; i++) {
        SeqState& s = c->seqs[seqs[i]];
        old_pages[i] = s.pages.size();
        if (alloc_pages(c, s, s.len + n_new, upd, seqs[i]) != B200KV_OK) {
            rollback(i + 1);
            return B200KV_KO;
        }
    }
    std::vector<int32_t> upd_off(n_seqs, -1), new_pn(n_seqs, 0);
    {
        // alloc_pages appended this call's pages sequence by sequence: recover each sequence's run
        size_t at = 0;
        for (int i = 0; i < n_seqs; i++) {
            const size_t grown = c->seqs[seqs[i]].pages.size() - old_pages[i];
            if (grown) upd_off[i] = (int32_t)at, new_pn[i] = (int32_t)old_pages[i];
            at += grown;
        }
    }
    // small batches travel as a kernel parameter; larger ones (and the KIVI kernels) through a descriptor slot
    InlineAppend ia{};
    const bool inline_batch = n_seqs <= INLINE_APPEND && upd.size() / 2 <= (size_t)INLINE_APPEND && !fmt_is_kivi(c->L.fmt);
    int slot = -1;
    uint8_t *h = nullptr, *d = nullptr;
    if (inline_batch) {
        ia.n = n_seqs;
        for (int i = 0; i < n_seqs; i++) ia.ent[i] = make_int4(seqs[i], (int)c->seqs[seqs[i]].len, upd_off[i], new_pn[i]);
        for (size_t i = 0; i < upd.size() / 2; i++) ia.upd[i] = make_int2(upd[2 * i], upd[2 * i + 1]);
    } else {
        size_t desc_words = (size_t)4 * n_seqs + upd.size();
        if (staging_acquire(c, desc_words * 4, &slot, &h, &d) != B200KV_OK) {
            rollback(n_seqs);
            return B200KV_KO;
        }
        int32_t* hw = (int32_t*)h;
        for (int i = 0; i < n_seqs; i++) {
            hw[4 * i] = seqs[i];
            hw[4 * i + 1] = (int32_t)c->seqs[seqs[i]].len;
            hw[4 * i + 2] = upd_off[i];
            hw[4 * i + 3] = new_pn[i];
        }
        if (!upd.empty()) memcpy(hw + 4 * n_seqs, upd.data(), upd.size() * 4);
        if (staging_upload(c, slot, desc_words * 4, stream) != B200KV_OK) {
            rollback(n_seqs);
            return B200KV_KO;
        }
    }
    if (!upd.empty() && fmt_is_kivi(c->L.fmt)) {  // the KIVI kernels read the table; the others take new pages from the descriptor
        int n = (int)(upd.size() / 2);
        ProfScope ps(c, K_SCATTER, stream);
        table_scatter_kernel<<<(n + 255) / 256, 256, 0, stream>>>(c->d_table, (const int32_t*)d + 4 * n_seqs, n);
    }
    AppendParams p{};
    p.upd = (const int32_t*)d + 4 * n_seqs, p.n_upd = (int32_t)(upd.size() / 2);
    p.pool = c->pool, p.table = c->d_table, p.desc = (const int32_t*)d, p.status = c->d_status;
    p.src[0] = k_new, p.src[1] = v_new;
    p.sb[0] = k_strides[0], p.sh[0] = k_strides[1], p.ss[0] = k_strides[2];
    if (v_new) p.sb[1] = v_strides[0], p.sh[1] = v_strides[1], p.ss[1] = v_strides[2];
    p.page_bytes = c->L.page_bytes, p.n_pages = (int32_t)c->n_pages, p.max_pages_per_seq = c->max_pages_per_seq;
    p.n_seqs = n_seqs, p.H = c->L.Hkv, p.S = n_new, p.D = c->L.D;
    p.chunk_bytes = c->L.chunk_bytes, p.data_bytes = c->L.data_bytes, p.plane_w = c->L.plane_w;
    p.units = c->L.row_bytes / 16;
    p.dtype = dtype, p.has_v = c->L.has_v;
    if (rope_cos) p.rope_cos = rope_cos, p.rope_sin = rope_sin, p.rope_b = rope_strides[0], p.rope_s = rope_strides[1];
    // 16-byte vector loads need aligned bases and strides
    const int esz = dtype_size(dtype);
    auto aligned = [&](const void* ptr, const int64_t* st) {
        return ptr == nullptr ||
               ((uintptr_t)ptr % 16 == 0 && (st[0] * esz) % 16 == 0 && (st[1] * esz) % 16 == 0 && (st[2] * esz) % 16 == 0);
    };
    p.vec_ok = aligned(k_new, k_strides) && aligned(v_new, v_strides);
    const int n_kv = c->L.has_v ? 2 : 1;
    if (fmt_is_kivi(c->L.fmt)) {
        kivi_append(c, n_seqs, seqs, n_new, k_new, k_strides, v_new, v_strides, dtype, (const int32_t*)d, stream);
    } else {
        ProfScope ps(c, K_APPEND, stream);
        switch (c->L.fmt) {
            case B200KV_FMT_F32: launch_append_fmt<B200KV_FMT_F32>(p, ia, n_kv, stream); break;
            case B200KV_FMT_F16: launch_append_fmt<B200KV_FMT_F16>(p, ia, n_kv, stream); break;
            case B200KV_FMT_BF16: launch_append_fmt<B200KV_FMT_BF16>(p, ia, n_kv, stream); break;
            case B200KV_FMT_Q8_1: launch_append_fmt<B200KV_FMT_Q8_1>(p, ia, n_kv, stream); break;
            case B200KV_FMT_Q4_0: launch_append_fmt<B200KV_FMT_Q4_0>(p, ia, n_kv, stream); break;
        }
    }
    cudaError_t e = cudaGetLastError();
    if (slot >= 0) staging_release(c, slot, stream);
    if (e != cudaSuccess) {
        rollback(n_seqs);
        return fail("append launch failed: %s", cudaGetErrorString(e));
    }
    for (int i = 0; i < n_seqs; i++) c->seqs[seqs[i]].len += n_new;
    return B200KV_OK;
}

int b200kv_append(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_new, const void* k_new,
                  const int64_t k_strides[3], const void* v_new, const int64_t v_strides[3], int32_t dtype, void* stream) {
    return append_impl(c, n_seqs, seqs, n_new, k_new, k_strides, v_new, v_strides, nullptr, nullptr, nullptr, dtype, stream);
}

int b200kv_append_rope(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, int32_t n_new, const void* k_new,
                       const int64_t k_strides[3], const void* v_new, const int64_t v_strides[3], const void* cos,
                       const void* sin, const int64_t rope_strides[2], int32_t dtype, void* stream) {
    if (!cos || !sin) return fail("cos and sin are required");
    return append_impl(c, n_seqs, seqs, n_new, k_new, k_strides, v_new, v_strides, cos, sin, rope_strides, dtype, stream);
}

int b200kv_export(b200kv_cache* c, int32_t seq, void* k_out, const int64_t k_strides[2], void* v_out,
                  const int64_t v_strides[2], int32_t dtype, void* stream) {
    if (validate_seqs(c, 1, &seq) != B200KV_OK) return B200KV_KO;
    if (c->seqs[seq].start > 0) return fail("sequence %d was trimmed to its last tokens: its front pages are gone", seq);
    if (!k_out || !k_strides) return fail("k_out and its strides are required");
    if (v_out && (!c->L.has_v || !v_strides)) return fail("v_out given but the cache has no values / no strides");
    if (dtype < B200KV_F32 || dtype > B200KV_BF16) return fail("unknown dtype %d", dtype);
    if (!fmt_is_block_quant(c->L.fmt) && !fmt_is_kivi(c->L.fmt) && dtype != c->L.fmt)
        return fail("a bit-copy cache exports its own element type (format %d), got dtype %d", c->L.fmt, dtype);
    DeviceGuard guard(c->cfg.device);
    if (fmt_is_kivi(c->L.fmt)) return kivi_export(c, seq, k_out, k_strides, v_out, v_strides, dtype, (cudaStream_t)stream);
    return launch_export(c, seq, k_out, k_strides, v_out, v_strides, dtype, (cudaStream_t)stream);
}

int b200kv_export_codes(b200kv_cache* c, int32_t seq, int32_t which, void* codes, void* scales, void* stream) {
    if (validate_seqs(c, 1, &seq) != B200KV_OK) return B200KV_KO;
    if (c->seqs[seq].start > 0) return fail("sequence %d was trimmed to its last tokens: its front pages are gone", seq);
    if (!fmt_is_block_quant(c->L.fmt)) return fail("format %d has no codes: use b200kv_export", c->L.fmt);
    if (which < 0 || which > (c->L.has_v ? 1 : 0)) return fail("which = %d out of range", which);
    if (!codes || !scales) return fail("codes and scales are required");
    DeviceGuard guard(c->cfg.device);
    const SeqState& s = c->seqs[seq];
    if (s.len == 0) return B200KV_OK;
    ExportParams p{};
    p.pool = c->pool;
    p.table_row = c->d_table + (int64_t)seq * c->max_pages_per_seq;
    p.codes = codes, p.scales = scales, p.which = which;
    p.page_bytes = c->L.page_bytes, p.len = s.len;
    p.H = c->L.Hkv, p.D = c->L.D, p.chunk_bytes = c->L.chunk_bytes, p.data_bytes = c->L.data_bytes;
    p.plane_w = c->L.plane_w, p.units = c->L.row_bytes / 16, p.row_bytes = c->L.row_bytes, p.has_v = c->L.has_v;
    int64_t threads = (int64_t)p.H * p.len * p.units;
    dim3 grid((unsigned)((threads + 255) / 256));
    if (c->L.fmt == B200KV_FMT_Q8_1) export_kernel<B200KV_FMT_Q8_1, 1><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
    else export_kernel<B200KV_FMT_Q4_0, 1><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
    B200KV_CUDA(cudaGetLastError());
    return B200KV_OK;
}

int b200kv_truncate(b200kv_cache* c, int32_t seq, int64_t len) {
    if (validate_seqs(c, 1, &seq) != B200KV_OK) return B200KV_KO;
    SeqState& s = c->seqs[seq];
    if (len < 0 || len > s.len) return fail("cannot truncate a sequence of %lld tokens to %lld", (long long)s.len, (long long)len);
    if (len < s.start) return fail("cannot truncate below token %lld: the pages before it were trimmed away", (long long)s.start);
    // QuantizedDynKvCacheState has no truncate: a finalised block cannot give its f32 rows back
    if (fmt_is_kivi(c->L.fmt) && len != s.len)
        return fail("a KIVI cache cannot be truncated (blocks are frozen once quantised; the reference has no truncate either)");
    size_t keep = (size_t)((len + PAGE_TOKENS - 1) / PAGE_TOKENS);
    while (s.pages.size() > keep) {
        c->free_pages.push_back(s.pages.back());
        s.pages.pop_back();
    }
    s.len = len;
    return B200KV_OK;
}

// b200kv_truncate for a batch: every sequence is checked before any is changed.
int b200kv_truncate_many(b200kv_cache* c, int32_t n_seqs, const int32_t* seqs, const int64_t* lens) {
    if (validate_seqs(c, n_seqs, seqs) != B200KV_OK) return B200KV_KO;
    if (!lens) return fail("null lengths");
    for (int i = 0; i < n_seqs; i++) {
        const SeqState& s = c->seqs[seqs[i]];
        if (lens[i] < 0 || lens[i] > s.len)
            return fail("cannot truncate sequence %d of %lld tokens to %lld", seqs[i], (long long)s.len, (long long)lens[i]);
        if (lens[i] < s.start) return fail("cannot truncate sequence %d below token %lld: the pages before it were trimmed away", seqs[i], (long long)s.start);
        if (fmt_is_kivi(c->L.fmt) && lens[i] != s.len) return fail("a KIVI cache cannot be truncated (blocks are frozen once quantised)");
    }
    for (int i = 0; i < n_seqs; i++) b200kv_truncate(c, seqs[i], lens[i]);
    return B200KV_OK;
}

// Gives the pages that lie wholly before the last `keep_last` tokens back to the pool: the bounded memory of the
// reference's sliding-window ring buffer (transformers/src/ops/window_kv_cache.rs:77-137) on a paged store.  Positions
// keep counting from the sequence's real start; attention from now on sees tokens >= len - keep_last at most.
int b200kv_trim(b200kv_cache* c, int32_t seq, int64_t keep_last) {
    if (validate_seqs(c, 1, &seq) != B200KV_OK) return B200KV_KO;
    if (keep_last <= 0) return fail("keep_last must be positive");
    if (fmt_is_kivi(c->L.fmt)) return fail("a KIVI cache keeps its sinks and blocks: it cannot be trimmed");
    SeqState& s = c->seqs[seq];
    const int64_t start = std::max<int64_t>(s.start, s.len - keep_last);
    for (int64_t pgi = s.start / PAGE_TOKENS; pgi < start / PAGE_TOKENS; pgi++)
        if (s.pages[(size_t)pgi] >= 0) {
            c->free_pages.push_back(s.pages[(size_t)pgi]);
            s.pages[(size_t)pgi] = -1;
        }
    s.start = start;
    return B200KV_OK;
}

int b200kv_fork(b200kv_cache* c, int32_t seq, int32_t* new_seq_out, void* stream_) {
    if (validate_seqs(c, 1, &seq) != B200KV_OK) return B200KV_KO;
    if (c->seqs[seq].start > 0) return fail("sequence %d was trimmed to its last tokens: its front pages are gone", seq);
    if (!new_seq_out) return fail("null argument");
    cudaStream_t stream = (cudaStream_t)stream_;
    DeviceGuard guard(c->cfg.device);
    int32_t ns;
    if (b200kv_seq_new(c, &ns) != B200KV_OK) return B200KV_KO;
    SeqState& src = c->seqs[seq];
    SeqState& dst = c->seqs[ns];
    std::vector<int32_t> upd;
    if (alloc_pages(c, dst, src.len, upd, ns) != B200KV_OK) {
        b200kv_seq_free(c, ns);
        return B200KV_KO;
    }
    auto undo = [&](int rc) {  // the new sequence and its pages go back; copies already enqueued only touch pages that are free again
        b200kv_seq_free(c, ns);
        return rc;
    };
    // the new page-table entries travel in slot-sized pieces, so that a sequence of any length can be forked
    const size_t per_slot = c->st.slot_bytes / 8;  // (index, page) pairs per piece
    for (size_t at = 0; at < upd.size() / 2; at += per_slot) {
        const size_t n = std::min(per_slot, upd.size() / 2 - at);
        int slot;
        uint8_t *h, *d;
        if (staging_acquire(c, n * 8, &slot, &h, &d) != B200KV_OK) return undo(B200KV_KO);
        memcpy(h, upd.data() + 2 * at, n * 8);
        if (staging_upload(c, slot, n * 8, stream) != B200KV_OK) return undo(B200KV_KO);
        table_scatter_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(c->d_table, (const int32_t*)d, (int)n);
        staging_release(c, slot, stream);
        if (cudaGetLastError() != cudaSuccess) return undo(fail("page-table update launch failed"));
    }
    if (!fmt_is_kivi(c->L.fmt))
        for (size_t i = 0; i < src.pages.size(); i++)
            if (cudaMemcpyAsync(c->pool + (int64_t)dst.pages[i] * c->L.page_bytes, c->pool + (int64_t)src.pages[i] * c->L.page_bytes,
                                c->L.page_bytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
                return undo(fail("page copy failed: %s", cudaGetErrorString(cudaGetLastError())));
    if (fmt_is_kivi(c->L.fmt) && kivi_fork(c, seq, ns, stream) != B200KV_OK) return undo(B200KV_KO);
    dst.len = src.len;
    *new_seq_out = ns;
    return B200KV_OK;
}

int b200kv_profile(b200kv_cache* c, int32_t enable) {
    if (!c) return fail("null cache");
    c->prof_on = (enable & 1) != 0;
    c->force_simt = (enable & 2) != 0;
    c->kivi_cuda_core = (enable & 4) != 0;
    if (enable & 8) c->stall_next_decode = true;  // consumed by the next decode launch
    return B200KV_OK;
}

int b200kv_profile_read(b200kv_cache* c, int32_t max_records, int32_t* kernel_ids, float* ms, int32_t* n_out) {
    if (!c || !n_out) return fail("null argument");
    DeviceGuard guard(c->cfg.device);
    int n = 0;
    for (auto& r : c->prof) {
        float t = 0.f;
        cudaError_t e = cudaEventSynchronize(r.b);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&t, r.a, r.b);
        cudaEventDestroy(r.a);
        cudaEventDestroy(r.b);
        if (e != cudaSuccess) {
            c->prof.clear();
            return fail("reading a timing record failed: %s", cudaGetErrorString(e));
        }
        if (n < max_records && kernel_ids && ms) kernel_ids[n] = r.id, ms[n] = t, n++;
    }
    c->prof.clear();
    *n_out = n;
    return B200KV_OK;
}

int b200kv_check(b200kv_cache* c, void* stream) {
    if (!c) return fail("null cache");
    DeviceGuard guard(c->cfg.device);
    B200KV_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    int st = 0;
    B200KV_CUDA(cudaMemcpy(&st, c->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st) {
        int zero = 0;
        cudaMemcpy(c->d_status, &zero, sizeof(int), cudaMemcpyHostToDevice);
        return fail("device status %d:%s%s", st, (st & STATUS_PAGE_OOB) ? " page index out of range" : "",
                    (st & STATUS_WAIT_EXPIRED) ? " a bounded wait expired" : "");
    }
    return B200KV_OK;
}

}  // extern "C"
