// Shared definitions of the b200kv kernels: page layout, element conversion, bulk-copy helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200kv.h"

namespace b200kv {

// A page holds PAGE_TOKENS consecutive tokens of every kv head, K and V.
constexpr int PAGE_TOKENS = 64;

// ---- page layout ---------------------------------------------------------------------------
// page   = [Hkv][K chunk, V chunk]            (V chunk absent when the cache has no values)
// chunk  = data region (PAGE_TOKENS rows of ROW_BYTES) followed, for the block-quantised
//          formats, by PAGE_TOKENS x (D/32) f16 scales in token order.
// A row is the byte string of one token-head: D elements (f32 / f16 / bf16), D code bytes
// (Q8_1, stored offset-binary: code + 128) or D/2 nibble bytes (Q4_0).  The data region is cut
// into column slabs ("planes") 128 bytes wide (or ROW_BYTES if smaller); inside a plane the
// bytes are linear in (token, byte) and the index of each 16-byte unit inside its 128-byte line
// is XOR-ed with a function of the line number (swz_mask) chosen so that the shared-memory
// access patterns of the kernels are free of bank conflicts.  For f16 / bf16 that function is
// the 128-byte swizzle of ldmatrix / tcgen05 operand tiles.  Because whole chunks are contiguous
// in HBM, one untiled cp.async.bulk brings a chunk into shared memory already in that arrangement.
//
// The layout is private to the library: at head_dim 128 the V rows of the quantised formats
// also store their codes in a permuted channel order that lets the tensor-core decode kernel
// build V^T operand fragments from 16 contiguous bytes per thread:
//   Q8_1 V: byte position 16r + 2j + h holds channel 16j + r + 8h        (r < 8, j < 8, h < 2)
//   Q4_0 V: byte position  8r + j holds channel 16j + r (low nibble) and 16j + r + 8 (high nibble)
// K rows keep the natural order (Q4_0: GGML block bytes, byte i of block b = channel 32b + i |
// channel 32b + 16 + i << 4).  b200kv_export_codes undoes all of this.
struct Layout {
    int fmt, D, Hkv, has_v;
    int row_bytes;    // bytes of one token-head row in the data region
    int plane_w;      // min(row_bytes, 128)
    int data_bytes;   // PAGE_TOKENS * row_bytes
    int scale_bytes;  // PAGE_TOKENS * (D/32) * 2 for Q8_1 / Q4_0, else 0
    int chunk_bytes;  // data_bytes + scale_bytes
    int64_t page_bytes;
};

__host__ __device__ inline int fmt_row_bytes(int fmt, int D) {
    switch (fmt) {
        case B200KV_FMT_F32: return D * 4;
        case B200KV_FMT_F16:
        case B200KV_FMT_BF16: return D * 2;
        case B200KV_FMT_Q8_1: return D;
        case B200KV_FMT_Q4_0: return D / 2;
        default: return 0;
    }
}
__host__ __device__ inline bool fmt_is_block_quant(int fmt) { return fmt == B200KV_FMT_Q8_1 || fmt == B200KV_FMT_Q4_0; }

inline Layout make_layout(int fmt, int D, int Hkv, int has_v) {
    Layout L;
    L.fmt = fmt;
    L.D = D;
    L.Hkv = Hkv;
    L.has_v = has_v;
    L.row_bytes = fmt_row_bytes(fmt, D);
    L.plane_w = L.row_bytes < 128 ? L.row_bytes : 128;
    L.data_bytes = PAGE_TOKENS * L.row_bytes;
    L.scale_bytes = fmt_is_block_quant(fmt) ? PAGE_TOKENS * (D / 32) * 2 : 0;
    L.chunk_bytes = L.data_bytes + L.scale_bytes;
    L.page_bytes = (int64_t)Hkv * (has_v ? 2 : 1) * L.chunk_bytes;
    return L;
}

// True when the V rows of this cache store their codes in the permuted channel order.
__host__ __device__ constexpr bool v_permuted(int fmt, int D, int kv) {
    return kv == 1 && D == 128 && (fmt == B200KV_FMT_Q8_1 || fmt == B200KV_FMT_Q4_0);
}

// XOR mask for the 16-byte-unit index inside 128-byte line `line` of a plane.
__host__ __device__ constexpr uint32_t swz_mask(int fmt, int D, int kv, uint32_t line) {
    // Q8_1 K at D = 128: the tensor-core kernel reads 32 bytes per row from 4 rows per wavefront
    if (D == 128 && fmt == B200KV_FMT_Q8_1 && kv == 0) return ((line & 3u) << 1) | ((line >> 2) & 1u);
    // Q4_0 V at D = 128: 32 bytes per row from rows two lines apart
    if (D == 128 && fmt == B200KV_FMT_Q4_0 && kv == 1) return (line & 3u) << 1;
    return line & 7u;
}

// Byte offset inside a chunk's data region of row byte `rb` of token slot `t`.
__host__ __device__ constexpr uint32_t chunk_addr(int fmt, int D, int kv, int t, int rb) {
    const uint32_t row = (uint32_t)fmt_row_bytes(fmt, D);
    const uint32_t pw = row < 128u ? row : 128u;
    const uint32_t plane = (uint32_t)rb / pw;
    const uint32_t lin = (uint32_t)t * pw + (uint32_t)rb % pw;
    return plane * (uint32_t)PAGE_TOKENS * pw + (lin ^ (swz_mask(fmt, D, kv, lin >> 7) << 4));
}

// Where the code of channel `ch` lives in a quantised row: byte position, and for Q4_0 the nibble.
__host__ __device__ constexpr int code_pos(int fmt, int D, int kv, int ch) {
    if (fmt == B200KV_FMT_Q8_1) return v_permuted(fmt, D, kv) ? (ch % 8) * 16 + 2 * (ch / 16) + ((ch / 8) & 1) : ch;
    return v_permuted(fmt, D, kv) ? (ch % 8) * 8 + ch / 16 : (ch / 32) * 16 + ch % 16;
}
__host__ __device__ constexpr int code_nibble(int fmt, int D, int kv, int ch) {
    return v_permuted(fmt, D, kv) ? (ch / 8) & 1 : (ch % 32) / 16;
}

// Index (in f16 units) of the scale of block `blk` of token slot `t` inside a chunk's scale region.  K rows
// and all D = 64 rows keep [token][block]; the permuted V rows keep [token pair][block][2], so that the
// tensor-core decode kernel reads (scale of token 2p, scale of token 2p + 1) of a block as one f16 pair.
__host__ __device__ constexpr int scale_index(int fmt, int D, int kv, int t, int blk) {
    return v_permuted(fmt, D, kv) ? ((t >> 1) * 4 + blk) * 2 + (t & 1) : t * (D / 32) + blk;
}

// Channel index of element e of the piece that starts at row byte rb (piece_bytes long), natural
// row order.  Q4_0 pieces yield their low-nibble elements first, then the high-nibble ones.
template <int FMT>
__host__ __device__ inline int row_channel(int rb, int e, int piece_bytes) {
    if (FMT == B200KV_FMT_F32) return rb / 4 + e;
    if (FMT == B200KV_FMT_F16 || FMT == B200KV_FMT_BF16) return rb / 2 + e;
    if (FMT == B200KV_FMT_Q8_1) return rb + e;
    int b = rb / 16, j0 = rb % 16;
    return e < piece_bytes ? b * 32 + j0 + e : b * 32 + 16 + j0 + (e - piece_bytes);
}
// The same for a row in the permuted V order (Q8_1 / Q4_0, D = 128).
template <int FMT>
__host__ __device__ inline int row_channel_vperm(int rb, int e, int piece_bytes) {
    if (FMT == B200KV_FMT_Q8_1) {
        int pos = rb + e;
        return 16 * ((pos % 16) / 2) + pos / 16 + 8 * (pos & 1);
    }
    int pos = rb + (e < piece_bytes ? e : e - piece_bytes);
    return 16 * (pos % 8) + pos / 8 + (e < piece_bytes ? 0 : 8);
}

// Elements held by `bytes` bytes of a row.
template <int FMT>
__host__ __device__ constexpr int elems_in_bytes(int bytes) {
    return FMT == B200KV_FMT_F32 ? bytes / 4
         : (FMT == B200KV_FMT_F16 || FMT == B200KV_FMT_BF16) ? bytes / 2
         : FMT == B200KV_FMT_Q8_1 ? bytes
                                  : bytes * 2;
}

// ---- element conversion ------------------------------------------------------------------------
__device__ inline float ld_as_f32(const void* p, int dtype, int64_t i) {
    if (dtype == B200KV_F32) return ((const float*)p)[i];
    if (dtype == B200KV_F16) return __half2float(((const __half*)p)[i]);
    return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ inline void st_from_f32(void* p, int dtype, int64_t i, float v) {
    if (dtype == B200KV_F32) ((float*)p)[i] = v;
    else if (dtype == B200KV_F16) ((__half*)p)[i] = __float2half_rn(v);
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}
__host__ __device__ inline int dtype_size(int dtype) { return dtype == B200KV_F32 ? 4 : 2; }

// ApplyRope (transformers/src/ops/apply_rope.rs:155-163): x * cos + rotate_half(x) * sin, where the three
// operations are separate ops of the tensor's own type: each result is rounded to that type (for f16 / bf16 the
// arithmetic is done in f32 and rounded back, as the `half` crate does), and nothing is fused.
__device__ inline float round_to_dtype(float v, int dtype) {
    if (dtype == B200KV_F16) return __half2float(__float2half_rn(v));
    if (dtype == B200KV_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}
__device__ inline float rope_value(float x, float rot, float c, float s, int dtype) {
    const float a = round_to_dtype(__fmul_rn(x, c), dtype), b = round_to_dtype(__fmul_rn(rot, s), dtype);
    return round_to_dtype(__fadd_rn(a, b), dtype);
}
// Element `ch` of ApplyRope(row, cos_row, sin_row) for rows of D elements of type dtype.
__device__ inline float rope_row_elem(const void* row, const void* cos_row, const void* sin_row, int dtype, int D, int ch) {
    const int half = D / 2;
    const float x = ld_as_f32(row, dtype, ch);
    const float rot = ch < half ? -ld_as_f32(row, dtype, ch + half) : ld_as_f32(row, dtype, ch - half);
    return rope_value(x, rot, ld_as_f32(cos_row, dtype, ch), ld_as_f32(sin_row, dtype, ch), dtype);
}

// Decodes one piece (PB bytes at p, 16-byte aligned when PB == 16) into floats.  Block-quantised
// formats return the integer codes as floats (Q8_1: byte - 128, Q4_0: nibble - 8); the caller applies the scale.
template <int FMT, int PB>
__device__ inline void load_piece(const uint8_t* p, float* out) {
    uint32_t w[4];
    if (PB == 16) {
        uint4 v = *(const uint4*)p;
        w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
    } else if (PB == 8) {
        uint2 v = *(const uint2*)p;
        w[0] = v.x, w[1] = v.y;
    } else if (PB == 4) {
        w[0] = *(const uint32_t*)p;
    } else {
        w[0] = *(const uint16_t*)p;
    }
    if (FMT == B200KV_FMT_F32) {
#pragma unroll
        for (int i = 0; i < PB / 4; i++) out[i] = __uint_as_float(w[i]);
    } else if (FMT == B200KV_FMT_F16) {
#pragma unroll
        for (int i = 0; i < PB / 4; i++) {
            float2 f = __half22float2(*(const __half2*)&w[i]);
            out[2 * i] = f.x, out[2 * i + 1] = f.y;
        }
    } else if (FMT == B200KV_FMT_BF16) {
#pragma unroll
        for (int i = 0; i < PB / 4; i++) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    } else if (FMT == B200KV_FMT_Q8_1) {
#pragma unroll
        for (int b = 0; b < PB; b++) out[b] = (float)((int)((w[b / 4] >> (8 * (b % 4))) & 0xffu) - 128);  // offset-binary
    } else {  // Q4_0: low nibbles of the PB bytes, then high nibbles
#pragma unroll
        for (int b = 0; b < PB; b++) {
            uint32_t byte = (w[b / 4] >> (8 * (b % 4))) & 0xffu;
            out[b] = (float)((int)(byte & 0xf) - 8);
            out[PB + b] = (float)((int)(byte >> 4) - 8);
        }
    }
}

// Integer code of channel ch of a quantised row: Q8_1 -> -128..127, Q4_0 -> nibble 0..15.
template <int FMT>
__device__ inline int load_code(const uint8_t* chunk, int D, int kv, int t, int ch) {
    const int pos = code_pos(FMT, D, kv, ch);
    const uint32_t byte = chunk[chunk_addr(FMT, D, kv, t, pos)];
    if (FMT == B200KV_FMT_Q8_1) return (int)byte - 128;
    return code_nibble(FMT, D, kv, ch) ? (int)(byte >> 4) : (int)(byte & 0xf);
}

// Element `ch` of token slot t of a chunk as a float: a bit copy widened, or code * f32(f16 scale) (q8_1.rs:50-63, q4_0.rs:82-95).
__device__ inline float chunk_elem(const uint8_t* chunk, int fmt, int D, int kv, int t, int ch) {
    if (fmt == B200KV_FMT_F32) return *(const float*)(chunk + chunk_addr(fmt, D, kv, t, ch * 4));
    if (fmt == B200KV_FMT_F16) return __half2float(*(const __half*)(chunk + chunk_addr(fmt, D, kv, t, ch * 2)));
    if (fmt == B200KV_FMT_BF16) return __bfloat162float(*(const __nv_bfloat16*)(chunk + chunk_addr(fmt, D, kv, t, ch * 2)));
    const __half* scales = (const __half*)(chunk + PAGE_TOKENS * fmt_row_bytes(fmt, D));
    const float d = __half2float(scales[scale_index(fmt, D, kv, t, ch / 32)]);
    if (fmt == B200KV_FMT_Q8_1) return __fmul_rn((float)load_code<B200KV_FMT_Q8_1>(chunk, D, kv, t, ch), d);
    return __fmul_rn((float)(load_code<B200KV_FMT_Q4_0>(chunk, D, kv, t, ch) - 8), d);
}

// ---- shared-memory barriers and bulk copies (sm_90+ PTX; no cluster multicast anywhere) -----
__device__ inline uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ inline void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ inline void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ inline void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ inline void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ inline uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits for a barrier phase, giving up after `limit_ns` (~1 s by default) so that a copy that never lands cannot hang the GPU.
__device__ inline bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint64_t limit_ns = 1000000000ull) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = globaltimer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (globaltimer_ns() - t0 > limit_ns) return false;
    }
}
// Untiled bulk copy global -> this CTA's shared memory; completion is counted in bytes on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ inline void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(__cvta_generic_to_global(src_gmem)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// ---- programmatic dependent launch ------------------------------------------------------------------
// A kernel launched with launch_after_predecessor may be scheduled while the kernel before it in the
// stream is still draining; it must call grid_dependency_wait() before it touches anything that kernel
// wrote.  A kernel calls grid_launch_dependents() once it no longer minds its successor being scheduled.
__device__ inline void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ inline void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... P>
inline cudaError_t launch_after_predecessor(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                            const P&... params) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, params...);
}

// Device status word bits.
constexpr int STATUS_PAGE_OOB = 1;      // a page-table entry outside the pool
constexpr int STATUS_WAIT_EXPIRED = 2;  // a bounded barrier wait gave up

}  // namespace b200kv
