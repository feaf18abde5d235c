// TEST INFRASTRUCTURE — not part of the product.
//
// CPU restatement of the algorithms tract runs on its default (CPU) runtime for
// the KV-cache + attention path.  Only tests, the smoke check and the CPU
// baseline leg of the benchmark may load this library; the CUDA library never
// links or calls it.
//
// The reference is Rust and cannot be compiled where this was written (no
// cargo/rustc), so this file restates the cited source ranges operation by
// operation.  Arithmetic is IEEE-754 binary32, evaluated in the written order
// with no FMA contraction (build with -ffp-contract=off); the only fused
// multiply-adds are the explicit fmaf() chains that restate the GEMM
// micro-kernel of the `matrixmultiply` crate (0.3.10, pinned by the
// reference's Cargo.lock) that ndarray 0.17.2 `dot` lowers to on x86-64 with
// FMA: one accumulator per output element, k ascending.
//
// Parity pins: the six `harness/nnef-test-cases/sdpa/*/io.npz` bundles of the
// reference (attention), its hand-written unit cases, and the block-quant
// round-trip known answers in `linalg/src/frame/block_quant/{q4_0,q8_1}.rs`.
// The exact codes / scales of Q8_1 and of QuantizedDynKeyValueCache are not
// pinned by any reference test ("parity unpinned" for those): this restatement
// of the cited lines is their sole arbiter.
//
// Rust semantics restated here:
//   f32::round        -> roundf (half away from zero)
//   `x as i8/u8`      -> truncate toward zero, saturate, NaN -> 0
//   f32::min / max    -> fminf / fmaxf (a NaN operand is ignored)
//   f16::from_f32     -> round to nearest even, overflow to inf (half 2.7.1)
//   f32::recip        -> 1.0f / x
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

// ---- scalar conversions ---------------------------------------------------

inline uint32_t f32_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}
inline float bits_f32(uint32_t u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// IEEE binary32 -> binary16, round to nearest even (what half::f16::from_f32 does).
uint16_t f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mant = x & 0x007fffffu;
    int32_t exp = (int32_t)((x >> 23) & 0xff);
    if (exp == 0xff) {  // inf / nan
        if (mant == 0) return (uint16_t)(sign | 0x7c00u);
        return (uint16_t)(sign | 0x7c00u | 0x0200u | (mant >> 13));
    }
    int32_t e = exp - 127 + 15;
    if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u);  // overflow
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;  // underflow to zero
        mant |= 0x00800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half_mant = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_mant & 1))) half_mant++;
        return (uint16_t)(sign | half_mant);
    }
    uint32_t half = sign | ((uint32_t)e << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;  // carries into exponent correctly
    return (uint16_t)half;
}

float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t mant = h & 0x3ffu;
    if (exp == 0) {
        if (mant == 0) return bits_f32(sign);
        // subnormal: normalise
        int e = -1;
        do {
            e++;
            mant <<= 1;
        } while (!(mant & 0x400u));
        mant &= 0x3ffu;
        return bits_f32(sign | ((uint32_t)(127 - 15 - e) << 23) | (mant << 13));
    }
    if (exp == 0x1f) return bits_f32(sign | 0x7f800000u | (mant << 13));
    return bits_f32(sign | ((exp + 127 - 15) << 23) | (mant << 13));
}

// Rust `x as i8` for f32 x.
inline int8_t sat_i8(float x) {
    if (std::isnan(x)) return 0;
    if (x <= -128.0f) return -128;
    if (x >= 127.0f) return 127;
    return (int8_t)x;  // truncates toward zero
}
// Rust `x as u8` for f32 x.
inline uint8_t sat_u8(float x) {
    if (std::isnan(x)) return 0;
    if (x <= 0.0f) return 0;
    if (x >= 255.0f) return 255;
    return (uint8_t)x;
}

// Rust f32::clamp(lo, hi): NaN stays NaN.
inline float clampf(float x, float lo, float hi) {
    if (x < lo) return lo;
    if (x > hi) return hi;
    return x;
}

// Runs fn(i) for i in [0, n) on `threads` host threads (the reference uses
// rayon's global pool for the same per-(batch, q-head) task list).
template <class F>
void parallel_for(int n, int threads, F fn) {
    if (threads <= 1 || n <= 1) {
        for (int i = 0; i < n; i++) fn(i);
        return;
    }
    std::atomic<int> next{0};
    std::vector<std::thread> pool;
    int nt = std::min(threads, n);
    for (int t = 0; t < nt; t++)
        pool.emplace_back([&] {
            for (;;) {
                int i = next.fetch_add(1);
                if (i >= n) return;
                fn(i);
            }
        });
    for (auto& th : pool) th.join();
}

// ndarray 0.17.2 `numeric_util::unrolled_fold` for a contiguous f32 sum:
// eight running partials, combined as (p0+p4),(p1+p5),(p2+p6),(p3+p7) into one
// accumulator, then the < 8 trailing elements in order.
float ndarray_sum(const float* x, int n) {
    float p[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (; i + 8 <= n; i += 8)
        for (int j = 0; j < 8; j++) p[j] = p[j] + x[i + j];
    float acc = 0.0f;
    acc = acc + (p[0] + p[4]);
    acc = acc + (p[1] + p[5]);
    acc = acc + (p[2] + p[6]);
    acc = acc + (p[3] + p[7]);
    for (; i < n; i++) acc = acc + x[i];
    return acc;
}

// One (batch, q-head) of transformers/src/ops/flash_sdpa.rs:239-341
// (`attend_one_head`): 32x32 tiles, kv tiles outer, O kept normalised after
// every tile.  q: [S, D] rows at stride q_rs; k, v: [T, D] rows at k_rs / v_rs;
// mask: [S, T] rows at stride m_rs or null; out: [S, D] contiguous.
void attend_one_head(const float* q, int64_t q_rs, const float* k, int64_t k_rs, const float* v,
                     int64_t v_rs, const float* mask, int64_t m_rs, int S, int T, int D,
                     float scale, bool causal, float* out) {
    const int BKV = 32, BQ = 32;
    std::fill(out, out + (size_t)S * D, 0.0f);
    std::vector<float> l(S, 0.0f), m(S, -std::numeric_limits<float>::infinity());
    std::vector<float> s(BQ * BKV), sv(BQ * D), tile_m(BQ), tile_l(BQ), m_new(BQ), l_new(BQ);
    const float NEG_INF = -std::numeric_limits<float>::infinity();
    for (int kb = 0; kb < (T + BKV - 1) / BKV; kb++) {
        for (int qb = 0; qb < (S + BQ - 1) / BQ; qb++) {
            int kv0 = kb * BKV, kv1 = std::min(kv0 + BKV, T), nk = kv1 - kv0;
            int q0 = qb * BQ, q1 = std::min(q0 + BQ, S), nq = q1 - q0;
            if (mask) {  // :266-274 skip a tile whose mask is entirely below -65503
                bool all = true;
                for (int r = 0; r < nq && all; r++)
                    for (int c = 0; c < nk; c++)
                        if (!(mask[(int64_t)(q0 + r) * m_rs + kv0 + c] < -65503.0f)) {
                            all = false;
                            break;
                        }
                if (all) continue;
            }
            // :282  S = (Q . K^T) * scale ; dot = matrixmultiply FMA micro-kernel order
            for (int r = 0; r < nq; r++)
                for (int c = 0; c < nk; c++) {
                    const float* qr = q + (int64_t)(q0 + r) * q_rs;
                    const float* kr = k + (int64_t)(kv0 + c) * k_rs;
                    float acc = 0.0f;
                    for (int d = 0; d < D; d++) acc = fmaf(qr[d], kr[d], acc);
                    s[r * nk + c] = acc * scale;
                }
            if (mask) {  // :283-284
                for (int r = 0; r < nq; r++)
                    for (int c = 0; c < nk; c++)
                        s[r * nk + c] = s[r * nk + c] + mask[(int64_t)(q0 + r) * m_rs + kv0 + c];
            } else if (causal) {  // :285-294  triu(-inf, diag = q0 - kv0 - S + T + 1), added
                int64_t diag = (int64_t)q0 - kv0 - S + T + 1;
                for (int r = 0; r < nq; r++)
                    for (int c = 0; c < nk; c++)
                        s[r * nk + c] = s[r * nk + c] + (((int64_t)c - r >= diag) ? NEG_INF : 0.0f);
            }
            // :295-304 row max with a total order (FloatOrd), subtract when finite
            for (int r = 0; r < nq; r++) {
                float mx = s[r * nk];
                for (int c = 1; c < nk; c++) {
                    float x = s[r * nk + c];
                    // FloatOrd: NaN sorts above everything; keep the later of equal maxima
                    // (value-identical, so no observable difference).
                    if (std::isnan(x) || (!std::isnan(mx) && x > mx)) mx = x;
                }
                tile_m[r] = mx;
                if (std::isfinite(mx))
                    for (int c = 0; c < nk; c++) s[r * nk + c] = s[r * nk + c] - mx;
            }
            // :306-307 exp, row sums
            for (int i = 0; i < nq * nk; i++) s[i] = expf(s[i]);
            for (int r = 0; r < nq; r++) tile_l[r] = ndarray_sum(&s[r * nk], nk);
            // :309-317
            for (int r = 0; r < nq; r++) {
                float mo = m[q0 + r];
                m_new[r] = fmaxf(mo, tile_m[r]);
                l_new[r] = expf(mo - m_new[r]) * l[q0 + r] + expf(tile_m[r] - m_new[r]) * tile_l[r];
            }
            // :321  sv = P . V  (same GEMM micro-kernel order: k ascending FMA chain)
            for (int r = 0; r < nq; r++)
                for (int j = 0; j < D; j++) {
                    float acc = 0.0f;
                    for (int c = 0; c < nk; c++) acc = fmaf(s[r * nk + c], v[(int64_t)(kv0 + c) * v_rs + j], acc);
                    sv[r * D + j] = acc;
                }
            // :322-337
            for (int r = 0; r < nq; r++) {
                float r_l_new = 1.0f / l_new[r];
                float mo = m[q0 + r];
                float mul_o = expf(mo - m_new[r]) * l[q0 + r] * r_l_new;
                float mul_sv = expf(tile_m[r] - m_new[r]) * r_l_new;
                float* orow = out + (size_t)(q0 + r) * D;
                for (int j = 0; j < D; j++) orow[j] = orow[j] * mul_o + sv[r * D + j] * mul_sv;
            }
            for (int r = 0; r < nq; r++) {
                l[q0 + r] = l_new[r];
                m[q0 + r] = m_new[r];
            }
        }
    }
}

}  // namespace

extern "C" {

// ---- dtype helpers (exposed so tests can pin them against numpy) ------------
uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

// ---- a1: DynKeyValueCache append ------------------------------------------
// transformers/src/ops/dyn_kv_cache.rs:158-174 (+ core/src/ops/array/concat.rs):
// output = concat(past, input) along the sequence axis of [lead, T, inner]
// byte arrays (dtype-agnostic bit copy).  `row_bytes` = inner * element size.
void orc_dyn_kv_concat(const uint8_t* past, int64_t P, const uint8_t* input, int64_t S, int64_t lead,
                       int64_t row_bytes, uint8_t* out) {
    for (int64_t i = 0; i < lead; i++) {
        uint8_t* o = out + i * (P + S) * row_bytes;
        if (P) std::memcpy(o, past + i * P * row_bytes, (size_t)(P * row_bytes));
        if (S) std::memcpy(o + P * row_bytes, input + i * S * row_bytes, (size_t)(S * row_bytes));
    }
}

// ---- a4: Q8_1 block (32 values) ---------------------------------------------
// linalg/src/frame/block_quant/q8_1.rs:20-48.  Output, per block: scale (f16
// bits), sum (f16 bits), 32 int8 codes.
void orc_q8_1_quant(const float* x, int64_t n_blocks, uint16_t* scales, uint16_t* sums, int8_t* codes) {
    for (int64_t b = 0; b < n_blocks; b++) {
        const float* v = x + b * 32;
        float amax = 0.0f, mx = 0.0f, sum = 0.0f;
        for (int i = 0; i < 32; i++) {
            if (amax < fabsf(v[i])) {
                amax = fabsf(v[i]);
                mx = v[i];
            }
            sum = sum + v[i];
        }
        float scale = mx / 127.0f;
        float r = (scale == 0.0f) ? 0.0f : 1.0f / scale;
        scales[b] = f32_to_f16(scale);
        sums[b] = f32_to_f16(sum);
        for (int i = 0; i < 32; i++) codes[b * 32 + i] = sat_i8(roundf(v[i] * r));
    }
}
// q8_1.rs:50-63 — dequant = code * f32(f16 scale); the sum field is ignored.
void orc_q8_1_dequant(const uint16_t* scales, const int8_t* codes, int64_t n_blocks, float* out) {
    for (int64_t b = 0; b < n_blocks; b++) {
        float d = f16_to_f32(scales[b]);
        for (int i = 0; i < 32; i++) out[b * 32 + i] = (float)codes[b * 32 + i] * d;
    }
}

// ---- a5: Q4_0 block (32 values) -----------------------------------------------
// linalg/src/frame/block_quant/q4_0.rs:19-45; nibble order from helpers.rs:57-68:
// byte j holds element j in the low nibble and element j+16 in the high nibble.
void orc_q4_0_quant(const float* x, int64_t n_blocks, uint16_t* scales, uint8_t* packed /*16 B per block*/) {
    for (int64_t b = 0; b < n_blocks; b++) {
        const float* v = x + b * 32;
        float amax = 0.0f, mx = 0.0f;
        for (int i = 0; i < 32; i++)
            if (amax < fabsf(v[i])) {
                amax = fabsf(v[i]);
                mx = v[i];
            }
        float scale = mx / -8.0f;
        float r = (scale == 0.0f) ? 0.0f : 1.0f / scale;
        scales[b] = f32_to_f16(scale);
        uint8_t nib[32];
        for (int i = 0; i < 32; i++) {
            int8_t c = sat_i8(v[i] * r + 8.5f);
            if (c > 15) c = 15;
            nib[i] = (uint8_t)c;
        }
        for (int j = 0; j < 16; j++) packed[b * 16 + j] = (uint8_t)(nib[j] | (uint8_t)(nib[j + 16] << 4));
    }
}
// q4_0.rs:82-95 — dequant = (nibble - 8) * f32(f16 scale).
void orc_q4_0_dequant(const uint16_t* scales, const uint8_t* packed, int64_t n_blocks, float* out) {
    for (int64_t b = 0; b < n_blocks; b++) {
        float d = f16_to_f32(scales[b]);
        for (int j = 0; j < 16; j++) {
            uint8_t byte = packed[b * 16 + j];
            out[b * 32 + j] = (float)((int8_t)(byte & 0x0f) - 8) * d;
            out[b * 32 + j + 16] = (float)((int8_t)(byte >> 4) - 8) * d;
        }
    }
}

// ---- a3: QuantizedDynKeyValueCache stores (KIVI) ----------------------------
// transformers/src/ops/quant_dyn_kv_cache.rs.  One store per (batch, head).
struct OrcKivi {
    int per_channel;  // 1 = Key store (BlockChannelStore :159-250), 0 = Value store (PerTokenStore :98-149)
    int d, bits, row_bytes;
    std::vector<float> sink;      // first 4 tokens, f32 (:92)
    std::vector<uint8_t> packed;  // codes
    std::vector<float> lo, scale; // value store: one pair per token; key store: D per finalised block
    std::vector<float> residual;  // key store: partial block rows
    int n_res = 0, n_finalized = 0, n_tokens_q = 0;
};

static void kivi_pack(const uint8_t* codes, int d, int bits, std::vector<uint8_t>& out) {  // :63-75
    if (bits == 8) {
        out.insert(out.end(), codes, codes + d);
    } else {
        for (int i = 0; i < d; i += 2) {
            uint8_t lo = codes[i] & 0x0f;
            uint8_t hi = (i + 1 < d) ? (codes[i + 1] & 0x0f) : 0;
            out.push_back((uint8_t)(lo | (hi << 4)));
        }
    }
}
static inline uint8_t kivi_unpack(const uint8_t* row, int c, int bits) {  // :79-88
    if (bits == 8) return row[c];
    uint8_t b = row[c >> 1];
    return (c & 1) == 0 ? (b & 0x0f) : (b >> 4);
}
static inline uint8_t kivi_code(float x, float lo, float scale, float lv) {
    return sat_u8(clampf(roundf((x - lo) / scale), 0.0f, lv));
}
static void kivi_finalize(OrcKivi* s) {  // :197-221
    int d = s->d;
    float lv = (float)((1u << s->bits) - 1);
    std::vector<float> lo(d, std::numeric_limits<float>::infinity()), hi(d, -std::numeric_limits<float>::infinity());
    for (int t = 0; t < s->n_res; t++)
        for (int c = 0; c < d; c++) {
            float v = s->residual[(size_t)t * d + c];
            lo[c] = fminf(lo[c], v);
            hi[c] = fmaxf(hi[c], v);
        }
    std::vector<float> sc(d);
    for (int c = 0; c < d; c++) sc[c] = (hi[c] > lo[c]) ? (hi[c] - lo[c]) / lv : 1.0f;
    std::vector<uint8_t> codes(d);
    for (int t = 0; t < s->n_res; t++) {
        for (int c = 0; c < d; c++) codes[c] = kivi_code(s->residual[(size_t)t * d + c], lo[c], sc[c], lv);
        kivi_pack(codes.data(), d, s->bits, s->packed);
    }
    s->lo.insert(s->lo.end(), lo.begin(), lo.end());
    s->scale.insert(s->scale.end(), sc.begin(), sc.end());
    s->residual.clear();
    s->n_res = 0;
    s->n_finalized++;
}

void* orc_kivi_new(int per_channel, int d, int bits) {
    OrcKivi* s = new OrcKivi();
    s->per_channel = per_channel;
    s->d = d;
    s->bits = bits;
    s->row_bytes = (d * bits + 7) / 8;
    return s;
}
void orc_kivi_free(void* p) { delete (OrcKivi*)p; }

void orc_kivi_push(void* p, const float* row) {
    OrcKivi* s = (OrcKivi*)p;
    int d = s->d;
    if ((int)(s->sink.size() / d) < 4) {  // SINK_TOKENS
        s->sink.insert(s->sink.end(), row, row + d);
        return;
    }
    if (s->per_channel) {  // :183-196
        s->residual.insert(s->residual.end(), row, row + d);
        s->n_res++;
        if (s->n_res == 32) kivi_finalize(s);
    } else {  // :118-131
        float lv = (float)((1u << s->bits) - 1);
        float lo = std::numeric_limits<float>::infinity(), hi = -std::numeric_limits<float>::infinity();
        for (int c = 0; c < d; c++) {
            lo = fminf(lo, row[c]);
            hi = fmaxf(hi, row[c]);
        }
        float scale = (hi > lo) ? (hi - lo) / lv : 1.0f;
        std::vector<uint8_t> codes(d);
        for (int c = 0; c < d; c++) codes[c] = kivi_code(row[c], lo, scale, lv);
        kivi_pack(codes.data(), d, s->bits, s->packed);
        s->lo.push_back(lo);
        s->scale.push_back(scale);
        s->n_tokens_q++;
    }
}
// n rows of d values, pushed one after the other (the reference ingests token by token, quant_dyn_kv_cache.rs:462-472)
void orc_kivi_push_rows(void* p, const float* rows, int64_t n, int d) {
    for (int64_t i = 0; i < n; i++) orc_kivi_push(p, rows + i * d);
}

int64_t orc_kivi_len(void* p) {
    OrcKivi* s = (OrcKivi*)p;
    int ns = (int)(s->sink.size() / s->d);
    return s->per_channel ? ns + s->n_finalized * 32 + s->n_res : ns + s->n_tokens_q;
}
// Number of quantised tokens (rows of codes), of parameter entries, of residual rows.
void orc_kivi_counts(void* p, int64_t* n_code_rows, int64_t* n_params, int64_t* n_res) {
    OrcKivi* s = (OrcKivi*)p;
    *n_code_rows = (int64_t)(s->packed.size() / s->row_bytes);
    *n_params = (int64_t)s->lo.size();
    *n_res = s->n_res;
}
void orc_kivi_raw(void* p, uint8_t* codes, float* lo, float* scale, float* sink, float* residual) {
    OrcKivi* s = (OrcKivi*)p;
    if (codes && !s->packed.empty()) std::memcpy(codes, s->packed.data(), s->packed.size());
    if (lo && !s->lo.empty()) std::memcpy(lo, s->lo.data(), s->lo.size() * 4);
    if (scale && !s->scale.empty()) std::memcpy(scale, s->scale.data(), s->scale.size() * 4);
    if (sink && !s->sink.empty()) std::memcpy(sink, s->sink.data(), s->sink.size() * 4);
    if (residual && !s->residual.empty()) std::memcpy(residual, s->residual.data(), s->residual.size() * 4);
}
// dequant_all (:132-148, :222-249): sinks, quantised rows as lo + code*scale, residual verbatim.
void orc_kivi_dequant(void* p, float* out) {
    OrcKivi* s = (OrcKivi*)p;
    int d = s->d, rb = s->row_bytes, bits = s->bits;
    int ns = (int)(s->sink.size() / d);
    std::memcpy(out, s->sink.data(), s->sink.size() * 4);
    if (s->per_channel) {
        for (int bi = 0; bi < s->n_finalized; bi++)
            for (int ti = 0; ti < 32; ti++) {
                int g = bi * 32 + ti;
                const uint8_t* src = &s->packed[(size_t)g * rb];
                for (int c = 0; c < d; c++)
                    out[(size_t)(ns + g) * d + c] =
                        s->lo[(size_t)bi * d + c] + (float)kivi_unpack(src, c, bits) * s->scale[(size_t)bi * d + c];
            }
        size_t base = (size_t)(ns + s->n_finalized * 32) * d;
        if (s->n_res) std::memcpy(out + base, s->residual.data(), (size_t)s->n_res * d * 4);
    } else {
        for (int i = 0; i < s->n_tokens_q; i++) {
            const uint8_t* src = &s->packed[(size_t)i * rb];
            for (int c = 0; c < d; c++)
                out[(size_t)(ns + i) * d + c] = s->lo[i] + (float)kivi_unpack(src, c, bits) * s->scale[i];
        }
    }
}

// ---- a7: FlashSdpaOp (the CPU attention the default runtime runs) ---------------
// transformers/src/ops/flash_sdpa.rs:103-163,187-227,239-341.  All tensors f32,
// contiguous: q [B,Hq,S,D], k/v [B,Hkv,T,D], optional mask [Mb,Mh,S,T] (Mb in
// {1,B}, Mh in {1,Hq}), out [B,Hq,S,D].  `has_scale` = 0 uses (D as f32).recip().sqrt().
void orc_flash_sdpa(const float* q, const float* k, const float* v, const float* mask, int B, int Hq, int Hkv,
                    int S, int T, int D, int Mb, int Mh, float scale, int has_scale, int causal, float* out,
                    int threads) {
    float sc = has_scale ? scale : sqrtf(1.0f / (float)D);
    int group = Hq / Hkv;
    parallel_for(B * Hq, threads, [&](int task) {
        int b = task / Hq, qh = task % Hq, kvh = qh / group;
        const float* m = nullptr;
        if (mask) {
            int mb = std::min(b, Mb - 1), mh = std::min(qh, Mh - 1);  // :256-257
            m = mask + ((int64_t)mb * Mh + mh) * S * T;
        }
        attend_one_head(q + ((int64_t)b * Hq + qh) * S * D, D, k + ((int64_t)b * Hkv + kvh) * T * D, D,
                        v + ((int64_t)b * Hkv + kvh) * T * D, D, m, T, S, T, D, sc, causal != 0,
                        out + ((int64_t)b * Hq + qh) * S * D);
    });
}

// Independent cross-check: the naive attention the reference's own tests compare
// against (test-rt/suite-unit/src/sdpa.rs:187-236; flash_sdpa.rs:372-399), in
// float64 so it is not just another ordering of the same f32 roundings.
void orc_naive_sdpa_f64(const float* q, const float* k, const float* v, const float* mask, int B, int Hq, int Hkv,
                        int S, int T, int D, int Mb, int Mh, float scale, int has_scale, int causal, double* out,
                        int threads) {
    double sc = has_scale ? (double)scale : 1.0 / std::sqrt((double)D);
    int group = Hq / Hkv;
    parallel_for(B * Hq, threads, [&](int task) {
        int b = task / Hq, qh = task % Hq, kvh = qh / group;
        const float* kk = k + ((int64_t)b * Hkv + kvh) * T * D;
        const float* vv = v + ((int64_t)b * Hkv + kvh) * T * D;
        const float* m = nullptr;
        if (mask) m = mask + ((int64_t)std::min(b, Mb - 1) * Mh + std::min(qh, Mh - 1)) * S * T;
        std::vector<double> p(T);
        for (int i = 0; i < S; i++) {
            const float* qr = q + (((int64_t)b * Hq + qh) * S + i) * D;
            double mx = -std::numeric_limits<double>::infinity();
            int p_off = T > S ? T - S : 0;
            for (int j = 0; j < T; j++) {
                double acc = 0;
                for (int d = 0; d < D; d++) acc += (double)qr[d] * (double)kk[(int64_t)j * D + d];
                acc *= sc;
                if (causal && j > p_off + i) acc = -std::numeric_limits<double>::infinity();
                if (m) acc += (double)m[(int64_t)i * T + j];
                p[j] = acc;
                mx = std::max(mx, acc);
            }
            double sum = 0;
            for (int j = 0; j < T; j++) {
                p[j] = std::exp(p[j] - mx);
                sum += p[j];
            }
            double* o = out + (((int64_t)b * Hq + qh) * S + i) * D;
            for (int d = 0; d < D; d++) {
                double acc = 0;
                for (int j = 0; j < T; j++) acc += p[j] * (double)vv[(int64_t)j * D + d];
                o[d] = acc / sum;
            }
        }
    });
}

// ---- Q4_0 weights x int8-quantised activations (linalg/src/frame/block_quant/q4_0.rs) ------------------
// Q4_0::quantize_row_q8 (:199-214): per block of 32, scale = max|a| / 127 (1 when the block is all zero),
// q = round(a * (1 / scale)) clamped to +-127 (round half away from zero; a NaN becomes 0 in the cast).
void orc_w4a8_quantize_row(const float* a, int64_t k, int8_t* q, float* scales) {
    for (int64_t b = 0; b < k / 32; b++) {
        const float* blk = a + b * 32;
        float amax = 0.f;
        for (int i = 0; i < 32; i++) amax = std::fmax(amax, std::fabs(blk[i]));  // f32::max ignores a NaN operand
        const float scale = amax > 0.f ? amax / 127.0f : 1.0f;
        scales[b] = scale;
        const float r = 1.0f / scale;
        for (int i = 0; i < 32; i++) q[b * 32 + i] = sat_i8(clampf(std::round(blk[i] * r), -127.f, 127.f));
    }
}

// Q4_0::w4a8_gemm (:260-310; w4a8_gemv :221-254 is the m = 1 case, bit-identical per row): out[m, n] accumulates,
// block after block in ascending order, (dot as f32) * w_scale * a_scale with dot the exact int32 dot product of
// the block's 32 weights (nibble - 8, GGML order: byte j = element j | element 16 + j << 4) and activations.
// `scales` / `packed` are the two halves of every 18-byte block: [n, k/32] f16 bits and [n, k/32, 16] nibble bytes.
void orc_w4a8_gemm(const uint16_t* scales, const uint8_t* packed, int64_t n, int64_t k, const float* a, int64_t m, float* out,
                   int threads) {
    const int64_t nb = k / 32;
    std::vector<int8_t> aq((size_t)(m * k));
    std::vector<float> asc((size_t)(m * nb));
    for (int64_t mi = 0; mi < m; mi++) orc_w4a8_quantize_row(a + mi * k, k, aq.data() + mi * k, asc.data() + mi * nb);
    parallel_for((int)n, threads, [&](int ni) {
        std::vector<float> accs((size_t)m, 0.f);
        int8_t w[32];
        for (int64_t b = 0; b < nb; b++) {
            const uint8_t* blk = packed + ((int64_t)ni * nb + b) * 16;
            const float wscale = f16_to_f32(scales[(int64_t)ni * nb + b]);
            for (int j = 0; j < 16; j++) w[j] = (int8_t)((blk[j] & 0x0F) - 8), w[16 + j] = (int8_t)((blk[j] >> 4) - 8);
            for (int64_t mi = 0; mi < m; mi++) {
                const int8_t* aqb = aq.data() + mi * k + b * 32;
                int32_t dot = 0;
                for (int i = 0; i < 32; i++) dot += (int32_t)w[i] * (int32_t)aqb[i];
                accs[mi] += (float)dot * wscale * asc[mi * nb + b];
            }
        }
        for (int64_t mi = 0; mi < m; mi++) out[mi * n + ni] = accs[mi];
    });
}

// ---- decoder glue: generic tract-linalg kernels -------------------------------------------------------
// rms_norm_f32 (linalg/src/generic/rms_norm.rs:7-18): left-to-right sum of squares, / n, + eps, sqrt, recip, scale.
void orc_rms_norm_f32(float* buf, int64_t rows, int64_t d, float eps) {
    for (int64_t r = 0; r < rows; r++) {
        float* x = buf + r * d;
        float sum_sq = 0.f;
        for (int64_t i = 0; i < d; i++) sum_sq += x[i] * x[i];
        const float inv_std = 1.0f / std::sqrt(sum_sq / (float)d + eps);
        for (int64_t i = 0; i < d; i++) x[i] *= inv_std;
    }
}
// ssigmoid (linalg/src/generic/sigmoid.rs:11-45)
static inline float clamp_keep_nan(float x, float lo, float hi) { return x != x ? x : std::fmin(std::fmax(x, lo), hi); }
static float ssigmoid(float x) {
    x = clamp_keep_nan(x, -18.6f, 18.6f);
    const float x2 = x * x;
    float p = -4.433153405e-18f;
    p = x2 * p + 1.169974371e-14f;
    p = x2 * p + -1.875289645e-11f;
    p = x2 * p + 4.257889523e-8f;
    p = x2 * p + 0.00004811817576f;
    p = x2 * p + 0.008163842030f;
    p = x2 * p + 0.2499999971f;
    p = p * x;
    float q = 3.922935744e-6f;
    q = x2 * q + 0.001524872358f;
    q = x2 * q + 0.1159886749f;
    q = x2 * q + 1.0f;
    return clamp_keep_nan(p / q + 0.5f, 0.f, 1.f);
}
void orc_ssigmoid(const float* x, int64_t n, float* out) {
    for (int64_t i = 0; i < n; i++) out[i] = ssigmoid(x[i]);
}
// SSiLU4::run (linalg/src/generic/silu.rs:26-30): x *= ssigmoid(x)
void orc_silu_f32(const float* x, int64_t n, float* out) {
    for (int64_t i = 0; i < n; i++) out[i] = x[i] * ssigmoid(x[i]);
}

int orc_hardware_threads() { return (int)std::thread::hardware_concurrency(); }

}  // extern "C"
