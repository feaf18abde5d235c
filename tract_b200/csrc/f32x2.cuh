// Two f32 values in a 64-bit register pair and the packed IEEE operations of sm_100 on them (add / mul / fma .rn.f32x2):
// each lane is rounded to nearest on its own, exactly as the scalar instruction would, at half the instruction count.
// Packing two registers that sit side by side costs nothing; the compiler places the halves.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace b200kv {

__device__ inline uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ inline uint64_t f2_pack_bits(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ inline float2 f2_unpack(uint64_t v) {
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
    return r;
}
__device__ inline uint2 f2_unpack_bits(uint64_t v) {
    uint2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(r.x), "=r"(r.y) : "l"(v));
    return r;
}
__device__ inline uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ inline uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ inline uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {  // a * b + c
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// 2^x for two values on the FMA pipe (the MUFU unit takes 8 cycles per warp instruction and is the scarce resource of a
// softmax): x is clamped to >= -126, split into the nearest integer r (the low bits of x + 1.5 * 2^23) and f = x - r in
// [-0.5, 0.5]; 2^f is a degree-4 polynomial (relative error 2.6e-6, fitted for the maximum error over the interval), and
// r goes into the exponent field with one shift-add.  x must be below 128.
__device__ inline float2 exp2_poly2(uint64_t x2) {
    const float2 xs = f2_unpack(x2);
    const uint64_t x = f2_pack(fmaxf(xs.x, -126.f), fmaxf(xs.y, -126.f));
    const uint64_t t = f2_add(x, f2_pack(12582912.f, 12582912.f));
    const uint64_t r = f2_add(t, f2_pack(-12582912.f, -12582912.f));
    const uint64_t f = f2_fma(r, f2_pack(-1.f, -1.f), x);
    uint64_t p = f2_fma(f2_pack(0.009570101276040077f, 0.009570101276040077f), f, f2_pack(0.05591785907745361f, 0.05591785907745361f));
    p = f2_fma(p, f, f2_pack(0.240247443318367f, 0.240247443318367f));
    p = f2_fma(p, f, f2_pack(0.6931217908859253f, 0.6931217908859253f));
    p = f2_fma(p, f, f2_pack(0.9999992847442627f, 0.9999992847442627f));
    const uint2 tb = f2_unpack_bits(t), pb = f2_unpack_bits(p);
    return make_float2(__uint_as_float(pb.x + (tb.x << 23)), __uint_as_float(pb.y + (tb.y << 23)));
}
__device__ inline float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

}  // namespace b200kv
