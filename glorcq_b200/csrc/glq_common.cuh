// Shared device helpers for the sm_100a kernels: fragment-level dequantisation of packed codes,
// the warp-level tensor-core dot product (used as a dot-product engine; the kernels are HBM-bound),
// reductions and small numeric helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/glorcq_b200.h"

namespace glq {

constexpr int kRowTile = 16;          // rows of one weight tile (the M of m16n8k16)
constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;

// ---------------------------------------------------------------------------------------------
// lop3 / prmt wrappers
// ---------------------------------------------------------------------------------------------
template <int LUT>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(d) : "r"(a), "r"(b), "r"(c), "n"(LUT));
    return d;
}
// (a & b) | c   -> truth table 0xEA
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) { return lop3<0xEA>(a, b, c); }

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// ---------------------------------------------------------------------------------------------
// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
// Fragment ownership for lane = 4*g + t:
//   A: a[0] = (row g,   k 2t,2t+1)   a[1] = (row g+8, k 2t,2t+1)
//      a[2] = (row g,   k 2t+8,+9)   a[3] = (row g+8, k 2t+8,+9)
//   B: b0 = (k 2t,2t+1 ; col g)      b1 = (k 2t+8,2t+9 ; col g)
//   C: c[0],c[1] = (row g ; col 2t,2t+1)   c[2],c[3] = (row g+8 ; col 2t,2t+1)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------------------------
// 2-bit affine codes.  A 32-bit word holds 16 codes, code j in bits [2j, 2j+1].  The word is
// turned into eight half2 values h[j] = (off_j + code_j , off_j + code_{j+8}) by placing the two
// code bits in the mantissa of an fp16 number whose exponent makes one mantissa step worth 1.0:
//   bits at mantissa position 4 -> exponent field 21 -> value 64 + q
//   bits at mantissa position 6 -> exponent field 19 -> value 16 + q
//   bits at mantissa position 8 -> exponent field 17 -> value  4 + q
// Two shifts and eight lop3 per 16 weights.  The constant offsets are removed after the fp32
// accumulation with sum_k off(k) * x_k, computed once per input vector (see q2_offset()).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack_q2(uint32_t w, uint32_t (&h)[8]) {
    const uint32_t w4 = w << 4, w6 = w >> 6;
    h[0] = and_or(w4, 0x00300030u, 0x54005400u);
    h[1] = and_or(w4, 0x00C000C0u, 0x4C004C00u);
    h[2] = and_or(w, 0x00300030u, 0x54005400u);
    h[3] = and_or(w, 0x00C000C0u, 0x4C004C00u);
    h[4] = and_or(w, 0x03000300u, 0x44004400u);
    h[5] = and_or(w6, 0x00300030u, 0x54005400u);
    h[6] = and_or(w6, 0x00C000C0u, 0x4C004C00u);
    h[7] = and_or(w6, 0x03000300u, 0x44004400u);
}
// offset carried by code position j (0..15) of a word after unpack_q2
__host__ __device__ __forceinline__ float q2_offset(int j) {
    const int jj = j & 7;
    return (jj == 4 || jj == 7) ? 4.f : ((jj == 1 || jj == 3 || jj == 6) ? 16.f : 64.f);
}

// ---------------------------------------------------------------------------------------------
// 4-bit affine codes.  A word holds 8 codes, code j in bits [4j, 4j+3].  h[j] = (64 + code_j,
// 64 + code_{j+4}), j = 0..3: the nibble is moved to mantissa bits 4..7 of an fp16 number with
// exponent field 21.  Three shifts and four lop3 per 8 weights; the offset is the same for every
// code, so it folds into the zero point.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack_q4(uint32_t w, uint32_t (&h)[4]) {
    h[0] = and_or(w << 4, 0x00F000F0u, 0x54005400u);
    h[1] = and_or(w, 0x00F000F0u, 0x54005400u);
    h[2] = and_or(w >> 4, 0x00F000F0u, 0x54005400u);
    h[3] = and_or(w >> 8, 0x00F000F0u, 0x54005400u);
}
constexpr float kQ4Offset = 64.f;

// ---------------------------------------------------------------------------------------------
// 2-bit codebook codes ("turbo").  The four codebook values are held as fp16 in two byte tables
// (TL = low bytes, TH = high bytes); prmt looks four codes up at a time.  Output pairs, in the
// order they are consumed: h[0]=(c0,c2) h[1]=(c4,c6) h[2]=(c8,c10) h[3]=(c12,c14)
//                          h[4]=(c1,c3) h[5]=(c5,c7) h[6]=(c9,c11) h[7]=(c13,c15)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack_t2(uint32_t w, uint32_t TL, uint32_t TH, uint32_t (&h)[8]) {
    const uint32_t se = w & 0x33333333u;               // even codes, one per nibble
    const uint32_t so = (w >> 2) & 0x33333333u;        // odd codes
    const uint32_t seh = se | 0x44444444u, soh = so | 0x44444444u;
    uint32_t lo, hi;
    lo = prmt(TL, TH, se);        hi = prmt(TL, TH, seh);
    h[0] = prmt(lo, hi, 0x5140u); h[1] = prmt(lo, hi, 0x7362u);
    lo = prmt(TL, TH, se >> 16);  hi = prmt(TL, TH, seh >> 16);
    h[2] = prmt(lo, hi, 0x5140u); h[3] = prmt(lo, hi, 0x7362u);
    lo = prmt(TL, TH, so);        hi = prmt(TL, TH, soh);
    h[4] = prmt(lo, hi, 0x5140u); h[5] = prmt(lo, hi, 0x7362u);
    lo = prmt(TL, TH, so >> 16);  hi = prmt(TL, TH, soh >> 16);
    h[6] = prmt(lo, hi, 0x5140u); h[7] = prmt(lo, hi, 0x7362u);
}

__device__ __forceinline__ void make_t2_tables(const float* __restrict__ centroids, uint32_t& TL, uint32_t& TH) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t b = __half_as_ushort(__float2half_rn(__ldg(centroids + i)));
        lo |= (b & 0xFFu) << (8 * i);
        hi |= (b >> 8) << (8 * i);
    }
    TL = lo;
    TH = hi;
}

// ---------------------------------------------------------------------------------------------
// small numeric helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float h2f(__half h) { return __half2float(h); }
__device__ __forceinline__ float round16(float v) { return __half2float(__float2half_rn(v)); }

// silu evaluated in fp32 on an fp16 value and rounded back to fp16, as an fp16 tensor op does
__device__ __forceinline__ float silu16(float g16) { return round16(g16 / (1.f + __expf(-g16))); }
__device__ __forceinline__ float sigmoid16(float v16) { return round16(1.f / (1.f + __expf(-v16))); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace glq
