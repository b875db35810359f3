// Load-time re-tiling kernels, the dequantised-tile check and the int8-code drop-in.
// None of these is on the decode hot path.
#pragma once

#include "glq_common.cuh"

namespace glq {

// ---------------------------------------------------------------------------------------------
// Pair-interleaved tiled layout of the quantized formats.  Source row tile i of a matrix goes to
// destination tile d = i*count + slot (count = 2 interleaves two matrices, e.g. gate and up);
// destination pair = d/2, j = d%2.  Block (pair, kb, j) starts at ((pair*nkb + kb)*2 + j)*BB bytes,
// BB = 576 (affine) or 512 (codebook): 32 lanes x 16 B of codes, lane = 4g+t holding codes
// k = KB*kb + (KB/4)*t + 0..KB/4-1 of row 16i+g (words 0,1) and of row 16i+g+8 (words 2,3); then,
// affine formats only, 8 x (scale g, zero g, scale g+8, zero g+8) fp16 of the group of block kb.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ size_t tiled_block_offset(int src_tile, int slot, int count, int kb, int nkb, int bb) {
    const int d = src_tile * count + slot;
    return (((size_t)(d >> 1) * nkb + kb) * 2 + (d & 1)) * bb;
}

// one thread per 32-bit word of the destination blocks of one source matrix
__global__ void pack_gptq_kernel(const int32_t* __restrict__ q, const __half* __restrict__ scales,
                                 const __half* __restrict__ zeros, int bits, int N, int K, int group_size,
                                 unsigned char* __restrict__ out, int slot, int count) {
    const int cpw = 32 / bits, kbk = 8 * cpw;
    const int nkb = (K + kbk - 1) / kbk, ntiles = (N + 15) / 16;
    const int G = (K + group_size - 1) / group_size;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)ntiles * nkb * 144;  // 144 words per block
    if (idx >= total) return;
    const int wsel = (int)(idx % 144);
    const size_t blk = idx / 144;
    const int kb = (int)(blk % nkb), tile = (int)(blk / nkb);
    uint32_t word = 0;
    if (wsel < 128) {
        const int lane = wsel >> 2, ws = wsel & 3;
        const int g = lane >> 2, t = lane & 3;
        const int row = tile * 16 + g + 8 * (ws >> 1);
        const int k0 = kb * kbk + t * 2 * cpw + (ws & 1) * cpw;
        if (row < N) {
            const uint32_t mask = (1u << bits) - 1u;
            for (int j = 0; j < cpw; ++j)
                if (k0 + j < K) word |= ((uint32_t)q[(size_t)row * K + k0 + j] & mask) << (bits * j);
        }
    } else {
        const int e = wsel - 128;           // 16 words: 8 x (s_g, z_g) (s_g8, z_g8)
        const int g = e >> 1, row = tile * 16 + g + 8 * (e & 1);
        const int grp = min((kb * kbk) / group_size, G - 1);
        if (row < N) {
            const unsigned short sv = __half_as_ushort(scales[(size_t)row * G + grp]);
            const unsigned short zv = zeros ? __half_as_ushort(zeros[(size_t)row * G + grp]) : (unsigned short)0;
            word = (uint32_t)sv | ((uint32_t)zv << 16);
        }
    }
    reinterpret_cast<uint32_t*>(out + tiled_block_offset(tile, slot, count, kb, nkb, 576))[wsel] = word;
}

// (N,K/4) uint8 packed 2-bit codes -> tiled codebook format
__global__ void pack_turbo_kernel(const uint8_t* __restrict__ packed, int N, int K, unsigned char* __restrict__ out,
                                  int slot, int count) {
    const int nkb = (K + 127) / 128, ntiles = (N + 15) / 16;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)ntiles * nkb * 128;
    if (idx >= total) return;
    const int wsel = (int)(idx & 127);
    const size_t blk = idx >> 7;
    const int kb = (int)(blk % nkb), tile = (int)(blk / nkb);
    const int lane = wsel >> 2, ws = wsel & 3;
    const int g = lane >> 2, t = lane & 3;
    const int row = tile * 16 + g + 8 * (ws >> 1);
    const int k0 = kb * 128 + t * 32 + (ws & 1) * 16;
    uint32_t word = 0;
    if (row < N) {
        const int rowbytes = K >> 2;
        for (int b = 0; b < 4; ++b) {
            const int byte = (k0 >> 2) + b;
            if (byte < rowbytes) word |= (uint32_t)packed[(size_t)row * rowbytes + byte] << (8 * b);
        }
    }
    reinterpret_cast<uint32_t*>(out + tiled_block_offset(tile, slot, count, kb, nkb, 512))[wsel] = word;
}

// clear the padding tile of an odd tile count (destination tile d_total, if d_total is odd)
__global__ void clear_bytes_kernel(unsigned char* __restrict__ p, size_t n) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) p[idx] = 0;
}

// per-row fp32 values (norms) -> tile order: out[(i*count + slot)*16 + r] = v[16i + r]
__global__ void pack_rows_f32_kernel(const float* __restrict__ v, int N, float* __restrict__ out, int slot, int count) {
    const int ntiles = (N + 15) / 16;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= ntiles * 16) return;
    const int tile = idx >> 4, r = idx & 15, row = tile * 16 + r;
    out[(size_t)(tile * count + slot) * 16 + r] = row < N ? v[row] : 0.f;
}

// SV (N, rank) fp16 -> [pair][64-column slice][32 rows of the pair][64 columns]
__global__ void pack_sv_kernel(const __half* __restrict__ sv, int N, int rank, __half* __restrict__ out, int slot,
                               int count) {
    const int ntiles = (N + 15) / 16, ns = (rank + 63) / 64;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)ntiles * ns * 16 * 64;
    if (idx >= total) return;
    const int c = (int)(idx & 63), r = (int)((idx >> 6) & 15);
    const size_t rest = idx >> 10;
    const int sl = (int)(rest % ns), tile = (int)(rest / ns);
    const int row = tile * 16 + r, col = sl * 64 + c;
    const int d = tile * count + slot;
    const __half v = (row < N && col < rank) ? sv[(size_t)row * rank + col] : __float2half(0.f);
    out[((((size_t)(d >> 1) * ns + sl) * 32) + (d & 1) * 16 + r) * 64 + c] = v;
}

// fp16 matrix (element (n,k) at W[n*stride_n + k*stride_k]) -> tiled m16n8k16 A fragments
__global__ void pack_f16_kernel(const __half* __restrict__ W, long stride_n, long stride_k, int N, int K,
                                __half* __restrict__ out, size_t nelem) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nelem) return;
    const int e = idx & 7, lane = (idx >> 3) & 31, ks = (idx >> 8) & 3;
    const size_t blk = idx >> 10;
    const int nkb = (K + 63) / 64;
    const int kb = (int)(blk % nkb), rt = (int)(blk / nkb);
    const int g = lane >> 2, t = lane & 3, reg = e >> 1;
    const int row = rt * 16 + g + 8 * (reg & 1);
    const int k = kb * 64 + ks * 16 + 2 * t + 8 * (reg >> 1) + (e & 1);
    out[idx] = (row < N && k < K) ? W[(size_t)row * stride_n + (size_t)k * stride_k] : __float2half(0.f);
}

// ---------------------------------------------------------------------------------------------
// Dequantised weights from the tiled layout (checks only).
// ---------------------------------------------------------------------------------------------
__global__ void dequant_tiled_q_kernel(int fmt, const unsigned char* __restrict__ tiled, int N, int K, int slot,
                                       int count, __half* __restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)N * K) return;
    const int n = (int)(idx / K), k = (int)(idx % K);
    const int bits = fmt == GLQ_FMT_Q2 ? 2 : 4;
    const int cpw = 32 / bits, kbk = 8 * cpw;
    const int nkb = (K + kbk - 1) / kbk;
    const int tile = n >> 4, rr = n & 15, g = rr & 7, hi = rr >> 3;
    const int kb = k / kbk, kin = k % kbk;
    const int t = kin / (2 * cpw), u = (kin % (2 * cpw)) / cpw, j = kin % cpw;
    const unsigned char* blk = tiled + tiled_block_offset(tile, slot, count, kb, nkb, 576);
    const uint32_t word = reinterpret_cast<const uint32_t*>(blk)[(g * 4 + t) * 4 + hi * 2 + u];
    const uint32_t code = (word >> (bits * j)) & ((1u << bits) - 1u);
    const __half* sz = reinterpret_cast<const __half*>(blk + 512) + g * 4 + hi * 2;
    // fp16 arithmetic step by step, as an fp16 tensor expression evaluates it
    out[idx] = __hmul(__hsub(__ushort2half_rn((unsigned short)code), sz[1]), sz[0]);
}

__global__ void dequant_tiled_t2_kernel(const unsigned char* __restrict__ tiled, const float* __restrict__ norms_t,
                                        const float* __restrict__ centroids, int N, int K, int slot, int count,
                                        float* __restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)N * K) return;
    const int n = (int)(idx / K), k = (int)(idx % K);
    const int nkb = (K + 127) / 128;
    const int tile = n >> 4, rr = n & 15, g = rr & 7, hi = rr >> 3;
    const int kb = k >> 7, kin = k & 127;
    const int t = kin >> 5, u = (kin & 31) >> 4, j = kin & 15;
    const unsigned char* blk = tiled + tiled_block_offset(tile, slot, count, kb, nkb, 512);
    const uint32_t word = reinterpret_cast<const uint32_t*>(blk)[(g * 4 + t) * 4 + hi * 2 + u];
    out[idx] = __fmul_rn(centroids[(word >> (2 * j)) & 3u], norms_t[(size_t)(tile * count + slot) * 16 + rr]);
}

// ---------------------------------------------------------------------------------------------
// Drop-in for the reference's int8-code GPTQ module (one byte per weight, arbitrary int8 codes,
// fp32 activations and output): y[b,n] = sum_k (q - z) * s * x[b,k] (+ lora_out[b,n]).
// One warp per output row; a lane owns 16 consecutive codes of every 512-code step and requests up to
// four steps' codes (64 bytes) before it consumes the first, so that a row's whole 2 KB .. 16 KB is in
// flight at once; activations of NB <= 8 rows in shared memory (fp32); the group's scale and zero point
// are looked up once per 16 codes (16 divides the group sizes in use; otherwise per code).
// ---------------------------------------------------------------------------------------------
template <int NB>
__global__ void __launch_bounds__(kThreads) gptq_i8_kernel(const float* __restrict__ x, const int8_t* __restrict__ q,
                                                           const __half* __restrict__ scales,
                                                           const __half* __restrict__ zeros,
                                                           const float* __restrict__ lora_out, float* __restrict__ y,
                                                           int nb, int N, int K, int groupsize, int G, int sym) {
    extern __shared__ float xsm[];
    for (int i = threadIdx.x; i < nb * K; i += blockDim.x) xsm[i] = x[i];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (n >= N) return;
    const int8_t* qrow = q + (size_t)n * K;
    const bool vec = ((reinterpret_cast<uintptr_t>(qrow) & 15u) == 0) && (K % 16 == 0);
    const bool group16 = groupsize % 16 == 0;
    float acc[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[b] = 0.f;
    constexpr int kAhead = 4;
    for (int k00 = lane * 16; k00 < K; k00 += kAhead * 32 * 16) {
        __align__(16) int8_t c[kAhead][16];
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            const int k0 = k00 + a * 32 * 16;
            if (vec && k0 < K) {
                *reinterpret_cast<uint4*>(c[a]) = __ldg(reinterpret_cast<const uint4*>(qrow + k0));
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) c[a][j] = (k0 + j < K) ? qrow[k0 + j] : (int8_t)0;
            }
        }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            const int k0 = k00 + a * 32 * 16;
            if (k0 >= K) break;
            int gi = -1;
            float sv = 0.f, zv = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int k = k0 + j;
                if (k < K) {
                    if (j == 0 || !group16) {
                        const int gk = k / groupsize;
                        if (gk != gi) {
                            gi = gk;
                            sv = __half2float(scales[(size_t)n * G + gi]);
                            zv = sym ? 0.f : __half2float(zeros[(size_t)n * G + gi]);
                        }
                    }
                    const float wv = ((float)c[a][j] - zv) * sv;
#pragma unroll
                    for (int b = 0; b < NB; ++b)
                        if (b < nb) acc[b] = fmaf(wv, xsm[b * K + k], acc[b]);
                }
            }
        }
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        if (b >= nb) break;
        const float v = warp_sum(acc[b]);
        if (lane == 0) y[(size_t)b * N + n] = v + (lora_out ? lora_out[(size_t)b * N + n] : 0.f);
    }
}

// ---------------------------------------------------------------------------------------------
// Randomized Hadamard rotation: y = scale * H_n * (signs . x) over one row, H_n the Sylvester-ordered
// Walsh-Hadamard matrix of the next power of two n >= d; the input is zero-padded to n and the first d
// outputs are kept.  One CTA per row; the butterflies run in fp32 in shared memory (n floats).
// ---------------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) rht_kernel(const TI* __restrict__ x, long long ldx, const float* __restrict__ signs,
                                                  int d, int n, float scale, TO* __restrict__ y, long long ldy) {
    extern __shared__ float rht_buf[];
    const TI* xr = x + (size_t)blockIdx.x * ldx;
    for (int i = threadIdx.x; i < n; i += blockDim.x) rht_buf[i] = i < d ? (float)xr[i] * __ldg(signs + i) : 0.f;
    __syncthreads();
    for (int h = 1; h < n; h <<= 1) {
        for (int p = threadIdx.x; p < (n >> 1); p += blockDim.x) {
            const int i = ((p / h) * 2 * h) + (p % h);
            const float a = rht_buf[i], b = rht_buf[i + h];
            rht_buf[i] = a + b;
            rht_buf[i + h] = a - b;
        }
        __syncthreads();
    }
    TO* yr = y + (size_t)blockIdx.x * ldy;
    for (int i = threadIdx.x; i < d; i += blockDim.x) yr[i] = (TO)(rht_buf[i] * scale);
}

}  // namespace glq
