// Load-time re-tiling kernels, the dequantised-tile check and the int8-code drop-in.
// None of these is on the decode hot path.
#pragma once

#include "glq_common.cuh"

namespace glq {

// ---------------------------------------------------------------------------------------------
// (N,K) int32 codes -> tiled Q2 / Q4.  One thread per output word.
// word index = ((rt*nkb + kb)*32 + lane)*4 + wsel ; lane = 4g+t ; wsel>>1 selects row g / g+8,
// wsel&1 the first / second word of the lane's codes.
// ---------------------------------------------------------------------------------------------
__global__ void pack_codes_i32_kernel(const int32_t* __restrict__ q, int bits, int N, int K,
                                      uint32_t* __restrict__ out, size_t nwords) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nwords) return;
    const int cpw = 32 / bits, kbk = 8 * cpw;  // codes per word, k per block (128 or 64)
    const int nkb = (K + kbk - 1) / kbk;
    const int wsel = idx & 3, lane = (idx >> 2) & 31;
    const size_t blk = idx >> 7;
    const int kb = (int)(blk % nkb), rt = (int)(blk / nkb);
    const int g = lane >> 2, t = lane & 3;
    const int row = rt * 16 + g + 8 * (wsel >> 1);
    const int k0 = kb * kbk + t * 2 * cpw + (wsel & 1) * cpw;
    uint32_t w = 0;
    if (row < N) {
        const uint32_t mask = (1u << bits) - 1u;
        for (int j = 0; j < cpw; ++j)
            if (k0 + j < K) w |= ((uint32_t)q[(size_t)row * K + k0 + j] & mask) << (bits * j);
    }
    out[idx] = w;
}

// (N,K/4) uint8 packed 2-bit codes -> tiled T2 / Q2
__global__ void pack_codes_u8_kernel(const uint8_t* __restrict__ packed, int N, int K, uint32_t* __restrict__ out,
                                     size_t nwords) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nwords) return;
    const int nkb = (K + 127) / 128;
    const int wsel = idx & 3, lane = (idx >> 2) & 31;
    const size_t blk = idx >> 7;
    const int kb = (int)(blk % nkb), rt = (int)(blk / nkb);
    const int g = lane >> 2, t = lane & 3;
    const int row = rt * 16 + g + 8 * (wsel >> 1);
    const int k0 = kb * 128 + t * 32 + (wsel & 1) * 16;
    uint32_t w = 0;
    if (row < N) {
        const int rowbytes = K >> 2;
        for (int b = 0; b < 4; ++b) {
            const int byte = (k0 >> 2) + b;
            if (byte < rowbytes) w |= (uint32_t)packed[(size_t)row * rowbytes + byte] << (8 * b);
        }
    }
    out[idx] = w;
}

// (N,G) fp16 scales, zeros -> [rt][grp][g][s_g, z_g, s_g+8, z_g+8]
__global__ void pack_sz_kernel(const __half* __restrict__ scales, const __half* __restrict__ zeros, int N, int G,
                               __half* __restrict__ out, size_t nelem) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nelem) return;
    const int c = idx & 3, g = (idx >> 2) & 7;
    const size_t blk = idx >> 5;
    const int grp = (int)(blk % G), rt = (int)(blk / G);
    const int row = rt * 16 + g + 8 * (c >> 1);
    __half v = __float2half(0.f);
    if (row < N) {
        if ((c & 1) == 0) v = scales[(size_t)row * G + grp];
        else if (zeros) v = zeros[(size_t)row * G + grp];
    }
    out[idx] = v;
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
__global__ void dequant_tiled_q_kernel(int fmt, const glq_weight_t w, int group_size, __half* __restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)w.N * w.K) return;
    const int n = (int)(idx / w.K), k = (int)(idx % w.K);
    const int bits = fmt == GLQ_FMT_Q2 ? 2 : 4;
    const int cpw = 32 / bits, kbk = 8 * cpw;
    const int nkb = (w.K + kbk - 1) / kbk;
    const int G = (w.K + group_size - 1) / group_size;
    const int rt = n >> 4, rr = n & 15, g = rr & 7, hi = rr >> 3;
    const int kb = k / kbk, kin = k % kbk;
    const int t = kin / (2 * cpw), u = (kin % (2 * cpw)) / cpw, j = kin % cpw;
    const uint32_t word =
        reinterpret_cast<const uint32_t*>(w.codes)[(((size_t)rt * nkb + kb) * 32 + g * 4 + t) * 4 + hi * 2 + u];
    const uint32_t code = (word >> (bits * j)) & ((1u << bits) - 1u);
    const __half* sz = reinterpret_cast<const __half*>(w.sz) + (((size_t)rt * G + k / group_size) * 8 + g) * 4 + hi * 2;
    // fp16 arithmetic step by step, as an fp16 tensor expression evaluates it
    out[idx] = __hmul(__hsub(__ushort2half_rn((unsigned short)code), sz[1]), sz[0]);
}

__global__ void dequant_tiled_t2_kernel(const glq_weight_t w, float* __restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)w.N * w.K) return;
    const int n = (int)(idx / w.K), k = (int)(idx % w.K);
    const int nkb = (w.K + 127) / 128;
    const int rt = n >> 4, rr = n & 15, g = rr & 7, hi = rr >> 3;
    const int kb = k >> 7, kin = k & 127;
    const int t = kin >> 5, u = (kin & 31) >> 4, j = kin & 15;
    const uint32_t word =
        reinterpret_cast<const uint32_t*>(w.codes)[(((size_t)rt * nkb + kb) * 32 + g * 4 + t) * 4 + hi * 2 + u];
    out[idx] = __fmul_rn(w.centroids[(word >> (2 * j)) & 3u], w.norms[n]);
}

// ---------------------------------------------------------------------------------------------
// Drop-in for the reference's int8-code GPTQ module (one byte per weight, arbitrary int8 codes,
// fp32 activations and output): y[b,n] = sum_k (q - z) * s * x[b,k] (+ lora_out[b,n]).
// One warp per output row, 16 codes per lane and step, activations in shared memory, NB <= 4 rows
// of x per launch.
// ---------------------------------------------------------------------------------------------
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
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = lane * 16; k0 < K; k0 += 32 * 16) {
        __align__(16) int8_t c[16];
        if (vec) {
            *reinterpret_cast<uint4*>(c) = __ldg(reinterpret_cast<const uint4*>(qrow + k0));
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) c[j] = (k0 + j < K) ? qrow[k0 + j] : (int8_t)0;
        }
        int gi = -1;
        float sv = 0.f, zv = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int k = k0 + j;
            if (k < K) {
                const int gk = k / groupsize;
                if (gk != gi) {
                    gi = gk;
                    sv = __half2float(scales[(size_t)n * G + gi]);
                    zv = sym ? 0.f : __half2float(zeros[(size_t)n * G + gi]);
                }
                const float wv = ((float)c[j] - zv) * sv;
                for (int b = 0; b < nb; ++b) acc[b] = fmaf(wv, xsm[b * K + k], acc[b]);
            }
        }
    }
    for (int b = 0; b < nb; ++b) {
        const float v = warp_sum(acc[b]);
        if (lane == 0) y[(size_t)b * N + n] = v + (lora_out ? lora_out[(size_t)b * N + n] : 0.f);
    }
}

}  // namespace glq
