// Output projection of the decoder ("lm_head"): logits = x . W^T for a dense fp16 W (V, H) kept in the
// row-major layout of the checkpoint, for the few rows of a decode step, with the greedy arg-max folded in.
// The reference leaves this product to the transformers model it wraps and takes the arg-max on the
// host side of every step (inference/graph_wrapper.py:186-208); at a vocabulary of 151936 x 2048 it
// is 622 MB per token, the largest single read of a decode step, so it is a pure HBM stream:
//   * a warp item is 16 vocabulary rows x one quarter of H; the four quarters of a tile are four warps
//     of one CTA, summed through shared memory in a fixed order (deterministic, no atomics);
//   * every lane reads 16 bytes (8 consecutive channels of one row) per load, eight loads in flight;
//     those 8 channels feed two m16n8k16 tensor-core ops as they are: the op's k index is only a
//     summation index, so the activations are read from shared memory in the matching order
//     (lane t of a 32-channel chunk takes channels 8t..8t+7) and nothing is shuffled;
//   * up to 8 activation rows ride along as the op's 8 columns;
//   * arg-max: every CTA keeps the best (fp16-rounded value, lowest index) per activation row, writes
//     it to the workspace, and the CTA that arrives last reduces the CTAs' candidates.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "glq_common.cuh"

using namespace glq;

namespace {

constexpr int kLmSplit = 4;                          // warps sharing one 16-row tile (quarters of H)
constexpr int kLmTilesPerCta = kWarpsPerCta / kLmSplit;
constexpr int kLmDepth = 8;                          // 16-byte loads in flight per lane and row half

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

struct LmParams {
    const __half* x;
    long long ldx;
    const __half* W;
    int B, V, H;
    __half* logits;
    long long ldl;
    long long* argmax_out;
    float* cand_val;      // [grid][8]
    int* cand_idx;        // [grid][8]
    int* counter;
};

__global__ void __launch_bounds__(kThreads, 2) lm_head_kernel(const LmParams p) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    // activation rows are padded by 64 bytes, so that the 16-byte reads of the lanes of a quarter warp (two
    // activation rows x four chunks) fall into distinct banks
    const int HS = p.H + 32;
    __half* xs = reinterpret_cast<__half*>(lm_smem);                              // [8][HS]
    float4* red = reinterpret_cast<float4*>(lm_smem + (size_t)8 * HS * 2);        // [warps][32]
    __shared__ float s_best[kLmTilesPerCta][8];
    __shared__ int s_besti[kLmTilesPerCta][8];
    __shared__ int s_last;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int H = p.H, V = p.V, B = p.B;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // activations: rows beyond B are zero
    for (int i = tid; i < 8 * (H / 8); i += kThreads) {
        const int row = i / (H / 8), c = i % (H / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < B) v = *reinterpret_cast<const uint4*>(p.x + (size_t)row * p.ldx + c * 8);
        *reinterpret_cast<uint4*>(xs + (size_t)row * HS + c * 8) = v;
    }
    __syncthreads();
    const int ntiles = (V + 15) / 16;
    const int tw = w / kLmSplit, s = w % kLmSplit;      // tile slot of the warp in its CTA, quarter of H
    const int chunks = H / 32;                          // 32-channel chunks in H
    const int c_lo = (int)((long)s * chunks / kLmSplit), c_hi = (int)((long)(s + 1) * chunks / kLmSplit);
    // lane (g, t) of column g = activation row g: this lane's best for rows 2t, 2t+1 is kept by the
    // lanes that own those output columns (see the epilogue)
    float best[2] = {-INFINITY, -INFINITY};
    int besti[2] = {0x7fffffff, 0x7fffffff};
    const int iters = (ntiles + kLmTilesPerCta * (int)gridDim.x - 1) / (kLmTilesPerCta * (int)gridDim.x);
    for (int it = 0; it < iters; ++it) {
        const int tile = (it * (int)gridDim.x + (int)blockIdx.x) * kLmTilesPerCta + tw;
        const bool live = tile < ntiles;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
            const int r0 = min(tile * 16 + g, V - 1), r1 = min(tile * 16 + g + 8, V - 1);
            const uint4* w0 = reinterpret_cast<const uint4*>(p.W + (size_t)r0 * H) + t;
            const uint4* w1 = reinterpret_cast<const uint4*>(p.W + (size_t)r1 * H) + t;
            const uint4* xb = reinterpret_cast<const uint4*>(xs + (size_t)g * HS) + t;
            uint4 qa[kLmDepth], qb[kLmDepth];
#pragma unroll
            for (int d = 0; d < kLmDepth; ++d) {
                const int c = c_lo + d;
                if (c < c_hi) {
                    qa[d] = ldg_stream(w0 + c * 4);
                    qb[d] = ldg_stream(w1 + c * 4);
                }
            }
            for (int c0 = c_lo; c0 < c_hi; c0 += kLmDepth) {
#pragma unroll
                for (int d = 0; d < kLmDepth; ++d) {
                    const int c = c0 + d;
                    if (c < c_hi) {
                        const uint4 a = qa[d], b = qb[d];
                        const int cn = c + kLmDepth;
                        if (cn < c_hi) {
                            qa[d] = ldg_stream(w0 + cn * 4);
                            qb[d] = ldg_stream(w1 + cn * 4);
                        }
                        const uint4 xv = xb[c * 4];
                        mma16816(acc, a.x, b.x, a.y, b.y, xv.x, xv.y);
                        mma16816(acc, a.z, b.z, a.w, b.w, xv.z, xv.w);
                    }
                }
            }
        }
        // quarters of H: fixed-order sum through shared memory
        if (s != 0) red[w * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        __syncthreads();
        if (s == 0 && live) {
            for (int s2 = 1; s2 < kLmSplit; ++s2) {
                const float4 v = red[(w + s2) * 32 + lane];
                acc[0] += v.x;
                acc[1] += v.y;
                acc[2] += v.z;
                acc[3] += v.w;
            }
            // acc[0], acc[1]: vocabulary row g, activation rows 2t, 2t+1; acc[2], acc[3]: vocabulary row g+8
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int row = 2 * t + e;
                if (row >= B) continue;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int n = tile * 16 + g + 8 * h;
                    if (n >= V) continue;
                    const __half hv = __float2half_rn(acc[2 * h + e]);
                    if (p.logits) p.logits[(size_t)row * p.ldl + n] = hv;
                    const float v = __half2float(hv);
                    // a value that is not a number never wins, as long as some number is there
                    if (v > best[e] || (v == best[e] && n < besti[e])) best[e] = v, besti[e] = n;
                }
            }
        }
        __syncthreads();
    }
    if (!p.argmax_out) return;
    // the 8 lanes g of one t hold candidates of the same activation rows: reduce over g, then over the tile slots
#pragma unroll
    for (int e = 0; e < 2; ++e) {
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best[e], o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti[e], o);
            if (ov > best[e] || (ov == best[e] && oi < besti[e])) best[e] = ov, besti[e] = oi;
        }
        if (s == 0 && g == 0) {
            s_best[tw][2 * t + e] = best[e];
            s_besti[tw][2 * t + e] = besti[e];
        }
    }
    __syncthreads();
    if (tid < 8) {
        float bv = s_best[0][tid];
        int bi = s_besti[0][tid];
        for (int j = 1; j < kLmTilesPerCta; ++j) {
            const float ov = s_best[j][tid];
            const int oi = s_besti[j][tid];
            if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
        }
        __stcg(&p.cand_val[(size_t)blockIdx.x * 8 + tid], bv);
        __stcg(&p.cand_idx[(size_t)blockIdx.x * 8 + tid], bi);
        __threadfence();
    }
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(p.counter, 1);
        s_last = (old == (int)gridDim.x - 1);
        if (s_last) *p.counter = 0;      // left zero for the next call
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // last CTA: warp r reduces the candidates of activation row r
    if (w < B) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int c = lane; c < (int)gridDim.x; c += 32) {
            const float ov = __ldcg(&p.cand_val[(size_t)c * 8 + w]);
            const int oi = __ldcg(&p.cand_idx[(size_t)c * 8 + w]);
            if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
        }
        if (lane == 0) p.argmax_out[w] = bi == 0x7fffffff ? 0 : bi;
    }
}

int lm_grid() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        sms = 148;
    return 2 * sms;
}

}  // namespace

extern "C" size_t glq_lm_head_workspace_bytes(void) { return (size_t)lm_grid() * 8 * (sizeof(float) + sizeof(int)); }

extern "C" int glq_lm_head(const void* x, int64_t ldx, const void* W, int B, int V, int H, void* logits, int64_t ldl,
                           int64_t* argmax_out, void* workspace, size_t workspace_bytes, int32_t* counter,
                           void* stream) {
    if (!x || !W || B < 0 || V < 0 || H <= 0 || (!logits && !argmax_out)) return GLQ_ERR_ARG;
    if (B == 0 || V == 0) return GLQ_OK;
    if (B > 8 || H % 32 != 0 || H > 8192) return GLQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(W) & 15u) || ldx % 8 != 0 ||
        (reinterpret_cast<uintptr_t>(logits) & 1u) || (reinterpret_cast<uintptr_t>(argmax_out) & 7u))
        return GLQ_ERR_ALIGN;
    const int grid = std::min(lm_grid(), (V + 16 * kLmTilesPerCta - 1) / (16 * kLmTilesPerCta));
    LmParams p{};
    p.x = reinterpret_cast<const __half*>(x);
    p.ldx = ldx;
    p.W = reinterpret_cast<const __half*>(W);
    p.B = B;
    p.V = V;
    p.H = H;
    p.logits = reinterpret_cast<__half*>(logits);
    p.ldl = ldl;
    p.argmax_out = reinterpret_cast<long long*>(argmax_out);
    if (argmax_out) {
        if (!workspace || workspace_bytes < glq_lm_head_workspace_bytes() || !counter) return GLQ_ERR_WORKSPACE;
        if (reinterpret_cast<uintptr_t>(workspace) & 15u) return GLQ_ERR_ALIGN;
        p.cand_val = reinterpret_cast<float*>(workspace);
        p.cand_idx = reinterpret_cast<int*>(p.cand_val + (size_t)lm_grid() * 8);
        p.counter = counter;
    }
    const size_t smem = (size_t)8 * (H + 32) * 2 + (size_t)kWarpsPerCta * 32 * sizeof(float4);
    static size_t configured[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return GLQ_ERR_CUDA;
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || configured[dev] < smem)) {
        if (cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return GLQ_ERR_CUDA;
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    lm_head_kernel<<<grid, kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(p);
    return cudaGetLastError() == cudaSuccess ? GLQ_OK : GLQ_ERR_CUDA;
}
