// One decode step of grouped-query attention over a static key/value cache, in one launch: optional
// per-head RMS norm of q and k, rotary embedding (rotate-half convention) of q and of the new key at
// the current position, cache write, softmax(q k^T / sqrt(hd)) v over positions 0..pos.
// The position is read from device memory, so a captured launch serves every step of a replayed graph
// and only the live part of the cache is read.  Host model code around the quantized projections
// (inference/graph_wrapper.py:84-127 drives the transformers attention modules for this).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "glq_common.cuh"

using namespace glq;

namespace {

constexpr int kAttnWarps = 8;

// EPL: head_dim / 32 elements per lane; lane l owns elements [l*EPL, (l+1)*EPL); its rotate-half partner
// (element +- hd/2) sits in lane l ^ 16 at the same offset.
template <int EPL>
__device__ __forceinline__ void rope_norm(float (&v)[EPL], const __half* __restrict__ norm_w, float eps, int hd,
                                          const __half* __restrict__ cs, const __half* __restrict__ sn, int lane) {
    if (norm_w) {   // RMS norm over the head, weight applied, rounded to fp16 as a tensor op does
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) ss += v[i] * v[i];
        ss = warp_sum(ss);
        const float r = rsqrtf(ss / hd + eps);
#pragma unroll
        for (int i = 0; i < EPL; ++i) v[i] = round16(__half2float(norm_w[lane * EPL + i]) * (v[i] * r));
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const float partner = __shfl_xor_sync(0xffffffffu, v[i], 16);
        const float rot = lane < 16 ? -partner : partner;          // rotate_half: (-x2, x1)
        const float c = __half2float(cs[lane * EPL + i]), s = __half2float(sn[lane * EPL + i]);
        v[i] = round16(round16(v[i] * c) + round16(rot * s));
    }
}

template <int EPL>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_decode_kernel(
    const __half* __restrict__ q, const __half* __restrict__ k_new, const __half* __restrict__ v_new,
    const __half* __restrict__ cos_t, const __half* __restrict__ sin_t, const long long* __restrict__ pos_p,
    __half* __restrict__ k_cache, __half* __restrict__ v_cache, __half* __restrict__ out, int n_heads, int n_kv, int max_len,
    const __half* __restrict__ q_norm_w, const __half* __restrict__ k_norm_w, float eps, float* __restrict__ partial,
    int* __restrict__ arrivals) {
    constexpr int HD = EPL * 32;
    const int h = blockIdx.x, b = blockIdx.y, z = blockIdx.z, nsplit = gridDim.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = n_heads / n_kv, kvh = h / group;
    long long pos = *pos_p;
    if (pos < 0) pos = 0;
    if (pos >= max_len) pos = max_len - 1;
    const __half* cs = cos_t + (size_t)pos * HD;
    const __half* sn = sin_t + (size_t)pos * HD;

    float qv[EPL], kn[EPL], vn[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        qv[i] = __half2float(q[((size_t)b * n_heads + h) * HD + lane * EPL + i]);
        kn[i] = __half2float(k_new[((size_t)b * n_kv + kvh) * HD + lane * EPL + i]);
        vn[i] = __half2float(v_new[((size_t)b * n_kv + kvh) * HD + lane * EPL + i]);
    }
    rope_norm<EPL>(qv, q_norm_w, eps, HD, cs, sn, lane);
    rope_norm<EPL>(kn, k_norm_w, eps, HD, cs, sn, lane);
    __half* kc = k_cache + ((size_t)b * n_kv + kvh) * max_len * HD;
    __half* vc = v_cache + ((size_t)b * n_kv + kvh) * max_len * HD;
    if (h % group == 0 && warp == 0 && z == 0) {     // one CTA per key/value head stores the new entry
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            kc[(size_t)pos * HD + lane * EPL + i] = __float2half_rn(kn[i]);
            vc[(size_t)pos * HD + lane * EPL + i] = __float2half_rn(vn[i]);
        }
    }
    const float scale = rsqrtf((float)HD);
    // online softmax per warp over its share of positions 0..pos-1 (the new position is warp 0's, from
    // registers: other CTAs of the group may not have stored it yet)
    float m = -INFINITY, l = 0.f, o[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) o[i] = 0.f;
    auto visit = [&](const float (&kk)[EPL], const float (&vv)[EPL]) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) s += qv[i] * kk[i];
        s = warp_sum(s) * scale;
        const float mn = fmaxf(m, s);
        const float a = __expf(m - mn), p = __expf(s - mn);
        l = l * a + p;
#pragma unroll
        for (int i = 0; i < EPL; ++i) o[i] = o[i] * a + p * vv[i];
        m = mn;
    };
    // this CTA's share of the cached positions (the grid's z dimension splits them)
    const long long per = (pos + nsplit - 1) / nsplit;
    const long long t_lo = (long long)z * per, t_hi = t_lo + per < pos ? t_lo + per : pos;
    // the rows of up to kAhead positions are requested before the first of them is used: the loop is a chain of
    // dependent updates, and one cache round trip per position would set its pace
    constexpr int kAhead = 8;
    for (long long t0 = t_lo + warp; t0 < t_hi; t0 += (long long)kAttnWarps * kAhead) {
        __half kr[kAhead][EPL], vr[kAhead][EPL];
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const long long t = t0 + (long long)u * kAttnWarps;
            if (t < t_hi) {
                if constexpr (EPL == 4) {
                    *reinterpret_cast<uint2*>(kr[u]) = *reinterpret_cast<const uint2*>(kc + (size_t)t * HD + lane * EPL);
                    *reinterpret_cast<uint2*>(vr[u]) = *reinterpret_cast<const uint2*>(vc + (size_t)t * HD + lane * EPL);
                } else {
#pragma unroll
                    for (int i = 0; i < EPL; ++i) {
                        kr[u][i] = kc[(size_t)t * HD + lane * EPL + i];
                        vr[u][i] = vc[(size_t)t * HD + lane * EPL + i];
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const long long t = t0 + (long long)u * kAttnWarps;
            if (t < t_hi) {
                float kk[EPL], vv[EPL];
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    kk[i] = __half2float(kr[u][i]);
                    vv[i] = __half2float(vr[u][i]);
                }
                visit(kk, vv);
            }
        }
    }
    if (warp == 0 && z == 0) visit(kn, vn);
    // combine the warps
    __shared__ float sm_m[kAttnWarps], sm_l[kAttnWarps], sm_o[kAttnWarps][HD];
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) sm_o[warp][lane * EPL + i] = o[i];
    __syncthreads();
    __shared__ int s_last;
    if (warp == 0) {
        float mm = -INFINITY;
        for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, sm_m[w]);
        float ll = 0.f, oo[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) oo[i] = 0.f;
        for (int w = 0; w < kAttnWarps; ++w) {
            const float a = sm_m[w] == -INFINITY ? 0.f : __expf(sm_m[w] - mm);
            ll += sm_l[w] * a;
#pragma unroll
            for (int i = 0; i < EPL; ++i) oo[i] += sm_o[w][lane * EPL + i] * a;
        }
        if (nsplit == 1) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) out[((size_t)b * n_heads + h) * HD + lane * EPL + i] = __float2half_rn(oo[i] / ll);
            return;
        }
        // several CTAs per head: leave (max, sum, weighted values) of this share; the CTA that arrives last
        // (counter per head, reset by it) merges the shares in a fixed order
        float* mine = partial + (((size_t)b * n_heads + h) * nsplit + z) * (HD + 2);
        if (lane == 0) {
            mine[0] = mm;
            mine[1] = ll;
        }
#pragma unroll
        for (int i = 0; i < EPL; ++i) mine[2 + lane * EPL + i] = oo[i];
        __threadfence();
        __syncwarp();
        if (lane == 0) s_last = atomicAdd(arrivals + (size_t)b * n_heads + h, 1) == nsplit - 1;
        __syncwarp();
        if (!s_last) return;
        __threadfence();
        const float* all = partial + ((size_t)b * n_heads + h) * nsplit * (HD + 2);
        float gm = -INFINITY;
        for (int s2 = 0; s2 < nsplit; ++s2) gm = fmaxf(gm, __ldcg(all + (size_t)s2 * (HD + 2)));
        float gl = 0.f, go[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) go[i] = 0.f;
        for (int s2 = 0; s2 < nsplit; ++s2) {
            const float* pp = all + (size_t)s2 * (HD + 2);
            const float pm = __ldcg(pp);
            const float a = pm == -INFINITY ? 0.f : __expf(pm - gm);
            gl += __ldcg(pp + 1) * a;
#pragma unroll
            for (int i = 0; i < EPL; ++i) go[i] += __ldcg(pp + 2 + lane * EPL + i) * a;
        }
#pragma unroll
        for (int i = 0; i < EPL; ++i) out[((size_t)b * n_heads + h) * HD + lane * EPL + i] = __float2half_rn(go[i] / gl);
        if (lane == 0) arrivals[(size_t)b * n_heads + h] = 0;
    }
}

// The prompt's form of the first half of attn_decode_kernel: per (token, head) one warp applies the optional RMS norm
// and the rotary embedding at the token's position to q and k in place, and writes the new keys and values into the
// static cache.  Same arithmetic (rope_norm) as the decode step.
template <int EPL>
__global__ void __launch_bounds__(kAttnWarps * 32) rope_prefill_kernel(
    __half* __restrict__ q, __half* __restrict__ k, const __half* __restrict__ v, const __half* __restrict__ cos_t,
    const __half* __restrict__ sin_t, const long long* __restrict__ positions, __half* __restrict__ k_cache,
    __half* __restrict__ v_cache, int T, int n_heads, int n_kv, int max_len, const __half* __restrict__ q_norm_w,
    const __half* __restrict__ k_norm_w, float eps) {
    constexpr int HD = EPL * 32;
    const int lane = threadIdx.x & 31, hw = blockIdx.y * kAttnWarps + (threadIdx.x >> 5);
    if (hw >= n_heads + 2 * n_kv) return;
    const int bt = blockIdx.x, b = bt / T, t = bt - b * T;
    long long pos = positions[t];
    if (pos < 0) pos = 0;
    if (pos >= max_len) pos = max_len - 1;
    const __half* cs = cos_t + (size_t)pos * HD;
    const __half* sn = sin_t + (size_t)pos * HD;
    float val[EPL];
    if (hw < n_heads) {
        __half* row = q + ((size_t)bt * n_heads + hw) * HD + lane * EPL;
#pragma unroll
        for (int i = 0; i < EPL; ++i) val[i] = __half2float(row[i]);
        rope_norm<EPL>(val, q_norm_w, eps, HD, cs, sn, lane);
#pragma unroll
        for (int i = 0; i < EPL; ++i) row[i] = __float2half_rn(val[i]);
    } else if (hw < n_heads + n_kv) {
        const int kvh = hw - n_heads;
        __half* row = k + ((size_t)bt * n_kv + kvh) * HD + lane * EPL;
        __half* crow = k_cache + (((size_t)b * n_kv + kvh) * max_len + pos) * HD + lane * EPL;
#pragma unroll
        for (int i = 0; i < EPL; ++i) val[i] = __half2float(row[i]);
        rope_norm<EPL>(val, k_norm_w, eps, HD, cs, sn, lane);
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const __half h = __float2half_rn(val[i]);
            row[i] = h;
            crow[i] = h;
        }
    } else {
        const int kvh = hw - n_heads - n_kv;
        const __half* row = v + ((size_t)bt * n_kv + kvh) * HD + lane * EPL;
        __half* crow = v_cache + (((size_t)b * n_kv + kvh) * max_len + pos) * HD + lane * EPL;
#pragma unroll
        for (int i = 0; i < EPL; ++i) crow[i] = row[i];
    }
}

// x_out = x + delta (fp16), h_out = rms_norm(x_out) * w: the residual add and the layer norm that follow the
// attention output projection in a decoder layer, one CTA per row (H <= 8192, a multiple of 8).
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ delta,
                                                          const __half* __restrict__ w, float eps, int H,
                                                          __half* __restrict__ x_out, __half* __restrict__ h_out) {
    const size_t row = (size_t)blockIdx.x * H;
    float val[4][8];
    float ss = 0.f;
#pragma unroll
    for (int step = 0; step < 4; ++step) {
        const int c0 = (step * 256 + threadIdx.x) * 8;
        if (c0 >= H) continue;
        __align__(16) __half a[8], b[8], o[8];
        *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(x + row + c0);
        *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(delta + row + c0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            o[i] = __float2half_rn(__half2float(a[i]) + __half2float(b[i]));
            val[step][i] = __half2float(o[i]);
            ss += val[step][i] * val[step][i];
        }
        *reinterpret_cast<uint4*>(x_out + row + c0) = *reinterpret_cast<const uint4*>(o);
    }
    __shared__ float red[8];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float r = rsqrtf(tot / H + eps);
#pragma unroll
    for (int step = 0; step < 4; ++step) {
        const int c0 = (step * 256 + threadIdx.x) * 8;
        if (c0 >= H) continue;
        __align__(16) __half o[8], wv[8];
        if (w) *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(w + c0);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __float2half_rn(w ? __half2float(wv[i]) * (val[step][i] * r) : val[step][i] * r);
        *reinterpret_cast<uint4*>(h_out + row + c0) = *reinterpret_cast<const uint4*>(o);
    }
}

}  // namespace

extern "C" int glq_add_rmsnorm(const void* x, const void* delta, const void* weight, float eps, int rows, int H, void* x_out,
                               void* h_out, void* stream) {
    if (!x || !delta || !x_out || !h_out || rows < 0 || H <= 0) return GLQ_ERR_ARG;
    if (H % 8 != 0 || H > 8192) return GLQ_ERR_UNSUPPORTED;
    if (rows == 0) return GLQ_OK;
    add_rmsnorm_kernel<<<rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const __half*>(x), reinterpret_cast<const __half*>(delta), reinterpret_cast<const __half*>(weight), eps,
        H, reinterpret_cast<__half*>(x_out), reinterpret_cast<__half*>(h_out));
    return cudaGetLastError() == cudaSuccess ? GLQ_OK : GLQ_ERR_CUDA;
}

// position splits per head: enough CTAs to fill the device for long caches
static int attn_splits(int B, int n_heads, int max_len) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int s = (2 * sms + B * n_heads - 1) / (B * n_heads);
    s = std::max(1, std::min(s, 16));
    return std::min(s, std::max(1, max_len / 64));
}

extern "C" size_t glq_attn_decode_workspace_bytes(int B, int n_heads, int head_dim, int max_len) {
    if (B <= 0 || n_heads <= 0 || head_dim <= 0) return 0;
    const int s = attn_splits(B, n_heads, max_len);
    return s == 1 ? 0 : (size_t)B * n_heads * s * (head_dim + 2) * sizeof(float);
}

extern "C" int glq_attn_decode(const void* q, const void* k_new, const void* v_new, const void* cos_t, const void* sin_t,
                               const int64_t* pos, void* k_cache, void* v_cache, void* out, int B, int n_heads, int n_kv,
                               int head_dim, int max_len, const void* q_norm_w, const void* k_norm_w, float eps,
                               void* workspace, size_t workspace_bytes, int32_t* counters, size_t n_counters,
                               void* stream) {
    if (!q || !k_new || !v_new || !cos_t || !sin_t || !pos || !k_cache || !v_cache || !out) return GLQ_ERR_ARG;
    if (B < 0 || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || max_len <= 0) return GLQ_ERR_ARG;
    if (B == 0) return GLQ_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int nsplit = attn_splits(B, n_heads, max_len);
    if (nsplit > 1) {
        if (!workspace || workspace_bytes < glq_attn_decode_workspace_bytes(B, n_heads, head_dim, max_len)) return GLQ_ERR_WORKSPACE;
        if (!counters || n_counters < (size_t)B * n_heads) return GLQ_ERR_WORKSPACE;
    }
    const dim3 grid(n_heads, B, nsplit), block(kAttnWarps * 32);
#define GLQ_ATTN(EPL)                                                                                              \
    attn_decode_kernel<EPL><<<grid, block, 0, st>>>(                                                               \
        reinterpret_cast<const __half*>(q), reinterpret_cast<const __half*>(k_new), reinterpret_cast<const __half*>(v_new), \
        reinterpret_cast<const __half*>(cos_t), reinterpret_cast<const __half*>(sin_t),                           \
        reinterpret_cast<const long long*>(pos), reinterpret_cast<__half*>(k_cache), reinterpret_cast<__half*>(v_cache), \
        reinterpret_cast<__half*>(out), n_heads, n_kv, max_len, reinterpret_cast<const __half*>(q_norm_w),         \
        reinterpret_cast<const __half*>(k_norm_w), eps, reinterpret_cast<float*>(workspace), counters)
    switch (head_dim) {
        case 32: GLQ_ATTN(1); break;
        case 64: GLQ_ATTN(2); break;
        case 128: GLQ_ATTN(4); break;
        case 256: GLQ_ATTN(8); break;
        default: return GLQ_ERR_UNSUPPORTED;
    }
#undef GLQ_ATTN
    return cudaGetLastError() == cudaSuccess ? GLQ_OK : GLQ_ERR_CUDA;
}

extern "C" int glq_rope_prefill(void* q, void* k, const void* v, const void* cos_t, const void* sin_t, const int64_t* positions,
                                void* k_cache, void* v_cache, int B, int T, int n_heads, int n_kv, int head_dim, int max_len,
                                const void* q_norm_w, const void* k_norm_w, float eps, void* stream) {
    if (!q || !k || !v || !cos_t || !sin_t || !positions || !k_cache || !v_cache) return GLQ_ERR_ARG;
    if (B < 0 || T < 0 || n_heads <= 0 || n_kv <= 0 || max_len <= 0) return GLQ_ERR_ARG;
    if (B == 0 || T == 0) return GLQ_OK;
    const dim3 grid(B * T, (n_heads + 2 * n_kv + kAttnWarps - 1) / kAttnWarps);
    auto st = reinterpret_cast<cudaStream_t>(stream);
#define GLQ_ROPE_CASE(EPL)                                                                                                  \
    rope_prefill_kernel<EPL><<<grid, kAttnWarps * 32, 0, st>>>(                                                             \
        reinterpret_cast<__half*>(q), reinterpret_cast<__half*>(k), reinterpret_cast<const __half*>(v),                     \
        reinterpret_cast<const __half*>(cos_t), reinterpret_cast<const __half*>(sin_t),                                     \
        reinterpret_cast<const long long*>(positions), reinterpret_cast<__half*>(k_cache), reinterpret_cast<__half*>(v_cache), \
        T, n_heads, n_kv, max_len, reinterpret_cast<const __half*>(q_norm_w), reinterpret_cast<const __half*>(k_norm_w), eps)
    switch (head_dim) {
        case 32: GLQ_ROPE_CASE(1); break;
        case 64: GLQ_ROPE_CASE(2); break;
        case 128: GLQ_ROPE_CASE(4); break;
        case 256: GLQ_ROPE_CASE(8); break;
        default: return GLQ_ERR_UNSUPPORTED;
    }
#undef GLQ_ROPE_CASE
    return cudaGetLastError() == cudaSuccess ? GLQ_OK : GLQ_ERR_CUDA;
}
