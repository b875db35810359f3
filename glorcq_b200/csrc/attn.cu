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

// ---------------------------------------------------------------------------------------------
// Causal attention of a prompt written at positions 0..T-1: y[t] = softmax(q[t] . k[0..t]^T / sqrt(hd)) v[0..t] per
// (batch, head), keys and values of the head's group (grouped-query attention).  One CTA = 64 queries of one head
// (four warps x 16 rows), key blocks of 64 up to the diagonal only; scores and the weighted values on the fp16
// `mma.m16n8k16` op with fp32 accumulators, softmax in base 2 with a running row maximum and row sum in registers
// (the probabilities are rounded to fp16 as the second product's operand), key / value blocks double-buffered in
// shared memory by 16-byte asynchronous copies (rows past T arrive as zeros).  q (B, T, n_heads, HD),
// k / v (B, T, n_kv, HD), y (B, T, n_heads, HD): the layout the projections write and the output projection reads.
// (inference/graph_wrapper.py:84-127 leaves this to the transformers attention modules.)
template <int HD>
struct PrefillCfg {
    static constexpr int BM = 64, BN = 64, LD = HD + 8;          // 16-byte pad per row: conflict-free fragment reads
    static constexpr int STAGE = 2 * BN * LD;                    // halfs per stage: keys, then values
    static constexpr size_t SMEM = (size_t)2 * STAGE * sizeof(__half);
};

__device__ __forceinline__ uint32_t pf_smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool live) {
    const int bytes = live ? 16 : 0;     // 0: the 16 bytes are filled with zeros, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// 2^x by the special-function unit alone (2 ulp; -inf -> 0; results below the normal range flush to zero)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int HD>
__global__ void __launch_bounds__(128, 3) attn_prefill_kernel(const __half* __restrict__ q, const __half* __restrict__ k,
                                                           const __half* __restrict__ v, __half* __restrict__ y, int B,
                                                           int T, int n_heads, int n_kv) {
    using C = PrefillCfg<HD>;
    constexpr int LD = C::LD, KS = HD / 16, NT = HD / 8;
    extern __shared__ __align__(16) unsigned char pf_smem[];
    __half* sm = reinterpret_cast<__half*>(pf_smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // launch order = work order: the query blocks with the most keys first, over all heads and batch rows
    const int n_hb = n_heads * B;
    const int qb = (int)(gridDim.x / n_hb) - 1 - (int)(blockIdx.x / n_hb);
    const int h = (int)(blockIdx.x % n_hb) % n_heads, b = (int)(blockIdx.x % n_hb) / n_heads;
    const int kvh = h / (n_heads / n_kv);
    const int q0 = qb * C::BM + warp * 16;                      // first query row of this warp
    const __half* kbase = k + ((size_t)b * T * n_kv + kvh) * HD;
    const __half* vbase = v + ((size_t)b * T * n_kv + kvh) * HD;
    const size_t kv_row = (size_t)n_kv * HD;

    auto load_block = [&](int kb, int stage) {
        __half* ks = sm + (size_t)stage * C::STAGE;
        __half* vs = ks + C::BN * LD;
        for (int idx = tid; idx < C::BN * (HD / 8); idx += 128) {
            const int r = idx / (HD / 8), c = idx % (HD / 8);
            const int key = kb * C::BN + r;
            const bool live = key < T;
            const size_t off = (size_t)(live ? key : 0) * kv_row + c * 8;
            cp_async_16(pf_smem_addr(ks + r * LD + c * 8), kbase + off, live);
            cp_async_16(pf_smem_addr(vs + r * LD + c * 8), vbase + off, live);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    const int nkb = qb + 1;            // key blocks 0 .. qb (BM == BN)
    load_block(0, 0);

    // the warp's 16 query rows as the first operand's fragments: rows g and g + 8, channels 16*ks + 2t (+8)
    uint32_t qf[KS][4];
    {
        const int r0 = q0 + g, r1 = q0 + g + 8;
        const __half* p0 = q + (((size_t)b * T + min(r0, T - 1)) * n_heads + h) * HD;
        const __half* p1 = q + (((size_t)b * T + min(r1, T - 1)) * n_heads + h) * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = r0 < T ? *reinterpret_cast<const uint32_t*>(p0 + 16 * ks + 2 * t) : 0u;
            qf[ks][1] = r1 < T ? *reinterpret_cast<const uint32_t*>(p1 + 16 * ks + 2 * t) : 0u;
            qf[ks][2] = r0 < T ? *reinterpret_cast<const uint32_t*>(p0 + 16 * ks + 8 + 2 * t) : 0u;
            qf[ks][3] = r1 < T ? *reinterpret_cast<const uint32_t*>(p1 + 16 * ks + 8 + 2 * t) : 0u;
        }
    }
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;     // rows g and g + 8: running maximum, this lane's share of the sum
    const float sc = rsqrtf((float)HD) * 1.4426950408889634f;     // scores in base 2

    for (int kb = 0; kb < nkb; ++kb) {
        if (kb + 1 < nkb) {
            load_block(kb + 1, (kb + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __half* ks_ = sm + (size_t)(kb & 1) * C::STAGE;
        const __half* vs_ = ks_ + C::BN * LD;
        // a warp whose rows all lie before this key block has nothing to add (only in the diagonal block, never)
        float sacc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[j][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            // keys as the second operand: 8x8 matrix loads, rows = keys (two 8-key tiles x two channel halves each)
            const int krow = (lane & 7) + (lane >> 4) * 8, kcol = 16 * ks + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(pf_smem_addr(ks_ + (16 * jp + krow) * LD + kcol), b0, b1, b2, b3);
                mma16816(sacc[2 * jp], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma16816(sacc[2 * jp + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }
        }
        // scale; the diagonal block hides keys after the query and keys past T
        const bool diag = kb == nkb - 1;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float sv = sacc[j][e] * sc;
                if (diag) {
                    const int key = kb * C::BN + 8 * j + 2 * t + (e & 1);
                    const int row = q0 + g + 8 * (e >> 1);
                    if (key > row || key >= T) sv = -INFINITY;
                }
                sacc[j][e] = sv;
                if (e < 2) mx0 = fmaxf(mx0, sv);
                else mx1 = fmaxf(mx1, sv);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        // a row with nothing visible so far keeps a zero offset (its probabilities are all exp2(-inf) = 0)
        const float f0 = n0 == -INFINITY ? 0.f : n0, f1 = n1 == -INFINITY ? 0.f : n1;
        const float a0 = ex2_approx(m0 - f0), a1 = ex2_approx(m1 - f1);
        m0 = n0;
        m1 = n1;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            sacc[j][0] = ex2_approx(sacc[j][0] - f0);
            sacc[j][1] = ex2_approx(sacc[j][1] - f0);
            sacc[j][2] = ex2_approx(sacc[j][2] - f1);
            sacc[j][3] = ex2_approx(sacc[j][3] - f1);
            s0 += sacc[j][0] + sacc[j][1];
            s1 += sacc[j][2] + sacc[j][3];
        }
        l0 = l0 * a0 + s0;
        l1 = l1 * a1 + s1;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            o[j][0] *= a0;
            o[j][1] *= a0;
            o[j][2] *= a1;
            o[j][3] *= a1;
        }
        // weighted values: probabilities as the first operand (keys 16*kk .. +15), values through transposing
        // 8x8 matrix loads (rows = keys, two 8-channel tiles per instruction)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const uint32_t pa0 = pack_half2(sacc[2 * kk][0], sacc[2 * kk][1]);
            const uint32_t pa1 = pack_half2(sacc[2 * kk][2], sacc[2 * kk][3]);
            const uint32_t pa2 = pack_half2(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
            const uint32_t pa3 = pack_half2(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
            const int vrow = 16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int jp = 0; jp < NT / 2; ++jp) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(pf_smem_addr(vs_ + vrow * LD + 16 * jp + (lane >> 4) * 8), b0, b1, b2, b3);
                mma16816(o[2 * jp], pa0, pa1, pa2, pa3, b0, b1);
                mma16816(o[2 * jp + 1], pa0, pa1, pa2, pa3, b2, b3);
            }
        }
        __syncthreads();          // the stage is overwritten by the copy issued in the next iteration
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    const int r0 = q0 + g, r1 = q0 + g + 8;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        if (r0 < T)
            *reinterpret_cast<uint32_t*>(y + (((size_t)b * T + r0) * n_heads + h) * HD + 8 * j + 2 * t) =
                pack_half2(o[j][0] * i0, o[j][1] * i0);
        if (r1 < T)
            *reinterpret_cast<uint32_t*>(y + (((size_t)b * T + r1) * n_heads + h) * HD + 8 * j + 2 * t) =
                pack_half2(o[j][2] * i1, o[j][3] * i1);
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

extern "C" int glq_attn_prefill(const void* q, const void* k, const void* v, void* y, int B, int T, int n_heads, int n_kv,
                                int head_dim, void* stream) {
    if (!q || !k || !v || !y) return GLQ_ERR_ARG;
    if (B < 0 || T < 0 || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0) return GLQ_ERR_ARG;
    if (B == 0 || T == 0) return GLQ_OK;
    if (head_dim != 64 && head_dim != 128) return GLQ_ERR_UNSUPPORTED;
    if ((long long)((T + 63) / 64) * n_heads * B > 0x7fffffffll) return GLQ_ERR_UNSUPPORTED;
    for (const void* ptr : {q, k, v, (const void*)y})
        if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return GLQ_ERR_ALIGN;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid((unsigned)((T + 63) / 64 * n_heads * B));     // every (query block, head, batch row), most keys first
#define GLQ_PREFILL(HD)                                                                                                  \
    {                                                                                                                    \
        static bool configured[64] = {};                                                                                 \
        int dev = 0;                                                                                                     \
        if (cudaGetDevice(&dev) != cudaSuccess) return GLQ_ERR_CUDA;                                                     \
        if (dev < 0 || dev >= 64 || !configured[dev]) {                                                                  \
            if (cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,               \
                                     (int)PrefillCfg<HD>::SMEM) != cudaSuccess)                                          \
                return GLQ_ERR_CUDA;                                                                                     \
            if (dev >= 0 && dev < 64) configured[dev] = true;                                                            \
        }                                                                                                                \
        attn_prefill_kernel<HD><<<grid, 128, PrefillCfg<HD>::SMEM, st>>>(                                                \
            reinterpret_cast<const __half*>(q), reinterpret_cast<const __half*>(k), reinterpret_cast<const __half*>(v),  \
            reinterpret_cast<__half*>(y), B, T, n_heads, n_kv);                                                              \
    }
    if (head_dim == 64) GLQ_PREFILL(64) else GLQ_PREFILL(128)
#undef GLQ_PREFILL
    return cudaGetLastError() == cudaSuccess ? GLQ_OK : GLQ_ERR_CUDA;
}
