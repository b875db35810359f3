// Grouped skinny matmul for sm_100a: y[rows x N] = x[rows x K] . dequant(W)^T (+ low-rank term),
// rows <= a few dozen.  This is the decode GEMV / batched-decode kernel; it is bound by the HBM
// stream of the packed codes, so everything is organised around that stream:
//   * weights are read once, 16 bytes per lane, fully coalesced (512 B per warp instruction) from
//     the tiled layout; a register ring keeps kDepth loads per lane in flight;
//   * codes are expanded to fp16 fragments with two-three bit-ops per pair (glq_common.cuh) and
//     reduced by the warp-level m16n8k16 tensor-core op into fp32 (it is used as a dot-product
//     engine: 8 activation rows ride along for free, which is the batched-decode case);
//   * activations are staged once per CTA in shared memory, already permuted into fragment order;
//   * scales / zero points are applied in fp32 per 128 (64) input channels;
//   * the rank-r output factor SV is applied in the epilogue from the precomputed a = x.U;
//   * k can be split over the 4 warps of a row tile and over CTAs (deterministic last-arriver
//     reduction through a scratch buffer; no spin waits).
#pragma once

#include "glq_common.cuh"

namespace glq {

// Self-checking accesses: the index of a global / shared access is compared with the extent implied
// by the shapes; the first violation is recorded in g_glq_err (code, index, limit, block<<32|thread)
// and the access is skipped, so a wrong index cannot fault the GPU.  Always on for the codebook
// format (whose unchecked build faulted for a reason that reading the code did not show, while the
// checked build is clean); on for every format when compiled with -DGLQ_CHECKED.
// (one copy per translation unit; glq_debug_error reads them all)
static __device__ unsigned long long g_glq_err[4] = {0, 0, 0, 0};
__device__ __forceinline__ bool glq_ok(bool cond, unsigned long long code, unsigned long long idx,
                                       unsigned long long lim) {
    if (!cond) {
        if (atomicCAS(&g_glq_err[0], 0ull, code) == 0ull) {
            g_glq_err[1] = idx;
            g_glq_err[2] = lim;
            g_glq_err[3] = ((unsigned long long)blockIdx.x << 32) | threadIdx.x;
        }
    }
    return cond;
}
#ifdef GLQ_CHECKED
#define GLQ_GUARDED(FMT) true
#else
#define GLQ_GUARDED(FMT) ((FMT) == GLQ_FMT_T2)
#endif
#define GLQ_OKAY(cond, code, idx, lim) \
    (GLQ_GUARDED(FMT) ? glq_ok((cond), (code), (unsigned long long)(idx), (unsigned long long)(lim)) : true)

constexpr int kRW = 2;     // row tiles per CTA
constexpr int kKW = kWarpsPerCta / kRW;  // warps splitting k for one row tile

struct SkinnyParams {
    glq_weight_t w;              // inline descriptor (used when table == nullptr)
    const glq_weight_t* table;   // per-problem descriptors
    int sv_slices;               // ceil(rank / 64) of the packed SV layout
    const int* slot_index;
    const int* n_slots;
    const int* slot_count;
    const int* slot_offset;
    const int* entry_row;
    const __half* entry_scale;
    const __half* x;
    long long ldx;
    const __half* a[2];
    long long lda;
    __half* y;
    long long ldy;
    float4* scratch;
    int* counters;
    int max_rows;
    int rows_stride;
    int tile_groups;   // CTA row groups per problem
    int sk;            // CTA-level k splits
    int kb_per_split;  // k blocks per CTA split
    int kb_chunk;      // k blocks staged in shared memory at a time (<= kb_per_split)
    int group_blocks;  // k blocks per scale group
    int nkb;           // k blocks in K
    int ntc;           // activation columns staged per pass (power of two, >= 2)
    int max_passes;
    int epilogue;
    int x_vec;         // 1: x rows can be read with 16-byte loads
    long long x_extent;  // elements of x / y that may be touched (0: unknown), self-check only
    long long y_extent;
    int slot_rows;     // row-major operands only: slot s uses weight rows [s*slot_rows, (s+1)*slot_rows)
};

// k per block, staged uint4 per block and column, 16-wide units per block
template <int FMT> struct Fmt;
// DEPTH: register ring depth (k blocks in flight per warp and weight)
template <> struct Fmt<GLQ_FMT_Q2> { static constexpr int KB = 128, XS = 16, UPK = 8, LD = 1, DEPTH = 4; };
template <> struct Fmt<GLQ_FMT_T2> { static constexpr int KB = 128, XS = 16, UPK = 8, LD = 1, DEPTH = 4; };
template <> struct Fmt<GLQ_FMT_Q4> { static constexpr int KB = 64, XS = 8, UPK = 4, LD = 1, DEPTH = 4; };
template <> struct Fmt<GLQ_FMT_F16> { static constexpr int KB = 64, XS = 8, UPK = 4, LD = 4, DEPTH = 2; };

// Pair-interleaved tiled layout of the quantized formats: [pair][k block][tile in pair][block bytes],
// block bytes = 512 B of codes (+ 64 B of (scale, zero) pairs for the affine formats).
template <int FMT> __host__ __device__ constexpr int block_bytes() {
    return (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_Q4) ? 576 : 512;
}
__host__ __device__ inline int block_bytes_of(int fmt) { return (fmt == GLQ_FMT_Q2 || fmt == GLQ_FMT_Q4) ? 576 : 512; }

__host__ __device__ inline size_t skinny_smem_bytes(int fmt, int kb_cta, int ntc, int nw, int ntt) {
    const int xs = (fmt == GLQ_FMT_Q2 || fmt == GLQ_FMT_T2) ? 16 : 8;
    size_t b = (size_t)kb_cta * xs * ntc * 16;                // staged activations
    b += (size_t)kb_cta * ntc * 8;                            // per-block (offset sum, plain sum)
    b += (size_t)kWarpsPerCta * nw * ntt * 32 * 16;           // warp-level k reduction
    return b + 16;
}

// ---------------------------------------------------------------------------------------------
// Activation staging: x rows -> shared memory in fragment order, plus per k block the two sums the
// affine formats need: O = sum off(k) x_k (offset carried by the unpack) and X = sum x_k.
// ---------------------------------------------------------------------------------------------
template <int FMT>
__device__ __forceinline__ void stage_x(const SkinnyParams& p, uint4* xs, float2* ox, int kb_lo, int nkb_cta,
                                        int e0, int pass0, int cnt, int K) {
    using F = Fmt<FMT>;
    const int ntc = p.ntc;
    const int total = ntc * nkb_cta * F::UPK;
    for (int base = 0; base < total; base += kThreads) {
        const int u = base + (int)threadIdx.x;
        const bool valid = u < total;
        const int col = valid ? u / (nkb_cta * F::UPK) : 0;
        const int rem = valid ? u % (nkb_cta * F::UPK) : 0;
        const int kbl = rem / F::UPK, wi = rem % F::UPK;
        const int k0 = (kb_lo + kbl) * F::KB + wi * 16;
        __align__(16) __half v[16];
        const bool live = valid && (pass0 + col < cnt) && (k0 < K);
        if (live) {
            const int entry = e0 + pass0 + col;
            const long long row = p.entry_row ? p.entry_row[entry] : entry;
            const __half* src = p.x + row * p.ldx + k0;
            if (!GLQ_OKAY(p.x_extent == 0 || (row >= 0 && row * p.ldx + k0 + min(16, K - k0) <= p.x_extent), 21,
                          row * p.ldx + k0, p.x_extent)) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __float2half(0.f);
            } else if (p.x_vec && k0 + 16 <= K) {
                *reinterpret_cast<uint4*>(&v[0]) = __ldg(reinterpret_cast<const uint4*>(src));
                *reinterpret_cast<uint4*>(&v[8]) = __ldg(reinterpret_cast<const uint4*>(src) + 1);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = (k0 + j < K) ? src[j] : __float2half(0.f);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __float2half(0.f);
        }
        __align__(16) __half o[16];
        if constexpr (FMT == GLQ_FMT_Q2) {
            // piece pp holds codes [0,8,1,9,2,10,3,11] (+4 for pp = 1)
#pragma unroll
            for (int pp = 0; pp < 2; ++pp)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    o[pp * 8 + 2 * j] = v[4 * pp + j];
                    o[pp * 8 + 2 * j + 1] = v[4 * pp + j + 8];
                }
        } else if constexpr (FMT == GLQ_FMT_T2) {
            // piece pp holds codes [0,2,4,...,14] (+1 for pp = 1)
#pragma unroll
            for (int pp = 0; pp < 2; ++pp)
#pragma unroll
                for (int j = 0; j < 8; ++j) o[pp * 8 + j] = v[2 * j + pp];
        } else if constexpr (FMT == GLQ_FMT_Q4) {
            // word u (8 codes) -> [0,4,1,5,2,6,3,7]
#pragma unroll
            for (int uu = 0; uu < 2; ++uu)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    o[uu * 8 + 2 * j] = v[uu * 8 + j];
                    o[uu * 8 + 2 * j + 1] = v[uu * 8 + j + 4];
                }
        } else {
            // lane t of the k step reads [2t, 2t+1, 2t+8, 2t+9]
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                o[4 * t] = v[2 * t];
                o[4 * t + 1] = v[2 * t + 1];
                o[4 * t + 2] = v[2 * t + 8];
                o[4 * t + 3] = v[2 * t + 9];
            }
        }
        if (valid) {
            const uint4 lo = *reinterpret_cast<const uint4*>(&o[0]);
            const uint4 hi = *reinterpret_cast<const uint4*>(&o[8]);
            if constexpr (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_T2) {
                const int t = wi >> 1, uu = wi & 1;
                if (GLQ_OKAY(((kbl * 4 + 2 * uu + 1) * ntc + col) * 4 + t < p.kb_chunk * F::XS * ntc, 1,
                             ((kbl * 4 + 2 * uu + 1) * ntc + col) * 4 + t, p.kb_chunk * F::XS * ntc)) {
                    xs[((kbl * 4 + 2 * uu) * ntc + col) * 4 + t] = lo;
                    xs[((kbl * 4 + 2 * uu + 1) * ntc + col) * 4 + t] = hi;
                }
            } else if constexpr (FMT == GLQ_FMT_Q4) {
                if (GLQ_OKAY(((kbl * 2 + 1) * ntc + col) * 4 + wi < p.kb_chunk * F::XS * ntc, 2,
                             ((kbl * 2 + 1) * ntc + col) * 4 + wi, p.kb_chunk * F::XS * ntc)) {
                    xs[((kbl * 2 + 0) * ntc + col) * 4 + wi] = lo;
                    xs[((kbl * 2 + 1) * ntc + col) * 4 + wi] = hi;
                }
            } else {
                if (GLQ_OKAY(((kbl * 4 + wi) * ntc + col) * 2 + 1 < p.kb_chunk * F::XS * ntc, 3,
                             ((kbl * 4 + wi) * ntc + col) * 2 + 1, p.kb_chunk * F::XS * ntc)) {
                    xs[((kbl * 4 + wi) * ntc + col) * 2 + 0] = lo;
                    xs[((kbl * 4 + wi) * ntc + col) * 2 + 1] = hi;
                }
            }
        }
        if constexpr (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_Q4) {
            float so = 0.f, sx = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float f = __half2float(v[j]);
                sx += f;
                so += (FMT == GLQ_FMT_Q2 ? q2_offset(j) : kQ4Offset) * f;
            }
#pragma unroll
            for (int d = 1; d < F::UPK; d <<= 1) {
                so += __shfl_xor_sync(0xffffffffu, so, d);
                sx += __shfl_xor_sync(0xffffffffu, sx, d);
            }
            if (valid && wi == 0 && GLQ_OKAY(kbl * ntc + col < p.kb_chunk * ntc, 4, kbl * ntc + col, p.kb_chunk * ntc))
                ox[kbl * ntc + col] = make_float2(so, sx);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// One k block of one weight for one warp: expand the lane's codes and feed the tensor-core dot.
// q: the lane's 16 bytes (F16: 4 x 16 bytes).  xs_kb: staged activations of this k block.
// ---------------------------------------------------------------------------------------------
template <int FMT, int NTT>
__device__ __forceinline__ void block_mma(const uint4 (&q)[Fmt<FMT>::LD], const uint4* __restrict__ xs_kb, int ntc,
                                          int g, int t, uint32_t TL, uint32_t TH, float (&c)[NTT][4], int lim) {
    (void)lim;
    if constexpr (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_T2) {
        const uint32_t wa[2] = {q[0].x, q[0].y}, wb[2] = {q[0].z, q[0].w};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            uint32_t ha[8], hb[8];
            if constexpr (FMT == GLQ_FMT_Q2) {
                unpack_q2(wa[u], ha);
                unpack_q2(wb[u], hb);
            } else {
                unpack_t2(wa[u], TL, TH, ha);
                unpack_t2(wb[u], TL, TH, hb);
            }
#pragma unroll
            for (int tt = 0; tt < NTT; ++tt) {
                const int col = (tt * 8 + g) & (ntc - 1);
                if (!GLQ_OKAY(((2 * u + 1) * ntc + col) * 4 + t < lim, 5, ((2 * u + 1) * ntc + col) * 4 + t, lim)) continue;
                const uint4 b0 = xs_kb[((2 * u) * ntc + col) * 4 + t];
                const uint4 b1 = xs_kb[((2 * u + 1) * ntc + col) * 4 + t];
                mma16816(c[tt], ha[0], hb[0], ha[1], hb[1], b0.x, b0.y);
                mma16816(c[tt], ha[2], hb[2], ha[3], hb[3], b0.z, b0.w);
                mma16816(c[tt], ha[4], hb[4], ha[5], hb[5], b1.x, b1.y);
                mma16816(c[tt], ha[6], hb[6], ha[7], hb[7], b1.z, b1.w);
            }
        }
    } else if constexpr (FMT == GLQ_FMT_Q4) {
        const uint32_t wa[2] = {q[0].x, q[0].y}, wb[2] = {q[0].z, q[0].w};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            uint32_t ha[4], hb[4];
            unpack_q4(wa[u], ha);
            unpack_q4(wb[u], hb);
#pragma unroll
            for (int tt = 0; tt < NTT; ++tt) {
                const int col = (tt * 8 + g) & (ntc - 1);
                if (!GLQ_OKAY((u * ntc + col) * 4 + t < lim, 6, (u * ntc + col) * 4 + t, lim)) continue;
                const uint4 b = xs_kb[(u * ntc + col) * 4 + t];
                mma16816(c[tt], ha[0], hb[0], ha[1], hb[1], b.x, b.y);
                mma16816(c[tt], ha[2], hb[2], ha[3], hb[3], b.z, b.w);
            }
        }
    } else {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int tt = 0; tt < NTT; ++tt) {
                const int col = (tt * 8 + g) & (ntc - 1);
                if (!GLQ_OKAY(((ks * ntc + col) * 4) + t < 2 * lim, 7, ((ks * ntc + col) * 4) + t, 2 * lim)) continue;
                const uint2 b = reinterpret_cast<const uint2*>(xs_kb)[((ks * ntc + col) * 4) + t];
                mma16816(c[tt], q[ks].x, q[ks].y, q[ks].z, q[ks].w, b.x, b.y);
            }
        }
    }
}

// load the lane's codes (and scale/zero pairs) of k block kb of tile (pair, j); F16 and the row-major
// operand address by row tile rt
template <int FMT, bool RM>
__device__ __forceinline__ void load_codes(const glq_weight_t& W, int rt, int pair, int j, int kb, int nkb, int lane,
                                           uint4 (&q)[Fmt<FMT>::LD], uint2& szv) {
    if constexpr (RM) {
        // row-major (N, K/4) uint8 operand of the reference's native module
        const int g = lane >> 2, t = lane & 3;
        const int rowbytes = W.K >> 2;
        const uint8_t* base = reinterpret_cast<const uint8_t*>(W.codes);
        const int boff = kb * 32 + t * 8;
        uint2 r[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int row = rt * kRowTile + g + 8 * h;
            row = row < W.N ? row : W.N - 1;
            const uint8_t* ptr = base + (size_t)row * rowbytes + boff;
            if (!GLQ_OKAY(row >= 0 && kb >= 0 && kb < nkb, 20, (size_t)row * rowbytes + boff, (size_t)W.N * rowbytes)) {
                r[h] = make_uint2(0, 0);
            } else if (W.reserved != 0 && (rowbytes & 7) == 0 && boff + 8 <= rowbytes) {   // reserved: base is 8-byte aligned
                r[h] = __ldg(reinterpret_cast<const uint2*>(ptr));
            } else {
                uint32_t lo = 0, hi = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    if (boff + b < rowbytes) lo |= (uint32_t)__ldg(ptr + b) << (8 * b);
                    if (boff + 4 + b < rowbytes) hi |= (uint32_t)__ldg(ptr + 4 + b) << (8 * b);
                }
                r[h] = make_uint2(lo, hi);
            }
        }
        q[0] = make_uint4(r[0].x, r[0].y, r[1].x, r[1].y);
    } else if constexpr (FMT == GLQ_FMT_F16) {
        const uint4* base = reinterpret_cast<const uint4*>(W.codes);
#pragma unroll
        for (int i = 0; i < Fmt<FMT>::LD; ++i) q[i] = __ldcs(base + ((size_t)(rt * nkb + kb) * Fmt<FMT>::LD + i) * 32 + lane);
    } else {
        const unsigned char* blk =
            reinterpret_cast<const unsigned char*>(W.codes) + (((size_t)pair * nkb + kb) * 2 + j) * block_bytes<FMT>();
        q[0] = __ldcs(reinterpret_cast<const uint4*>(blk) + lane);
        if constexpr (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_Q4)
            szv = __ldg(reinterpret_cast<const uint2*>(blk + 512) + (lane >> 2));
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel.  grid.x = n_problems * tile_groups * sk, block = 256 threads = kRW row tiles x kKW.
// ---------------------------------------------------------------------------------------------
template <int FMT, int NW, int NTT, bool RM>
__global__ void __launch_bounds__(kThreads, 2) skinny_kernel(const SkinnyParams p) {
    using F = Fmt<FMT>;
    constexpr int kDepth = F::DEPTH;
    extern __shared__ uint4 smem_u4[];
    __shared__ int s_last;
    // Programmatic dependent launch, both no-ops for a plain launch: wait for the preceding grid of the
    // stream (this kernel reads its results from the first load on), then let the next grid be scheduled
    // (it waits for this one in the same way before it reads what this one writes).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    int bid = blockIdx.x;
    const int s = bid % p.sk;
    bid /= p.sk;
    const int tg = bid % p.tile_groups;
    const int slot = bid / p.tile_groups;
    if (p.n_slots && slot >= __ldg(p.n_slots)) return;
    const int cnt = p.slot_count ? __ldg(p.slot_count + slot) : p.max_rows;
    if (cnt <= 0) return;
    const int e0 = p.slot_offset ? __ldg(p.slot_offset + slot) : slot * p.rows_stride;
    const int widx = p.slot_index ? __ldg(p.slot_index + slot) : slot;

    // one weight per problem; NW == 2 means a fused gate|up weight whose pair p is (gate tile p, up tile p)
    glq_weight_t W = p.table ? p.table[widx] : p.w;
    if constexpr (RM) {
        if (p.slot_rows > 0) {
            W.codes = reinterpret_cast<const uint8_t*>(W.codes) + (size_t)slot * p.slot_rows * (W.K >> 2);
            W.norms += (size_t)slot * p.slot_rows;
        }
    }
    const int N = W.N, K = W.K;
    const int ntiles = (N + kRowTile - 1) / kRowTile;
    const int nkb = p.nkb;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rw = warp / kKW, kw = warp % kKW;
    const int rt = tg * kRW + rw;
    const bool tile_ok = rt < ntiles;

    // k range of this CTA; it is walked in chunks of kb_chunk blocks (what shared memory holds)
    const int kb_lo = s * p.kb_per_split;
    const int kb_hi = min(nkb, kb_lo + p.kb_per_split);

    const int ntc = p.ntc;
    uint4* xs = smem_u4;
    float2* ox = reinterpret_cast<float2*>(xs + (size_t)p.kb_chunk * F::XS * ntc);
    float4* red = reinterpret_cast<float4*>(ox + (size_t)p.kb_chunk * ntc);

    uint32_t TL[NW], TH[NW];  // a fused gate|up weight carries two codebooks (4 floats each)
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        TL[i] = TH[i] = 0;
        if constexpr (FMT == GLQ_FMT_T2) make_t2_tables(W.centroids + 4 * i, TL[i], TH[i]);
    }
    // tile i of this warp in the pair-interleaved layout
    const int pr = NW == 2 ? rt : (rt >> 1);
    const int pj0 = NW == 2 ? 0 : (rt & 1);

    const int rows_per_pass = 8 * NTT;
    const int npass = (cnt + rows_per_pass - 1) / rows_per_pass;
    int iter = 0;

    for (int pass = 0; pass < npass; ++pass) {
        const int pass0 = pass * rows_per_pass;

        float acc[NW][NTT][4];
#pragma unroll
        for (int i = 0; i < NW; ++i)
#pragma unroll
            for (int tt = 0; tt < NTT; ++tt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][tt][j] = 0.f;

        for (int kc_lo = kb_lo; kc_lo < kb_hi; kc_lo += p.kb_chunk) {
            const int kc_hi = min(kb_hi, kc_lo + p.kb_chunk);
            const int nkc = kc_hi - kc_lo;
            const int per_w = (nkc + kKW - 1) / kKW;
            const int wk_lo = min(kc_hi, kc_lo + kw * per_w);
            const int wk_hi = min(kc_hi, wk_lo + per_w);

            // ---- prefetch the first code blocks, then stage the activations ----
            uint4 q[NW][kDepth][F::LD];
            uint2 szv[NW][kDepth];
            if (tile_ok) {
#pragma unroll
                for (int d = 0; d < kDepth; ++d) {
                    const int kb = wk_lo + d;
                    if (kb < wk_hi) {
#pragma unroll
                        for (int i = 0; i < NW; ++i) load_codes<FMT, RM>(W, rt, pr, pj0 + i, kb, nkb, lane, q[i][d], szv[i][d]);
                    }
                }
            }
            if (iter++ > 0) __syncthreads();  // everyone is done with the previous contents of shared memory
            stage_x<FMT>(p, xs, ox, kc_lo, nkc, e0, pass0, cnt, K);
            __syncthreads();

            if (tile_ok) {
                for (int kb0 = wk_lo; kb0 < wk_hi; kb0 += kDepth) {
#pragma unroll
                    for (int d = 0; d < kDepth; ++d) {
                        const int kb = kb0 + d;
                        if (kb < wk_hi) {
                            const int kbl = kb - kc_lo;
                            const uint4* xs_kb = xs + (size_t)kbl * F::XS * ntc;
#pragma unroll
                            for (int i = 0; i < NW; ++i) {
                                if constexpr (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_Q4) {
                                    float c[NTT][4];
#pragma unroll
                                    for (int tt = 0; tt < NTT; ++tt)
#pragma unroll
                                        for (int j = 0; j < 4; ++j) c[tt][j] = 0.f;
                                    block_mma<FMT, NTT>(q[i][d], xs_kb, ntc, g, t, TL[i], TH[i], c, (p.kb_chunk - kbl) * F::XS * ntc);
                                    const __half2 sz0 = *reinterpret_cast<const __half2*>(&szv[i][d].x);
                                    const __half2 sz1 = *reinterpret_cast<const __half2*>(&szv[i][d].y);
                                    const float s0 = __low2float(sz0), z0 = __high2float(sz0);
                                    const float s1 = __low2float(sz1), z1 = __high2float(sz1);
#pragma unroll
                                    for (int tt = 0; tt < NTT; ++tt) {
                                        const int col = (tt * 8 + 2 * t) & (ntc - 1);
                                        if (!GLQ_OKAY(kbl * ntc + col + 1 < p.kb_chunk * ntc, 9, kbl * ntc + col, p.kb_chunk * ntc)) continue;
                                        const float4 o = *reinterpret_cast<const float4*>(&ox[kbl * ntc + col]);
                                        acc[i][tt][0] = fmaf(s0, fmaf(-z0, o.y, c[tt][0] - o.x), acc[i][tt][0]);
                                        acc[i][tt][1] = fmaf(s0, fmaf(-z0, o.w, c[tt][1] - o.z), acc[i][tt][1]);
                                        acc[i][tt][2] = fmaf(s1, fmaf(-z1, o.y, c[tt][2] - o.x), acc[i][tt][2]);
                                        acc[i][tt][3] = fmaf(s1, fmaf(-z1, o.w, c[tt][3] - o.z), acc[i][tt][3]);
                                    }
                                } else {
                                    block_mma<FMT, NTT>(q[i][d], xs_kb, ntc, g, t, TL[i], TH[i], acc[i], (p.kb_chunk - kbl) * F::XS * ntc);
                                }
                                const int kn = kb + kDepth;
                                if (kn < wk_hi) load_codes<FMT, RM>(W, rt, pr, pj0 + i, kn, nkb, lane, q[i][d], szv[i][d]);
                            }
                        }
                    }
                }
            }
        }

        // ---- reduce the kKW warps of a row tile (fixed order) ----
        if (kw != 0) {
#pragma unroll
            for (int i = 0; i < NW; ++i)
#pragma unroll
                for (int tt = 0; tt < NTT; ++tt)
                    red[((warp * NW + i) * NTT + tt) * 32 + lane] =
                        make_float4(acc[i][tt][0], acc[i][tt][1], acc[i][tt][2], acc[i][tt][3]);
        }
        __syncthreads();
        if (kw == 0) {
            for (int k2 = 1; k2 < kKW; ++k2)
#pragma unroll
                for (int i = 0; i < NW; ++i)
#pragma unroll
                    for (int tt = 0; tt < NTT; ++tt) {
                        const float4 v = red[(((warp + k2) * NW + i) * NTT + tt) * 32 + lane];
                        acc[i][tt][0] += v.x;
                        acc[i][tt][1] += v.y;
                        acc[i][tt][2] += v.z;
                        acc[i][tt][3] += v.w;
                    }
        }

        // ---- CTA-level split-k: last arriver sums the partials in split order ----
        if (p.sk > 1) {
            const size_t tile_id = ((size_t)slot * p.tile_groups + tg) * p.max_passes + pass;
            float4* part = p.scratch + tile_id * p.sk * (kRW * NW * NTT * 32);
            if (kw == 0) {
#pragma unroll
                for (int i = 0; i < NW; ++i)
#pragma unroll
                    for (int tt = 0; tt < NTT; ++tt)
                        __stcg(&part[(size_t)s * (kRW * NW * NTT * 32) + ((rw * NW + i) * NTT + tt) * 32 + lane],
                               make_float4(acc[i][tt][0], acc[i][tt][1], acc[i][tt][2], acc[i][tt][3]));
                __threadfence();
            }
            __syncthreads();
            if (tid == 0) {
                const int old = atomicAdd(&p.counters[tile_id], 1);
                const int last = (old == p.sk - 1);
                if (last) p.counters[tile_id] = 0;
                s_last = last;
            }
            __syncthreads();
            if (!s_last) continue;
            __threadfence();
            if (kw == 0) {
#pragma unroll
                for (int i = 0; i < NW; ++i)
#pragma unroll
                    for (int tt = 0; tt < NTT; ++tt) {
                        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                        for (int s2 = 0; s2 < p.sk; ++s2) {
                            const float4 v = __ldcg(
                                &part[(size_t)s2 * (kRW * NW * NTT * 32) + ((rw * NW + i) * NTT + tt) * 32 + lane]);
                            sum.x += v.x;
                            sum.y += v.y;
                            sum.z += v.z;
                            sum.w += v.w;
                        }
                        acc[i][tt][0] = sum.x;
                        acc[i][tt][1] = sum.y;
                        acc[i][tt][2] = sum.z;
                        acc[i][tt][3] = sum.w;
                    }
            }
        }

        // ---- epilogue: one warp per row tile ----
        if (kw == 0 && tile_ok) {
            const int r0 = rt * kRowTile + g, r1 = r0 + 8;
            const int r0c = min(r0, N - 1), r1c = min(r1, N - 1);
            float res[NW][NTT][4];
#pragma unroll
            for (int i = 0; i < NW; ++i) {
                float n0 = 1.f, n1 = 1.f;
                if constexpr (FMT == GLQ_FMT_T2) {
                    // row-major operand: norms by row; tiled: norms in tile order
                    const size_t i0 = RM ? (size_t)r0c : ((size_t)(pr * 2 + pj0 + i) * 16 + g);
                    const size_t i1 = RM ? (size_t)r1c : i0 + 8;
                    if (GLQ_OKAY(W.norms != nullptr, 12, i1, N)) {
                        n0 = __ldg(W.norms + i0);
                        n1 = __ldg(W.norms + i1);
                    }
                }
                // low-rank term a . SV^T through the same tensor-core dot
                float lo[NTT][4];
#pragma unroll
                for (int tt = 0; tt < NTT; ++tt)
#pragma unroll
                    for (int j = 0; j < 4; ++j) lo[tt][j] = 0.f;
                const int rank = W.rank;
                const bool has_lr = !RM && FMT != GLQ_FMT_F16 && rank > 0 && W.sv != nullptr && p.a[i] != nullptr;
                if (has_lr) {
                    // packed SV: [pair][64-column slice][32 rows of the pair][64 columns]
                    const __half* sv = reinterpret_cast<const __half*>(W.sv);
                    for (int c0 = 0; c0 < rank; c0 += 64) {
                        const int cc = c0 + 16 * t;
                        uint4 sa[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
                        uint4 sb[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
                        if (cc < rank) {
                            const size_t row0 = ((size_t)pr * p.sv_slices + (c0 >> 6)) * 32 + (pj0 + i) * 16 + g;
                            const uint4* pa = reinterpret_cast<const uint4*>(sv + row0 * 64 + 16 * t);
                            const uint4* pb = reinterpret_cast<const uint4*>(sv + (row0 + 8) * 64 + 16 * t);
                            sa[0] = __ldg(pa); sa[1] = __ldg(pa + 1);
                            sb[0] = __ldg(pb); sb[1] = __ldg(pb + 1);
                        }
#pragma unroll
                        for (int tt = 0; tt < NTT; ++tt) {
                            const int row = pass0 + tt * 8 + g;
                            uint4 av[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
                            if (row < cnt && cc < rank) {
                                const uint4* pav =
                                    reinterpret_cast<const uint4*>(p.a[i] + (size_t)(e0 + row) * p.lda + cc);
                                av[0] = __ldg(pav);
                                av[1] = __ldg(pav + 1);
                            }
                            mma16816(lo[tt], sa[0].x, sb[0].x, sa[0].y, sb[0].y, av[0].x, av[0].y);
                            mma16816(lo[tt], sa[0].z, sb[0].z, sa[0].w, sb[0].w, av[0].z, av[0].w);
                            mma16816(lo[tt], sa[1].x, sb[1].x, sa[1].y, sb[1].y, av[1].x, av[1].y);
                            mma16816(lo[tt], sa[1].z, sb[1].z, sa[1].w, sb[1].w, av[1].z, av[1].w);
                        }
                    }
                }
                const __half* bias = reinterpret_cast<const __half*>(W.bias);
                const float b0 = bias ? __half2float(__ldg(bias + r0c)) : 0.f;
                const float b1 = bias ? __half2float(__ldg(bias + r1c)) : 0.f;
#pragma unroll
                for (int tt = 0; tt < NTT; ++tt)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float v = round16(acc[i][tt][j] * (j < 2 ? n0 : n1));
                        if (has_lr) v = round16(v + round16(lo[tt][j]));
                        if (bias) v = round16(v + (j < 2 ? b0 : b1));
                        res[i][tt][j] = v;
                    }
            }
#pragma unroll
            for (int tt = 0; tt < NTT; ++tt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int row = pass0 + tt * 8 + 2 * t + (j & 1);
                    const int n = (j < 2) ? r0 : r1;
                    if (row < cnt && n < N) {
                        float v;
                        if constexpr (NW == 2) {
                            v = round16(silu16(res[0][tt][j]) * res[1][tt][j]);
                        } else {
                            v = res[0][tt][j];
                            if (p.entry_scale) v = round16(__half2float(__ldg(p.entry_scale + e0 + row)) * v);
                        }
                        if (GLQ_OKAY(p.y_extent == 0 || (long long)(e0 + row) * p.ldy + n < p.y_extent, 22,
                                     (long long)(e0 + row) * p.ldy + n, p.y_extent))
                            p.y[(size_t)(e0 + row) * p.ldy + n] = __float2half_rn(v);
                    }
                }
        }
    }
}

}  // namespace glq
