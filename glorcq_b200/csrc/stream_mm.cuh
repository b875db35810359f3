// Persistent streaming kernel of the grouped skinny matmul: the decode GEMV / batched-decode fast
// path (skinny_mm.cuh has the same maths for every shape and is the fallback).
//
// The op is bound by the HBM stream of packed codes, so the kernel is a copy pipeline with compute
// attached:
//   * one CTA per SM walks a contiguous range of work items (problem, tile pair, k split); the
//     activations of a problem are staged once per CTA, not once per tile;
//   * every warp owns a ring of shared-memory stages filled by bulk asynchronous copies
//     (cp.async.bulk global -> shared, completion counted on an mbarrier) that the warp issues itself,
//     several stages ahead of where it computes and across item boundaries, so the bytes in flight
//     per SM stay constant.  In the pair-interleaved layout the codes and scales of a tile pair for
//     consecutive k blocks are one contiguous run: one copy per stage (4.5 KB); the 32 rows of the
//     packed output-side factor SV are one more 4 KB copy on the same ring;
//   * a warp item is a PAIR of row tiles that share the activation fragments (gate and up tile of an
//     expert, or two consecutive tiles of one matrix);
//   * up to 8 activation rows take the integer path: the activations are turned into 16-bit block
//     fixed point (two int8 digits per value, one power-of-two scale per row and k block) when they
//     are staged, the 2/4-bit codes become int8 with two bit-ops per four weights, and the s8 x s8
//     -> s32 tensor-core op (m16n8k32) does the dot products exactly; scale, zero point and the digit
//     weights are applied in fp32 per k block.  More rows (and the codebook format) use the fp16 op;
//   * k splits of a pair are warps of one CTA, reduced through shared memory in a fixed order
//     (named barrier per pair): no global scratch, no atomics, deterministic.
// Every mbarrier wait is bounded in time; a wait that runs out records an error word and the warp
// stops waiting, so the kernel always terminates.  No cluster launch, no multicast.
#pragma once

#include "skinny_mm.cuh"

namespace glq {

constexpr int kMaxStages = 6;
#ifndef GLQ_STREAM_CB
#define GLQ_STREAM_CB 4
#endif
constexpr int kStreamCB = GLQ_STREAM_CB;  // k blocks per ring stage
#ifndef GLQ_STREAM_CTAS
#define GLQ_STREAM_CTAS 2
#endif
constexpr int kStreamCtasPerSm = GLQ_STREAM_CTAS;

struct StreamParams {
    SkinnyParams b;    // operands (of its geometry fields only ntc, nkb are used)
    int N, K, rank;
    int n_problems;
    int swiglu;        // 1: the weight is a fused gate|up matrix, the output is silu(gate) * up
    int sk;            // k splits (warps of one CTA): 1, 2, 4 or 8
    int sk_log2;
    int kb_per_split;
    int npairs;        // tile pairs per problem
    int ips;           // iterations (8 warp items) per problem
    int stages;        // ring depth
    int stage_bytes;
    int off_xs, off_ox, off_as, off_ring, off_red;  // shared memory carve-up (bytes)
    int cnt_lo, cnt_hi;  // only slots with cnt_lo < rows <= cnt_hi are this launch's (others belong to a sibling launch)
    int dependent;  // 1: launched with programmatic stream serialization
    int a_late;   // 1: the x.U operand is still being written when this kernel starts (programmatic dependent launch)
};

// ---- shared memory, mbarrier and bulk copy primitives ------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: polls for at most about 2 ms.  A wait that runs out records error code 100 and
// marks the warp dead; a dead warp no longer waits, so the kernel always ends within milliseconds.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, bool& dead) {
    if (dead) return;
    if (mbar_try_wait(bar, parity)) return;
    const unsigned long long t0 = global_ns();
    // try_wait suspends the thread in hardware for a bounded time: a waiting warp takes no issue slots
    while (!mbar_try_wait(bar, parity)) {
        if (global_ns() - t0 > 2000000ull) {
            glq_ok(false, 100, bar, parity);
            dead = true;
            return;
        }
    }
}
__device__ __forceinline__ uint4 ld_global_u4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// D(16x8, s32) = A(16x32, s8, row) * B(32x8, s8, col) + C.  Lane = 4g+t owns
//   a0 = (row g, k 4t..4t+3)  a1 = (row g+8, same k)  a2 = (row g, k 16+4t..)  a3 = (row g+8, k 16+4t..)
//   b0 = (k 4t..4t+3 ; col g) b1 = (k 16+4t.. ; col g);  d0,d1 = (row g ; col 2t,2t+1)  d2,d3 = (row g+8)
__device__ __forceinline__ void imma16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1, int c0, int c1, int c2, int c3) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}

// ---- integer path: staging of the activations ----------------------------------------------------
// x rows -> int8 digit fragments.  Per row and k block: sh = 14 - exponent(max |x|), v = rint(x * 2^sh)
// (|v| < 2^15, exact for every x within 2^-13 of the block maximum), v = 256*d1 + d0 with d0, d1 in
// [-128, 127].  Fragment order: for the lane-t chunk of a block, word u, op m: b0 = digits of codes
// {2m, 2m+4, 2m+8, 2m+12}, b1 = codes {2m+1, ...} (2-bit); word u: b0 = even codes, b1 = odd codes
// (4-bit).  Layout: xs[kb][piece][col = 2*row + digit][t] of uint4, piece = u (2-bit) / 0 (4-bit);
// ox[kb][row] = (2^-sh, sum of x).
template <int FMT>
__device__ __forceinline__ void stage_x_i8(const SkinnyParams& p, uint4* xs, float2* ox, int nkb, int ncol, int e0,
                                           int cnt, int K) {
    using F = Fmt<FMT>;
    constexpr int P8 = F::UPK / 4;  // pieces per block: 2 (2-bit), 1 (4-bit)
    const int nrow = ncol >> 1;
    // only the live rows are staged; columns of absent rows keep stale (finite or not) data, and the
    // outputs computed from them are never stored
    const int total = min(nrow, cnt) * nkb * F::UPK;
    for (int base = 0; base < total; base += kThreads) {
        const int u = base + (int)threadIdx.x;
        const bool valid = u < total;
        const int row = valid ? u / (nkb * F::UPK) : 0;
        const int rem = valid ? u % (nkb * F::UPK) : 0;
        const int kb = rem / F::UPK, wi = rem % F::UPK;
        const int k0 = kb * F::KB + wi * 16;
        __align__(16) __half v[16];
        const bool live = valid && row < cnt && k0 < K;
        if (live) {
            const int entry = e0 + row;
            const long long xr = p.entry_row ? p.entry_row[entry] : entry;
            const __half* src = p.x + xr * p.ldx + k0;
            if (p.x_vec && k0 + 16 <= K) {
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
        float f[16], mx = 0.f, sx = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            f[j] = __half2float(v[j]);
            mx = fmaxf(mx, fabsf(f[j]));
            sx += f[j];
        }
#pragma unroll
        for (int d = 1; d < F::UPK; d <<= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
            sx += __shfl_xor_sync(0xffffffffu, sx, d);
        }
        int ex = 0;
        if (mx > 0.f) (void)frexpf(mx, &ex);  // mx = m * 2^ex, m in [0.5, 1)
        const int sh = 14 - ex;
        const float scale = ldexpf(1.f, sh);
        int d0[16], d1[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int q = __float2int_rn(f[j] * scale);
            d1[j] = (q + 128) >> 8;
            d0[j] = q - (d1[j] << 8);
        }
        // byte order of a word's fragment pair (b0, b1)
        auto pack4 = [](const int* d, int c0, int c1, int c2, int c3) -> uint32_t {
            return (uint32_t)(d[c0] & 0xff) | ((uint32_t)(d[c1] & 0xff) << 8) | ((uint32_t)(d[c2] & 0xff) << 16) |
                   ((uint32_t)(d[c3] & 0xff) << 24);
        };
        if (valid) {
            uint4 lo, hi;  // digit 0, digit 1
            int t, piece;
            if constexpr (FMT != GLQ_FMT_Q4) {
                t = wi >> 1;
                piece = wi & 1;
                lo = make_uint4(pack4(d0, 0, 4, 8, 12), pack4(d0, 1, 5, 9, 13), pack4(d0, 2, 6, 10, 14),
                                pack4(d0, 3, 7, 11, 15));
                hi = make_uint4(pack4(d1, 0, 4, 8, 12), pack4(d1, 1, 5, 9, 13), pack4(d1, 2, 6, 10, 14),
                                pack4(d1, 3, 7, 11, 15));
            } else {
                t = wi;
                piece = 0;
                lo = make_uint4(pack4(d0, 0, 2, 4, 6), pack4(d0, 1, 3, 5, 7), pack4(d0, 8, 10, 12, 14),
                                pack4(d0, 9, 11, 13, 15));
                hi = make_uint4(pack4(d1, 0, 2, 4, 6), pack4(d1, 1, 3, 5, 7), pack4(d1, 8, 10, 12, 14),
                                pack4(d1, 9, 11, 13, 15));
            }
            xs[((size_t)(kb * P8 + piece) * ncol + 2 * row) * 4 + t] = lo;
            xs[((size_t)(kb * P8 + piece) * ncol + 2 * row + 1) * 4 + t] = hi;
            if (wi == 0) ox[kb * nrow + row] = make_float2(ldexpf(1.f, -sh), sx);
        }
    }
}

// ---- fp16 path: one k block of one tile against preloaded activation fragments --------------------
template <int FMT, int NTT>
__device__ __forceinline__ void tile_block(const uint4 q, const uint4 (&bx)[NTT][4], uint32_t TL, uint32_t TH,
                                           float (&c)[NTT][4], int nt_live = NTT) {
    const uint32_t wa[2] = {q.x, q.y}, wb[2] = {q.z, q.w};
    if constexpr (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_T2) {
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
                if (tt >= nt_live) continue;      // activation tiles beyond the problem's rows (warp-uniform)
                const uint4 b0 = bx[tt][2 * u], b1 = bx[tt][2 * u + 1];
                mma16816(c[tt], ha[0], hb[0], ha[1], hb[1], b0.x, b0.y);
                mma16816(c[tt], ha[2], hb[2], ha[3], hb[3], b0.z, b0.w);
                mma16816(c[tt], ha[4], hb[4], ha[5], hb[5], b1.x, b1.y);
                mma16816(c[tt], ha[6], hb[6], ha[7], hb[7], b1.z, b1.w);
            }
        }
    } else {  // Q4
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            uint32_t ha[4], hb[4];
            unpack_q4(wa[u], ha);
            unpack_q4(wb[u], hb);
#pragma unroll
            for (int tt = 0; tt < NTT; ++tt) {
                if (tt >= nt_live) continue;
                const uint4 b = bx[tt][u];
                mma16816(c[tt], ha[0], hb[0], ha[1], hb[1], b.x, b.y);
                mma16816(c[tt], ha[2], hb[2], ha[3], hb[3], b.z, b.w);
            }
        }
    }
}

// ---- integer path: one k block of one tile; bx[nt][piece] are the digit fragments ------------------
template <int FMT, int NT>
__device__ __forceinline__ void tile_block_i8(const uint4 q, const uint4 (&bx)[NT][2], int (&c)[NT][4]) {
    if constexpr (FMT == GLQ_FMT_Q2) {
        const uint32_t m = 0x03030303u;
        const uint32_t wa[2] = {q.x, q.y}, wb[2] = {q.z, q.w};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const uint32_t a0 = wa[u] & m, a1 = (wa[u] >> 2) & m, a2 = (wa[u] >> 4) & m, a3 = (wa[u] >> 6) & m;
            const uint32_t b0 = wb[u] & m, b1 = (wb[u] >> 2) & m, b2 = (wb[u] >> 4) & m, b3 = (wb[u] >> 6) & m;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 x = bx[nt][u];
                if (u == 0)
                    imma16832(c[nt], a0, b0, a1, b1, x.x, x.y, 0, 0, 0, 0);
                else
                    imma16832(c[nt], a0, b0, a1, b1, x.x, x.y, c[nt][0], c[nt][1], c[nt][2], c[nt][3]);
                imma16832(c[nt], a2, b2, a3, b3, x.z, x.w, c[nt][0], c[nt][1], c[nt][2], c[nt][3]);
            }
        }
    } else if constexpr (FMT == GLQ_FMT_Q4) {  // a word holds 8 codes = the A operand of one op
        const uint32_t m = 0x0F0F0F0Fu;
        const uint32_t a0 = q.x & m, a1 = (q.x >> 4) & m, a2 = q.y & m, a3 = (q.y >> 4) & m;
        const uint32_t b0 = q.z & m, b1 = (q.z >> 4) & m, b2 = q.w & m, b3 = (q.w >> 4) & m;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint4 x = bx[nt][0];
            imma16832(c[nt], a0, b0, a1, b1, x.x, x.y, 0, 0, 0, 0);
            imma16832(c[nt], a2, b2, a3, b3, x.z, x.w, c[nt][0], c[nt][1], c[nt][2], c[nt][3]);
        }
    }
}

// ---- integer path of the codebook format -----------------------------------------------------------
// A 4-entry codebook is c(q) = c0 + d0*q + dh*(2*b1) + e*(b0 & b1) with q = b0 + 2*b1 the code,
// d0 = c1 - c0, dh = (c2 - c0)/2 - d0, e = c3 - c2 - c1 + c0.  A symmetric codebook (-a, -b, b, a) has
// e = 0: two integer products per k block, codes against digits (cq) and the high code bits against
// digits (cb); the third (ce) is computed only for a codebook with e != 0 (warp-uniform).
template <int NT>
__device__ __forceinline__ void tile_block_t2_i8(const uint4 q, const uint4 (&bx)[NT][2], bool cross,
                                                 int (&cq)[NT][4], int (&cb)[NT][4], int (&ce)[NT][4]) {
    const uint32_t m = 0x03030303u, mh = 0x02020202u, m1 = 0x01010101u;
    const uint32_t wa[2] = {q.x, q.y}, wb[2] = {q.z, q.w};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const uint32_t a0 = wa[u] & m, a1 = (wa[u] >> 2) & m, a2 = (wa[u] >> 4) & m, a3 = (wa[u] >> 6) & m;
        const uint32_t b0 = wb[u] & m, b1 = (wb[u] >> 2) & m, b2 = (wb[u] >> 4) & m, b3 = (wb[u] >> 6) & m;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint4 x = bx[nt][u];
            if (u == 0) {
                imma16832(cq[nt], a0, b0, a1, b1, x.x, x.y, 0, 0, 0, 0);
                imma16832(cb[nt], a0 & mh, b0 & mh, a1 & mh, b1 & mh, x.x, x.y, 0, 0, 0, 0);
            } else {
                imma16832(cq[nt], a0, b0, a1, b1, x.x, x.y, cq[nt][0], cq[nt][1], cq[nt][2], cq[nt][3]);
                imma16832(cb[nt], a0 & mh, b0 & mh, a1 & mh, b1 & mh, x.x, x.y, cb[nt][0], cb[nt][1], cb[nt][2],
                          cb[nt][3]);
            }
            imma16832(cq[nt], a2, b2, a3, b3, x.z, x.w, cq[nt][0], cq[nt][1], cq[nt][2], cq[nt][3]);
            imma16832(cb[nt], a2 & mh, b2 & mh, a3 & mh, b3 & mh, x.z, x.w, cb[nt][0], cb[nt][1], cb[nt][2],
                      cb[nt][3]);
        }
        if (cross) {
            const uint32_t e0 = a0 & (a0 >> 1) & m1, e1 = a1 & (a1 >> 1) & m1, e2 = a2 & (a2 >> 1) & m1,
                           e3 = a3 & (a3 >> 1) & m1;
            const uint32_t f0 = b0 & (b0 >> 1) & m1, f1 = b1 & (b1 >> 1) & m1, f2 = b2 & (b2 >> 1) & m1,
                           f3 = b3 & (b3 >> 1) & m1;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 x = bx[nt][u];
                if (u == 0)
                    imma16832(ce[nt], e0, f0, e1, f1, x.x, x.y, 0, 0, 0, 0);
                else
                    imma16832(ce[nt], e0, f0, e1, f1, x.x, x.y, ce[nt][0], ce[nt][1], ce[nt][2], ce[nt][3]);
                imma16832(ce[nt], e2, f2, e3, f3, x.z, x.w, ce[nt][0], ce[nt][1], ce[nt][2], ce[nt][3]);
            }
        }
    }
}

// ---- the kernel -----------------------------------------------------------------------------------
// I8 = true : NT tiles of 4 activation rows (integer path: affine formats and the 2-bit codebook)
// I8 = false: NT tiles of 8 activation rows (fp16 path)
template <int FMT, bool I8, int NT>
__global__ void __launch_bounds__(kThreads, kStreamCtasPerSm) stream_kernel(const StreamParams sp) {
    using F = Fmt<FMT>;
    static_assert(FMT != GLQ_FMT_F16, "dense weights use the fallback kernel");
    constexpr bool kAffine = (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_Q4);
    constexpr int BB = block_bytes<FMT>();
    constexpr int kPieces = I8 ? F::UPK / 4 : F::XS / 4;  // uint4 fragments per k block, lane and column
    constexpr int kRowsPerTile = I8 ? 4 : 8;
    constexpr int kRows = kRowsPerTile * NT;
    const SkinnyParams& p = sp.b;
    extern __shared__ __align__(128) unsigned char smem[];

    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int N = sp.N, K = sp.K, rank = sp.rank;
    const int nkb = p.nkb, ntc = p.ntc;
    const int S = sp.stages, sk = sp.sk;
    const bool swiglu = sp.swiglu != 0;
    const int ns = (rank + 63) / 64;

    // Programmatic dependent launch (no-ops for a plain launch).  a_late: only the x.U operand comes from
    // the preceding grid, the wait sits in front of the low-rank term; otherwise wait here.
    if (!sp.a_late) asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int n_live = p.n_slots ? min(__ldg(p.n_slots), sp.n_problems) : sp.n_problems;
    const long total = (long)n_live * sp.ips;
    const int it_lo = (int)((long)blockIdx.x * total / gridDim.x);
    const int it_hi = (int)((long)(blockIdx.x + 1) * total / gridDim.x);
    if (it_lo >= it_hi) {
        // a dependent launch must not end before the launch it depends on has: later launches of the
        // stream order themselves after this grid only
        if (sp.a_late) asm volatile("griddepcontrol.wait;" ::: "memory");
        return;
    }

    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem);
    uint4* xs = reinterpret_cast<uint4*>(smem + sp.off_xs);
    float2* ox = reinterpret_cast<float2*>(smem + sp.off_ox);
    __half* as = reinterpret_cast<__half*>(smem + sp.off_as);
    float4* red = reinterpret_cast<float4*>(smem + sp.off_red);
    const uint32_t xs_a = smem_u32(xs), ox_a = smem_u32(ox);
    const uint32_t ring_a = smem_u32(smem + sp.off_ring) + (uint32_t)(w * S * sp.stage_bytes);
    const uint32_t bar_a = smem_u32(bars) + (uint32_t)(w * kMaxStages * 8);

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(bar_a + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    // ---- per-slot data and item description: one copy for the fetch cursor, one for the compute loop
    struct Slot {
        int slot = -1, cnt = 0, e0 = 0;
        const unsigned char* codes = nullptr;
        const unsigned char* sv = nullptr;
        const float* norms = nullptr;
        const float* centroids = nullptr;
        const __half* bias = nullptr;
    };
    auto load_slot = [&](Slot& sc, int slot) {
        if (slot == sc.slot) return;
        sc.slot = slot;
        sc.cnt = p.slot_count ? __ldg(p.slot_count + slot) : p.max_rows;
        if (sc.cnt <= sp.cnt_lo || sc.cnt > sp.cnt_hi) sc.cnt = 0;     // not this launch's slot: skipped like an empty one
        sc.cnt = min(sc.cnt, p.max_rows);
        sc.e0 = p.slot_offset ? __ldg(p.slot_offset + slot) : slot * p.rows_stride;
        const int widx = p.slot_index ? __ldg(p.slot_index + slot) : slot;
        const glq_weight_t* W = p.table ? p.table + widx : &p.w;
        sc.codes = reinterpret_cast<const unsigned char*>(W->codes);
        sc.sv = (rank > 0 && p.a[0] != nullptr) ? reinterpret_cast<const unsigned char*>(W->sv) : nullptr;
        sc.norms = W->norms;
        sc.centroids = W->centroids;
        sc.bias = reinterpret_cast<const __half*>(W->bias);
    };
    // item of warp w in iteration it: (slot, pair, split) -> k range and chunk counts
    struct Item {
        int slot, pair, s, kb_lo, kb_hi, ncode, nch;
        bool valid;
    };
    auto make_item = [&](Item& im, const Slot& sc, int slot, int rem) {   // iteration = slot * ips + rem
        const int local = rem * kWarpsPerCta + w;
        im.slot = slot;
        im.pair = local >> sp.sk_log2;
        im.s = local & (sk - 1);
        im.valid = im.pair < sp.npairs && sc.cnt > 0;
        im.kb_lo = im.s * sp.kb_per_split;
        im.kb_hi = min(nkb, im.kb_lo + sp.kb_per_split);
        im.ncode = im.kb_hi > im.kb_lo ? (im.kb_hi - im.kb_lo + kStreamCB - 1) / kStreamCB : 0;
        im.nch = im.ncode + ((im.s == 0 && sc.sv != nullptr) ? ns : 0);
    };

    // ---- fetch cursor: runs over the same (item, chunk) sequence as the compute loop, S stages ahead
    bool dead = false;
    Slot fs, cs;
    Item fi;
    // cursors keep (iteration, slot, iteration within the slot) and ring positions incrementally: no divisions
    int f_it = it_lo, f_slot = it_lo / sp.ips, f_rem = it_lo % sp.ips, f_c = 0;
    int f_stage = 0, f_inflight = 0;      // next stage to fill, chunks issued and not yet consumed
    int c_stage = 0;                      // next stage to consume
    uint32_t c_phase = 0;                 // its mbarrier phase parity
    bool f_live = false;
    auto fetch_seek = [&]() {
        f_live = false;
        while (f_it < it_hi) {
            load_slot(fs, f_slot);
            make_item(fi, fs, f_slot, f_rem);
            if (fi.valid && fi.nch > 0) {
                f_live = true;
                return;
            }
            ++f_it;
            if (++f_rem == sp.ips) f_rem = 0, ++f_slot;
        }
    };
    auto fetch_one = [&]() {
        if (lane == 0) {
            const int stage = f_stage;
            const uint32_t bar = bar_a + 8 * stage;
            const uint32_t dst = ring_a + (uint32_t)(stage * sp.stage_bytes);
            const void* src;
            uint32_t bytes;
            if (f_c < fi.ncode) {
                const int kb0 = fi.kb_lo + f_c * kStreamCB;
                bytes = (uint32_t)(min(kStreamCB, fi.kb_hi - kb0) * 2 * BB);
                src = fs.codes + ((size_t)fi.pair * nkb + kb0) * (2 * BB);
            } else {
                bytes = 4096;
                src = fs.sv + ((size_t)fi.pair * ns + (f_c - fi.ncode)) * 4096;
            }
            mbar_expect_tx(bar, bytes);
            bulk_g2s(dst, src, bytes, bar);
        }
        if (++f_stage == S) f_stage = 0;
        ++f_inflight;
        if (++f_c >= fi.nch) {
            f_c = 0;
            ++f_it;
            if (++f_rem == sp.ips) f_rem = 0, ++f_slot;
            fetch_seek();
        }
    };
    // the consumer side of the ring: wait for the next stage / release it and refill
    auto ring_wait = [&]() -> uint32_t {
        mbar_wait(bar_a + 8 * c_stage, c_phase, dead);
        return ring_a + (uint32_t)(c_stage * sp.stage_bytes);
    };
    auto ring_release = [&]() {
        __syncwarp();
        if (++c_stage == S) c_stage = 0, c_phase ^= 1u;
        --f_inflight;
        if (f_live) fetch_one();
    };
    fetch_seek();
    while (f_live && f_inflight < S) fetch_one();

    uint32_t TL[2] = {0, 0}, TH[2] = {0, 0};  // codebook tables of the two tiles of a pair
    // integer path of the codebook format: coefficients of the two tiles' codebooks (tile_block_t2_i8)
    float cb_c0[2] = {0.f, 0.f}, cb_d0[2] = {0.f, 0.f}, cb_dh[2] = {0.f, 0.f}, cb_e[2] = {0.f, 0.f};
    bool cb_cross = false;
    int staged_slot = -1, red_par = 0;
    bool dep_waited = false;
    constexpr int ncol_i8 = 2 * kRows;  // digit columns staged on the integer path

    int c_slot = it_lo / sp.ips, c_rem = it_lo % sp.ips;
    for (int it = it_lo; it < it_hi; ++it, c_rem = (c_rem + 1 == sp.ips ? 0 : c_rem + 1), c_slot += (c_rem == 0)) {
        load_slot(cs, c_slot);
        Item im;
        make_item(im, cs, c_slot, c_rem);
        const int cnt = cs.cnt, e0 = cs.e0;

        // ---- activations of a new problem: staged once per CTA ----
        if (im.slot != staged_slot) {
            __syncthreads();
            if (cnt > 0) {
                if constexpr (I8)
                    stage_x_i8<FMT>(p, xs, ox, nkb, ncol_i8, e0, cnt, K);
                else
                    stage_x<FMT>(p, xs, ox, 0, nkb, e0, 0, cnt, K);
                if (cs.sv != nullptr && !sp.a_late) {
                    const int na = swiglu ? 2 : 1, r8 = rank / 8;
                    for (int idx = tid; idx < na * kRows * r8; idx += kThreads) {
                        const int i = idx / (kRows * r8), rem = idx % (kRows * r8);
                        const int row = rem / r8, ch = rem % r8;
                        uint4 v = make_uint4(0, 0, 0, 0);
                        if (row < cnt && p.a[i] != nullptr)
                            v = __ldg(reinterpret_cast<const uint4*>(p.a[i] + (size_t)(e0 + row) * p.lda) + ch);
                        reinterpret_cast<uint4*>(as)[idx] = v;
                    }
                }
            }
            __syncthreads();
            staged_slot = im.slot;
            if constexpr (FMT == GLQ_FMT_T2) {
                // a fused gate|up weight carries two codebooks (4 floats each)
                if constexpr (I8) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const float* cbk = cs.centroids + ((j && swiglu) ? 4 : 0);
                        const float c0 = __ldg(cbk), c1 = __ldg(cbk + 1), c2 = __ldg(cbk + 2), c3 = __ldg(cbk + 3);
                        cb_c0[j] = c0;
                        cb_d0[j] = c1 - c0;
                        cb_dh[j] = 0.5f * (c2 - c0) - (c1 - c0);
                        cb_e[j] = (c3 - c2) - (c1 - c0);
                    }
                    // a cross term below 2^-22 of the codebook's span (the residue of an iterative codebook
                    // fit) is dropped: its share of an output is below 2^-16 of the output for K <= 2^16
                    cb_cross = false;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const float span = fabsf(cb_c0[j]) + fabsf(cb_c0[j] + cb_d0[j]) + fabsf(cb_dh[j]);
                        if (fabsf(cb_e[j]) > span * 2.384185791015625e-7f) cb_cross = true;
                    }
                } else {
                    make_t2_tables(cs.centroids, TL[0], TH[0]);
                    make_t2_tables(cs.centroids + (swiglu ? 4 : 0), TL[1], TH[1]);
                }
            }
        }
        if (!im.valid) continue;
        const int nt_live = I8 ? NT : min(NT, (cnt + 7) >> 3);     // fp16 path: activation tiles that hold rows

        // accumulators [tile in pair][activation tile]: {row g: 2 values, row g+8: 2 values}.
        // fp16 path: the two values are activation rows 2t, 2t+1 of the tile; integer path: only
        // [0] and [2] are used (activation row t of the tile)
        float acc[2][NT][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[j][nt][q] = 0.f;

        // ---- code chunks ----
        for (int c = 0; c < im.ncode; ++c) {
            const uint32_t st = ring_wait();
            const int kb0 = im.kb_lo + c * kStreamCB;
            const int nblk = min(kStreamCB, im.kb_hi - kb0);
#pragma unroll
            for (int b = 0; b < kStreamCB; ++b) {
                if (b >= nblk) break;
                const int kb = kb0 + b;
                if constexpr (I8) {
                    uint4 bx[NT][2];
                    float2 o[NT];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                        for (int i = 0; i < kPieces; ++i)
                            bx[nt][i] = lds128(
                                xs_a + (uint32_t)((((kb * kPieces + i) * ncol_i8) + nt * 8 + g) * 4 + t) * 16u);
                        const uint2 ov = lds64(ox_a + (uint32_t)(kb * kRows + nt * 4 + t) * 8u);
                        o[nt] = make_float2(__uint_as_float(ov.x), __uint_as_float(ov.y));
                    }
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint32_t blk = st + (uint32_t)((b * 2 + j) * BB);
                        const uint4 q = lds128(blk + lane * 16);
                        if constexpr (FMT == GLQ_FMT_T2) {
                            int cq[NT][4], cb[NT][4], ce[NT][4];
                            tile_block_t2_i8<NT>(q, bx, cb_cross, cq, cb, ce);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                const float kd = cb_d0[j] * o[nt].x, kh = cb_dh[j] * o[nt].x;
                                const float base = cb_c0[j] * o[nt].y;
                                float v0 = fmaf(kd, (float)(cq[nt][0] + (cq[nt][1] << 8)),
                                                fmaf(kh, (float)(cb[nt][0] + (cb[nt][1] << 8)), base));
                                float v1 = fmaf(kd, (float)(cq[nt][2] + (cq[nt][3] << 8)),
                                                fmaf(kh, (float)(cb[nt][2] + (cb[nt][3] << 8)), base));
                                if (cb_cross) {
                                    const float ke = cb_e[j] * o[nt].x;
                                    v0 = fmaf(ke, (float)(ce[nt][0] + (ce[nt][1] << 8)), v0);
                                    v1 = fmaf(ke, (float)(ce[nt][2] + (ce[nt][3] << 8)), v1);
                                }
                                acc[j][nt][0] += v0;
                                acc[j][nt][2] += v1;
                            }
                        } else {
                            const uint2 szv = lds64(blk + 512 + g * 8);
                            int ci[NT][4];
                            tile_block_i8<FMT, NT>(q, bx, ci);
                            const __half2 sz0 = *reinterpret_cast<const __half2*>(&szv.x);
                            const __half2 sz1 = *reinterpret_cast<const __half2*>(&szv.y);
                            const float s0 = __low2float(sz0), z0 = __high2float(sz0);
                            const float s1 = __low2float(sz1), z1 = __high2float(sz1);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                const float f0 = (float)(ci[nt][0] + (ci[nt][1] << 8)) * o[nt].x;
                                const float f1 = (float)(ci[nt][2] + (ci[nt][3] << 8)) * o[nt].x;
                                acc[j][nt][0] = fmaf(s0, fmaf(-z0, o[nt].y, f0), acc[j][nt][0]);
                                acc[j][nt][2] = fmaf(s1, fmaf(-z1, o[nt].y, f1), acc[j][nt][2]);
                            }
                        }
                    }
                } else {
                    uint4 bx[NT][4];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int col = (nt * 8 + g) & (ntc - 1);
#pragma unroll
                        for (int i = 0; i < kPieces; ++i)
                            bx[nt][i] = (nt < nt_live && (NT > 1 || g < ntc))
                                            ? lds128(xs_a + (uint32_t)(((kb * kPieces + i) * ntc + col) * 4 + t) * 16u)
                                            : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint32_t blk = st + (uint32_t)((b * 2 + j) * BB);
                        const uint4 q = lds128(blk + lane * 16);
                        if constexpr (kAffine) {
                            const uint2 szv = lds64(blk + 512 + g * 8);
                            float cc[NT][4];
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                                for (int q4 = 0; q4 < 4; ++q4) cc[nt][q4] = 0.f;
                            tile_block<FMT, NT>(q, bx, 0, 0, cc, nt_live);
                            const __half2 sz0 = *reinterpret_cast<const __half2*>(&szv.x);
                            const __half2 sz1 = *reinterpret_cast<const __half2*>(&szv.y);
                            const float s0 = __low2float(sz0), z0 = __high2float(sz0);
                            const float s1 = __low2float(sz1), z1 = __high2float(sz1);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                if (nt >= nt_live) continue;
                                const int col = (nt * 8 + 2 * t) & (ntc - 1);
                                const uint4 ov = lds128(ox_a + (uint32_t)(kb * ntc + col) * 8u);
                                const float ox0 = __uint_as_float(ov.x), xx0 = __uint_as_float(ov.y);
                                const float ox1 = __uint_as_float(ov.z), xx1 = __uint_as_float(ov.w);
                                acc[j][nt][0] = fmaf(s0, fmaf(-z0, xx0, cc[nt][0] - ox0), acc[j][nt][0]);
                                acc[j][nt][1] = fmaf(s0, fmaf(-z0, xx1, cc[nt][1] - ox1), acc[j][nt][1]);
                                acc[j][nt][2] = fmaf(s1, fmaf(-z1, xx0, cc[nt][2] - ox0), acc[j][nt][2]);
                                acc[j][nt][3] = fmaf(s1, fmaf(-z1, xx1, cc[nt][3] - ox1), acc[j][nt][3]);
                            }
                        } else {
                            tile_block<FMT, NT>(q, bx, TL[j], TH[j], acc[j], nt_live);
                        }
                    }
                }
            }
            ring_release();
        }

        // ---- k splits of this pair: fixed-order reduction through shared memory ----
        if (sk > 1) {
            float4* rbuf = red + (size_t)red_par * (kWarpsPerCta * 2 * NT * 32);
            if (im.s != 0) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                        rbuf[((w * 2 + j) * NT + nt) * 32 + lane] =
                            make_float4(acc[j][nt][0], acc[j][nt][1], acc[j][nt][2], acc[j][nt][3]);
            }
            named_bar_sync(1 + w / sk, sk * 32);
            if (im.s == 0) {
                for (int s2 = 1; s2 < sk; ++s2)
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const float4 v = rbuf[(((w + s2) * 2 + j) * NT + nt) * 32 + lane];
                            acc[j][nt][0] += v.x;
                            acc[j][nt][1] += v.y;
                            acc[j][nt][2] += v.z;
                            acc[j][nt][3] += v.w;
                        }
            }
            red_par ^= 1;
        }
        if (im.s != 0) continue;

        // ---- low-rank term on the fp16 op: SV chunks from the ring, a from shared memory.
        // lo[j][m] covers activation rows 8m + 2t, 8m + 2t + 1 (the columns of the op)
        constexpr int NM = (kRows + 7) / 8;
        float lo[2][NM][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int m = 0; m < NM; ++m)
#pragma unroll
                for (int q = 0; q < 4; ++q) lo[j][m][q] = 0.f;
        const int nsv = im.nch - im.ncode;
        if (sp.a_late && nsv > 0 && !dep_waited) {
            // programmatic dependent launch: everything up to here overlapped the launch that produces x.U
            asm volatile("griddepcontrol.wait;" ::: "memory");
            dep_waited = true;
        }
        for (int c = 0; c < nsv; ++c) {
            const uint32_t st = ring_wait();
            // every lane runs the (warp-wide) op; lanes beyond the rank feed zeros
            const int cc0 = c * 64 + 16 * t;
            const bool in_rank = cc0 < rank;
            const uint4 z4 = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t pa = st + (uint32_t)((j * 16 + g) * 128 + t * 32);
                const uint4 sa0 = in_rank ? lds128(pa) : z4, sa1 = in_rank ? lds128(pa + 16) : z4;
                const uint4 sb0 = in_rank ? lds128(pa + 8 * 128) : z4, sb1 = in_rank ? lds128(pa + 8 * 128 + 16) : z4;
#pragma unroll
                for (int m = 0; m < NM; ++m) {
                    const int row = m * 8 + g;
                    const bool ok = in_rank && row < kRows;
                    uint4 av0 = z4, av1 = z4;
                    if (!sp.a_late) {
                        const uint4* pav = reinterpret_cast<const uint4*>(
                            as + ((size_t)(swiglu ? j : 0) * kRows + (ok ? row : 0)) * rank + (ok ? cc0 : 0));
                        if (ok) av0 = pav[0], av1 = pav[1];
                    } else if (ok && row < cnt) {
                        // written by the launch before this one, which has completed by now (see the wait above)
                        const uint4* pav = reinterpret_cast<const uint4*>(p.a[swiglu ? j : 0] + (size_t)(e0 + row) * p.lda + cc0);
                        av0 = ld_global_u4(pav);
                        av1 = ld_global_u4(pav + 1);
                    }
                    mma16816(lo[j][m], sa0.x, sb0.x, sa0.y, sb0.y, av0.x, av0.y);
                    mma16816(lo[j][m], sa0.z, sb0.z, sa0.w, sb0.w, av0.z, av0.w);
                    mma16816(lo[j][m], sa1.x, sb1.x, sa1.y, sb1.y, av1.x, av1.y);
                    mma16816(lo[j][m], sa1.z, sb1.z, sa1.w, sb1.w, av1.z, av1.w);
                }
            }
            ring_release();
        }

        // ---- epilogue: this lane's activation rows, weight rows g and g+8 of both tiles ----
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            constexpr int kVals = I8 ? 1 : 2;  // activation rows this lane owns per tile
#pragma unroll
            for (int e = 0; e < kVals; ++e) {
                const int row = I8 ? (nt * 4 + t) : (nt * 8 + 2 * t + e);
                float val[2][2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    float n0 = 1.f, n1 = 1.f;
                    if constexpr (FMT == GLQ_FMT_T2) {
                        n0 = __ldg(cs.norms + ((size_t)im.pair * 2 + j) * 16 + g);
                        n1 = __ldg(cs.norms + ((size_t)im.pair * 2 + j) * 16 + g + 8);
                    }
                    float v0 = round16(acc[j][nt][I8 ? 0 : e] * n0);
                    float v1 = round16(acc[j][nt][I8 ? 2 : 2 + e] * n1);
                    if (nsv > 0) {
                        float l0, l1;
                        if constexpr (I8) {
                            // the low-rank op holds rows 2t', 2t'+1 in lane t': fetch this lane's row
                            const int src = (g << 2) | ((row & 7) >> 1);
                            const float a0 = __shfl_sync(0xffffffffu, lo[j][0][0], src);
                            const float a1 = __shfl_sync(0xffffffffu, lo[j][0][1], src);
                            const float b0 = __shfl_sync(0xffffffffu, lo[j][0][2], src);
                            const float b1 = __shfl_sync(0xffffffffu, lo[j][0][3], src);
                            l0 = (row & 1) ? a1 : a0;
                            l1 = (row & 1) ? b1 : b0;
                        } else {
                            l0 = lo[j][nt][e];
                            l1 = lo[j][nt][2 + e];
                        }
                        v0 = round16(v0 + round16(l0));
                        v1 = round16(v1 + round16(l1));
                    }
                    val[j][0] = v0;
                    val[j][1] = v1;
                }
                if (row >= cnt) continue;
                if (swiglu) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int n = im.pair * kRowTile + g + 8 * h;
                        if (n < N)
                            p.y[(size_t)(e0 + row) * p.ldy + n] =
                                __float2half_rn(round16(silu16(val[0][h]) * val[1][h]));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int n = (im.pair * 2 + j) * kRowTile + g + 8 * h;
                            if (n < N) {
                                float v = val[j][h];
                                if (cs.bias) v = round16(v + __half2float(__ldg(cs.bias + n)));
                                if (p.entry_scale) v = round16(__half2float(__ldg(p.entry_scale + e0 + row)) * v);
                                p.y[(size_t)(e0 + row) * p.ldy + n] = __float2half_rn(v);
                            }
                        }
                }
            }
        }
    }
    // see the early exit above: a dependent grid ends only after the grid it depends on
    if (sp.a_late && !dep_waited) asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace glq
