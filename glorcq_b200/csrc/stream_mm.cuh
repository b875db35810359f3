// Persistent streaming variant of the grouped skinny matmul (same maths and the same operands as
// skinny_mm.cuh; this is the fast path, that one the general fallback).
//
// The decode GEMV is bound by the HBM stream of packed codes, so this kernel is built as a copy
// pipeline with compute attached:
//   * one CTA per SM, each CTA walks a contiguous range of work items (problem, row-tile pair,
//     k split), so the activations of a problem are staged once per CTA and not once per tile;
//   * every warp owns a ring of shared-memory stages that is filled by bulk asynchronous copies
//     (cp.async.bulk global -> shared, completion on an mbarrier), issued by the warp itself several
//     stages ahead of where it computes, across item boundaries: the bytes in flight per SM stay
//     constant (about 100 KB) instead of collapsing at every tile boundary.  In the tiled layout a
//     row tile's codes for consecutive k blocks are contiguous, so a stage is one 2 KB copy per tile
//     plus one small copy of its scales; the 16 rows of the output-side factor SV ride the same ring;
//   * a warp item is TWO row tiles that share the activation fragments (gate and up of one expert,
//     or two consecutive tiles of one matrix), halving the shared-memory traffic per weight;
//   * k splits of a tile are the warps of one CTA, reduced through shared memory in a fixed order
//     (named barrier per tile group): no global scratch, no atomics, deterministic.
// Every mbarrier wait is bounded; a wait that runs out records an error word and carries on, so
// the kernel always terminates.  No cluster launch, no multicast.
#pragma once

#include "skinny_mm.cuh"

namespace glq {

constexpr int kMaxStages = 4;
constexpr int kStreamCB = 4;  // k blocks per ring stage and tile

struct StreamParams {
    SkinnyParams b;    // operands (geometry fields of the fallback kernel unused except ntc, nkb, group_blocks)
    int N, K, rank;
    int n_problems;
    int sk;            // k splits (warps of one CTA): 1, 2, 4 or 8
    int kb_per_split;
    int npairs;        // warp items per problem and split: tile pairs
    int ips;           // iterations (8 warp items) per problem
    int stages;        // ring depth
    int stage_bytes;
    int off_xs, off_ox, off_as, off_ring, off_red;  // shared memory carve-up (bytes)
};

// ---- mbarrier / bulk copy primitives -----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
    while (!mbar_test_wait(bar, parity)) {
        if (global_ns() - t0 > 2000000ull) {
            glq_ok(false, 100, bar, parity);
            dead = true;
            return;
        }
        __nanosleep(64);
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- one k block of one tile against preloaded activation fragments ---------------------------
template <int FMT, int NTT>
__device__ __forceinline__ void tile_block(const uint4 q, const uint4 (&bx)[NTT][4], uint32_t TL, uint32_t TH,
                                           float (&c)[NTT][4]) {
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
                const uint4 b = bx[tt][u];
                mma16816(c[tt], ha[0], hb[0], ha[1], hb[1], b.x, b.y);
                mma16816(c[tt], ha[2], hb[2], ha[3], hb[3], b.z, b.w);
            }
        }
    }
}

// ---- the kernel -----------------------------------------------------------------------------------
template <int FMT, int NW, int NTT>
__global__ void __launch_bounds__(kThreads, 1) stream_kernel(const StreamParams sp) {
    using F = Fmt<FMT>;
    static_assert(FMT != GLQ_FMT_F16, "dense weights use the fallback kernel");
    constexpr bool kAffine = (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_Q4);
    constexpr int kPieces = F::XS / 4;                      // uint4 fragments per k block, lane and column
    constexpr int kCodeBytes = kStreamCB * 512;              // per tile and stage
    constexpr int kSzBytes = kAffine ? kStreamCB * 64 : 0;   // per tile and stage
    const SkinnyParams& p = sp.b;
    extern __shared__ __align__(128) unsigned char smem[];

    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int N = sp.N, K = sp.K, rank = sp.rank;
    const int ntiles = (N + kRowTile - 1) / kRowTile;
    const int nkb = p.nkb, gb = p.group_blocks, ntc = p.ntc;
    const int G = (nkb + gb - 1) / gb;
    const int S = sp.stages, sk = sp.sk;

    const int n_live = p.n_slots ? min(__ldg(p.n_slots), sp.n_problems) : sp.n_problems;
    const long total = (long)n_live * sp.ips;
    const int it_lo = (int)((long)blockIdx.x * total / gridDim.x);
    const int it_hi = (int)((long)(blockIdx.x + 1) * total / gridDim.x);
    if (it_lo >= it_hi) return;

    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem);
    uint4* xs = reinterpret_cast<uint4*>(smem + sp.off_xs);
    float2* ox = reinterpret_cast<float2*>(smem + sp.off_ox);
    __half* as = reinterpret_cast<__half*>(smem + sp.off_as);
    unsigned char* ring = smem + sp.off_ring + (size_t)w * S * sp.stage_bytes;
    float4* red = reinterpret_cast<float4*>(smem + sp.off_red);

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_u32(&bars[w * kMaxStages + s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    // ---- item description, shared by the fetch cursor and the compute cursor ----
    struct Item {
        int it, slot, pair, s, kb_lo, kb_hi, ncode, nch, rt[2];
        bool valid, tile_ok[2];
        const unsigned char* codes[2];
        const unsigned char* sz[2];
        const unsigned char* sv[2];
    };
    struct SlotCache {
        int slot = -1, cnt = 0;
        glq_weight_t W[NW];
    };
    auto resolve = [&](Item& im, SlotCache& sc, int it) {
        im.it = it;
        im.slot = it / sp.ips;
        const int local = (it % sp.ips) * kWarpsPerCta + w;
        im.pair = local / sk;
        im.s = local % sk;
        if (im.slot != sc.slot) {
            sc.slot = im.slot;
            sc.cnt = min(p.slot_count ? __ldg(p.slot_count + im.slot) : p.max_rows, p.max_rows);
            const int widx = p.slot_index ? __ldg(p.slot_index + im.slot) : im.slot;
#pragma unroll
            for (int i = 0; i < NW; ++i) sc.W[i] = p.table[i] ? p.table[i][widx] : p.w[i];
        }
        im.valid = im.pair < sp.npairs && sc.cnt > 0;
        im.kb_lo = im.s * sp.kb_per_split;
        im.kb_hi = min(nkb, im.kb_lo + sp.kb_per_split);
        im.ncode = im.kb_hi > im.kb_lo ? (im.kb_hi - im.kb_lo + kStreamCB - 1) / kStreamCB : 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int wi = NW == 2 ? j : 0;
            im.rt[j] = NW == 2 ? im.pair : 2 * im.pair + j;
            im.tile_ok[j] = im.rt[j] < ntiles;
            im.codes[j] = reinterpret_cast<const unsigned char*>(sc.W[wi].codes);
            im.sz[j] = reinterpret_cast<const unsigned char*>(sc.W[wi].sz);
            im.sv[j] = reinterpret_cast<const unsigned char*>(sc.W[wi].sv);
        }
        const bool has_lr = rank > 0 && im.sv[0] != nullptr && p.a[0] != nullptr;
        im.nch = im.ncode + ((im.s == 0 && has_lr) ? (rank + 63) / 64 : 0);
    };

    // ---- fetch side: issue the copies of chunk c of item im into ring stage (seq % S) ----
    auto issue = [&](const Item& im, int c, int seq) {
        const int stage = seq % S;
        const uint32_t bar = smem_u32(&bars[w * kMaxStages + stage]);
        const uint32_t dst = smem_u32(ring + (size_t)stage * sp.stage_bytes);
        if (c < im.ncode) {
            const int kb0 = im.kb_lo + c * kStreamCB;
            const int nblk = min(kStreamCB, im.kb_hi - kb0);
            const int g0 = kb0 / gb, g1 = (kb0 + nblk - 1) / gb;
            if (lane == 0) {
                uint32_t bytes = 0;
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    if (im.tile_ok[j]) bytes += nblk * 512 + (kAffine ? (g1 - g0 + 1) * 64 : 0);
                mbar_expect_tx(bar, bytes);
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    if (im.tile_ok[j]) {
                        bulk_g2s(dst + j * kCodeBytes, im.codes[j] + ((size_t)im.rt[j] * nkb + kb0) * 512, nblk * 512,
                                 bar);
                        if constexpr (kAffine)
                            bulk_g2s(dst + 2 * kCodeBytes + j * kSzBytes, im.sz[j] + ((size_t)im.rt[j] * G + g0) * 64,
                                     (g1 - g0 + 1) * 64, bar);
                    }
            }
        } else {
            // 16 rows x (up to) 64 columns of SV per tile: one 128-byte copy per row and lane
            const int r0 = (c - im.ncode) * 64;
            const int j = lane >> 4, row = im.rt[j] * kRowTile + (lane & 15);
            const uint32_t nb = (im.tile_ok[j] && row < N) ? (uint32_t)min(64, rank - r0) * 2u : 0u;
            uint32_t tot = nb;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
            if (lane == 0) mbar_expect_tx(bar, tot);
            __syncwarp();
            if (nb) bulk_g2s(dst + j * 2048 + (lane & 15) * 128, im.sv[j] + ((size_t)row * rank + r0) * 2, nb, bar);
        }
    };

    // The fetch cursor runs over the same (item, chunk) sequence as the compute loop, S stages ahead.
    Item fi;
    SlotCache fcache, ccache;
    int f_it = it_lo, f_c = 0, fseq = 0, cseq = 0;
    bool f_live = false;
    auto fetch_seek = [&]() {  // position the fetch cursor on the next item that has chunks
        f_live = false;
        while (f_it < it_hi) {
            resolve(fi, fcache, f_it);
            if (fi.valid && fi.nch > 0) {
                f_live = true;
                return;
            }
            ++f_it;
        }
    };
    auto fetch_one = [&]() {
        issue(fi, f_c, fseq);
        ++fseq;
        if (++f_c >= fi.nch) {
            f_c = 0;
            ++f_it;
            fetch_seek();
        }
    };
    fetch_seek();
    while (f_live && fseq < S) fetch_one();

    uint32_t TL[NW], TH[NW];
    int staged_slot = -1;
    int red_par = 0;
    bool dead = false;

    for (int it = it_lo; it < it_hi; ++it) {
        Item im;
        resolve(im, ccache, it);
        const int cnt = ccache.cnt;
        const glq_weight_t(&W)[NW] = ccache.W;

        // ---- activations of a new problem: stage x (all of K) and a = x.U once per CTA ----
        if (im.slot != staged_slot) {
            __syncthreads();
            const int e0s = p.slot_offset ? __ldg(p.slot_offset + im.slot) : im.slot * p.rows_stride;
            if (cnt > 0) {
                stage_x<FMT>(p, xs, ox, 0, nkb, e0s, 0, cnt, K);
                if (rank > 0 && p.a[0] != nullptr) {
                    for (int idx = tid; idx < NW * ntc * (rank / 8); idx += kThreads) {
                        const int i = idx / (ntc * (rank / 8)), rem = idx % (ntc * (rank / 8));
                        const int col = rem / (rank / 8), ch = rem % (rank / 8);
                        uint4 v = make_uint4(0, 0, 0, 0);
                        if (col < cnt && p.a[i] != nullptr)
                            v = __ldg(reinterpret_cast<const uint4*>(p.a[i] + (size_t)(e0s + col) * p.lda) + ch);
                        reinterpret_cast<uint4*>(as)[idx] = v;
                    }
                }
            }
            __syncthreads();
            staged_slot = im.slot;
#pragma unroll
            for (int i = 0; i < NW; ++i) {
                TL[i] = TH[i] = 0;
                if constexpr (FMT == GLQ_FMT_T2) make_t2_tables(W[i].centroids, TL[i], TH[i]);
            }
        }
        if (!im.valid) continue;
        const int e0 = p.slot_offset ? __ldg(p.slot_offset + im.slot) : im.slot * p.rows_stride;

        float acc[2][NTT][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int tt = 0; tt < NTT; ++tt)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[j][tt][q] = 0.f;

        // values the epilogue needs, requested early
        float nrm[2][2] = {{1.f, 1.f}, {1.f, 1.f}};
        if constexpr (FMT == GLQ_FMT_T2) {
            if (im.s == 0) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int r0 = min(im.rt[j] * kRowTile + g, N - 1), r1 = min(im.rt[j] * kRowTile + g + 8, N - 1);
                    nrm[j][0] = __ldg(W[NW == 2 ? j : 0].norms + r0);
                    nrm[j][1] = __ldg(W[NW == 2 ? j : 0].norms + r1);
                }
            }
        }

        // ---- code chunks ----
        for (int c = 0; c < im.ncode; ++c) {
            const int stage = cseq % S;
            mbar_wait(smem_u32(&bars[w * kMaxStages + stage]), (cseq / S) & 1, dead);
            const unsigned char* st = ring + (size_t)stage * sp.stage_bytes;
            const int kb0 = im.kb_lo + c * kStreamCB;
            const int nblk = min(kStreamCB, im.kb_hi - kb0);
            const int g0 = kb0 / gb;
#pragma unroll 1
            for (int b = 0; b < nblk; ++b) {
                const int kb = kb0 + b;
                uint4 bx[NTT][4];
#pragma unroll
                for (int tt = 0; tt < NTT; ++tt) {
                    const int col = (tt * 8 + g) & (ntc - 1);
#pragma unroll
                    for (int i = 0; i < kPieces; ++i)
                        bx[tt][i] = (NTT > 1 || g < ntc) ? xs[(((size_t)kb * kPieces + i) * ntc + col) * 4 + t]
                                                        : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    if (!im.tile_ok[j]) continue;
                    const uint4 q = reinterpret_cast<const uint4*>(st + j * kCodeBytes)[b * 32 + lane];
                    if constexpr (kAffine) {
                        float cc[NTT][4];
#pragma unroll
                        for (int tt = 0; tt < NTT; ++tt)
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) cc[tt][q4] = 0.f;
                        tile_block<FMT, NTT>(q, bx, 0, 0, cc);
                        const uint2 szv =
                            reinterpret_cast<const uint2*>(st + 2 * kCodeBytes + j * kSzBytes)[(kb / gb - g0) * 8 + g];
                        const __half2 sz0 = *reinterpret_cast<const __half2*>(&szv.x);
                        const __half2 sz1 = *reinterpret_cast<const __half2*>(&szv.y);
                        const float s0 = __low2float(sz0), z0 = __high2float(sz0);
                        const float s1 = __low2float(sz1), z1 = __high2float(sz1);
#pragma unroll
                        for (int tt = 0; tt < NTT; ++tt) {
                            const int col = (tt * 8 + 2 * t) & (ntc - 1);
                            const float4 o = *reinterpret_cast<const float4*>(&ox[kb * ntc + col]);
                            acc[j][tt][0] = fmaf(s0, fmaf(-z0, o.y, cc[tt][0] - o.x), acc[j][tt][0]);
                            acc[j][tt][1] = fmaf(s0, fmaf(-z0, o.w, cc[tt][1] - o.z), acc[j][tt][1]);
                            acc[j][tt][2] = fmaf(s1, fmaf(-z1, o.y, cc[tt][2] - o.x), acc[j][tt][2]);
                            acc[j][tt][3] = fmaf(s1, fmaf(-z1, o.w, cc[tt][3] - o.z), acc[j][tt][3]);
                        }
                    } else {
                        tile_block<FMT, NTT>(q, bx, TL[NW == 2 ? j : 0], TH[NW == 2 ? j : 0], acc[j]);
                    }
                }
            }
            __syncwarp();
            ++cseq;
            if (f_live) fetch_one();
        }

        // ---- k splits of this tile pair: fixed-order reduction through shared memory ----
        if (sk > 1) {
            float4* rbuf = red + (size_t)red_par * (kWarpsPerCta * 2 * NTT * 32);
            if (im.s != 0) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int tt = 0; tt < NTT; ++tt)
                        rbuf[((w * 2 + j) * NTT + tt) * 32 + lane] =
                            make_float4(acc[j][tt][0], acc[j][tt][1], acc[j][tt][2], acc[j][tt][3]);
            }
            named_bar_sync(1 + w / sk, sk * 32);
            if (im.s == 0) {
                for (int s2 = 1; s2 < sk; ++s2)
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int tt = 0; tt < NTT; ++tt) {
                            const float4 v = rbuf[(((w + s2) * 2 + j) * NTT + tt) * 32 + lane];
                            acc[j][tt][0] += v.x;
                            acc[j][tt][1] += v.y;
                            acc[j][tt][2] += v.z;
                            acc[j][tt][3] += v.w;
                        }
            }
            red_par ^= 1;
        }
        if (im.s != 0) continue;

        // ---- low-rank term: SV chunks from the ring, a from shared memory ----
        float lo[2][NTT][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int tt = 0; tt < NTT; ++tt)
#pragma unroll
                for (int q = 0; q < 4; ++q) lo[j][tt][q] = 0.f;
        const int nsv = im.nch - im.ncode;
        for (int c = 0; c < nsv; ++c) {
            const int stage = cseq % S;
            mbar_wait(smem_u32(&bars[w * kMaxStages + stage]), (cseq / S) & 1, dead);
            const unsigned char* st = ring + (size_t)stage * sp.stage_bytes;
            // every lane runs the tensor-core op (it is warp-wide); lanes beyond the rank feed zeros
            const int cc0 = c * 64 + 16 * t;
            const bool in_rank = cc0 < rank;
            const uint4 z4 = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (!im.tile_ok[j]) continue;
                const uint4* pa = reinterpret_cast<const uint4*>(st + j * 2048 + g * 128 + t * 32);
                const uint4* pb = reinterpret_cast<const uint4*>(st + j * 2048 + (g + 8) * 128 + t * 32);
                const uint4 sa0 = in_rank ? pa[0] : z4, sa1 = in_rank ? pa[1] : z4;
                const uint4 sb0 = in_rank ? pb[0] : z4, sb1 = in_rank ? pb[1] : z4;
#pragma unroll
                for (int tt = 0; tt < NTT; ++tt) {
                    const int col = (tt * 8 + g) & (ntc - 1);
                    const uint4* pav =
                        reinterpret_cast<const uint4*>(as + ((size_t)(NW == 2 ? j : 0) * ntc + col) * rank + cc0);
                    const uint4 av0 = in_rank ? pav[0] : z4, av1 = in_rank ? pav[1] : z4;
                    mma16816(lo[j][tt], sa0.x, sb0.x, sa0.y, sb0.y, av0.x, av0.y);
                    mma16816(lo[j][tt], sa0.z, sb0.z, sa0.w, sb0.w, av0.z, av0.w);
                    mma16816(lo[j][tt], sa1.x, sb1.x, sa1.y, sb1.y, av1.x, av1.y);
                    mma16816(lo[j][tt], sa1.z, sb1.z, sa1.w, sb1.w, av1.z, av1.w);
                }
            }
            __syncwarp();
            ++cseq;
            if (f_live) fetch_one();
        }

        // ---- epilogue ----
        float res[2][NTT][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int wi = NW == 2 ? j : 0;
            const __half* bias = reinterpret_cast<const __half*>(W[wi].bias);
            const int r0c = min(im.rt[j] * kRowTile + g, N - 1), r1c = min(im.rt[j] * kRowTile + g + 8, N - 1);
            const float b0 = bias ? __half2float(__ldg(bias + r0c)) : 0.f;
            const float b1 = bias ? __half2float(__ldg(bias + r1c)) : 0.f;
#pragma unroll
            for (int tt = 0; tt < NTT; ++tt)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float v = round16(acc[j][tt][q] * nrm[j][q >> 1]);
                    if (nsv > 0) v = round16(v + round16(lo[j][tt][q]));
                    if (bias) v = round16(v + (q < 2 ? b0 : b1));
                    res[j][tt][q] = v;
                }
        }
#pragma unroll
        for (int tt = 0; tt < NTT; ++tt)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int row = tt * 8 + 2 * t + (q & 1);
                if (row >= cnt) continue;
                if constexpr (NW == 2) {
                    const int n = im.rt[0] * kRowTile + g + (q < 2 ? 0 : 8);
                    if (n < N)
                        p.y[(size_t)(e0 + row) * p.ldy + n] =
                            __float2half_rn(round16(silu16(res[0][tt][q]) * res[1][tt][q]));
                } else {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int n = im.rt[j] * kRowTile + g + (q < 2 ? 0 : 8);
                        if (im.tile_ok[j] && n < N) {
                            float v = res[j][tt][q];
                            if (p.entry_scale) v = round16(__half2float(__ldg(p.entry_scale + e0 + row)) * v);
                            p.y[(size_t)(e0 + row) * p.ldy + n] = __float2half_rn(v);
                        }
                    }
                }
            }
    }
}

}  // namespace glq
