// SPDX-License-Identifier: Apache-2.0
//
// Persistent form of the tensor-memory dequant-GEMM (2-bit affine codes, tc_ts_kernel).
//
// One CTA per SM works through the list of (token tile, 128-feature tile) items; the warps keep their roles
// over all of a CTA's items, so barrier set-up, the TMEM allocation and the pipeline fill are paid once per
// CTA instead of once per tile.  Roles, stage layout and the epilogue arithmetic are those of tc_ts_kernel:
// 16 producer warps unpack the codes of a 128-channel stage into the tensor-memory ring, one warp issues
// the MMAs, one thread bulk-copies the token operand.
//
//  * Work items are drawn from a grid-wide counter (zeroed by the pre-pass) by the loader warp and handed
//    to the other warps through a small queue in shared memory, so an SM that runs faster takes more items.
//  * The rings run on across item boundaries: the loader fetches the next item's token operand while the
//    producers still finish the current one.
//  * A finished accumulator is read into registers (epilogue arithmetic, fp16 pairs) and released at once;
//    the results go to y after the weight ring of the next item is full again, through a staging tile in
//    shared memory ([token][feature], two passes) with 16-byte row-contiguous stores.
//
// Every wait is bounded (tc_wait); a wait that runs out marks the CTA dead, all roles leave their loops
// and the kernel ends.
#pragma once

#include "tc_mm.cuh"

#ifndef GLQ_PS_FLUSH_AT
#define GLQ_PS_FLUSH_AT (S - 1)
#endif
#ifndef GLQ_PS_FLUSH_GAP
#define GLQ_PS_FLUSH_GAP 0
#endif

namespace glq {

constexpr int kPsQueue = 4;        // work items the loader may be ahead of the slowest warp

template <int TN, bool SW> struct TcPsCfg {
    using T = TcTsCfg<TN, SW>;
    static constexpr int NH = TN >= 128 ? 2 : 1;                 // the results leave in NH passes over a staging tile
    static constexpr int TH = TN / NH;                           // tokens per pass
    static constexpr int OUT_BYTES = TH * 256;                   // staged results [TH][128] fp16
    static constexpr size_t SMEM = (size_t)T::S * T::B_BYTES + OUT_BYTES + 1024;
    static_assert(SMEM <= 227 * 1024, "shared memory");
};

template <int TN, bool SW>
__global__ void __launch_bounds__(kTcThreads, 1) tc_ps_kernel(const TcParams p) {
    using C = TcTsCfg<TN, SW>;
    using P = TcPsCfg<TN, SW>;
    constexpr int S = C::S, NM = C::NM;
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * S + 4 + 2 * kPsQueue];
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;
    __shared__ int s_tile[kPsQueue];          // work items in the order the loader drew them; -1 ends the list

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sbase = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
    const uint32_t obase = sbase + (uint32_t)S * C::B_BYTES;      // staging tile of the results
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * S;
    const uint32_t bar_acc = bar_full + 16 * S, bar_acc_free = bar_acc + 8;
    const uint32_t bar_drained = bar_acc + 16, bar_stored = bar_acc + 24;   // staging tile written / read by all producers
    const uint32_t bar_tq_full = bar_acc + 32, bar_tq_empty = bar_tq_full + 8 * kPsQueue;
    volatile int* dead = &s_dead;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, kTcProducers + 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        mbar_init(bar_acc_free, kTcProducers);
        mbar_init(bar_drained, kTcProducers);
        mbar_init(bar_stored, kTcProducers);
        for (int i = 0; i < kPsQueue; ++i) {
            mbar_init(bar_tq_full + 8 * i, 1);
            mbar_init(bar_tq_empty + 8 * i, kTcProducers + 1);
        }
        s_dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTcProducers) tc_alloc(smem_u32(&s_tmem), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t ring = tmem + C::ACC;      // first column of the weight ring

    const int N = p.N;
    const bool has_lr = p.rank > 0 && p.a[0] != nullptr;
    const int nst = p.nkb + (has_lr ? p.ns : 0);
    const int n_work = p.n_ft * p.tiles_max;
    // next work item of this CTA (every consumer warp calls it with all lanes): -1 = none left or the CTA is dead
    auto next_item = [&](int n) -> int {
        const int qi = n % kPsQueue;
        const bool got = __all_sync(0xffffffffu, tc_wait(bar_tq_full + 8 * qi, (uint32_t)((n / kPsQueue) & 1), dead, 108));
        int wk = -1;
        if (got) wk = *reinterpret_cast<volatile int*>(&s_tile[qi]);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tq_empty + 8 * qi);
        return wk;
    };

    if (warp < kTcProducers) {
        // ================= producers: unpack into tensor memory, then the tile's epilogue =================
        const int g = lane >> 2, t = lane & 3;
        const int q = warp & 3, sub = warp >> 2;
        const int tl = 2 * q + (sub & 1), wh = sub >> 1;
        const uint32_t lane_base = (uint32_t)(16 * tl) << 16;
        int s = 0;
        uint32_t ph = 0;
        int it = 0;
        const int part = warp >> 2;                                // quarter of a pass's token columns
        const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16);
        const uint32_t orow = obase + (uint32_t)(q * 32 + lane) * 2u;
        // results of the tile before, fp16 pairs of this thread's feature: columns h*TH + part*TH/4 + 2i, +1
        constexpr int PK = TN / 8;
        constexpr int kFlushAt = GLQ_PS_FLUSH_AT, kFlushGap = GLQ_PS_FLUSH_GAP;
        uint32_t packed[PK];
        bool st_ok = true;
        int pv_ft = 0, pv_lt = 0, pv_cnt = 0, pv_e0 = 0, pass = 0;

        // write the held results to y: per pass, staging tile [token][feature] in shared memory, then 16 lanes
        // per 256-byte token row; bounded handshakes between the sixteen warps around the staging tile
        int pend = 0;                 // passes of the tile before that are still to be written
        auto flush_pass = [&]() {
            const int f0 = pv_ft * kTcFeat;
            const int nf = min(kTcFeat, N - f0);
            const int hcur = P::NH - pend;
            if (pass > 0) st_ok = __all_sync(0xffffffffu, st_ok && tc_wait(bar_stored, (uint32_t)((pass - 1) & 1), dead, 106));
#pragma unroll
            for (int h = 0; h < P::NH; ++h) {
                if (h == hcur) {
#pragma unroll
                    for (int i = 0; i < P::TH / 8; ++i) {
                        const uint32_t v = packed[h * (P::TH / 8) + i];
                        const uint32_t a = orow + (uint32_t)(part * (P::TH / 4) + 2 * i) * 256u;
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"((unsigned short)(v & 0xffffu)) : "memory");
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(a + 256u), "h"((unsigned short)(v >> 16)) : "memory");
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_drained);
            st_ok = __all_sync(0xffffffffu, st_ok && tc_wait(bar_drained, (uint32_t)(pass & 1), dead, 107));
            if (st_ok) {
                const int tid = threadIdx.x;
                for (int r = tid >> 4; r < P::TH; r += kTcProducers * 2) {
                    const int rr = pv_lt * TN + hcur * P::TH + r;
                    if (rr >= pv_cnt) break;
                    const int c8 = (tid & 15) * 8;
                    __half* dst = p.y + (size_t)(pv_e0 + rr) * p.ldy + f0 + c8;
                    if (p.y_vec) {
                        if (c8 < nf) *reinterpret_cast<uint4*>(dst) = lds128(obase + (uint32_t)r * 256u + (uint32_t)c8 * 2u);
                    } else {
                        for (int i = 0; i < 8 && c8 + i < nf; ++i) {
                            unsigned short hv;
                            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(hv) : "r"(obase + (uint32_t)r * 256u + (uint32_t)(c8 + i) * 2u) : "memory");
                            dst[i] = __ushort_as_half(hv);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_stored);
            ++pass;
            --pend;
        };

        for (;;) {
            const int wk = next_item(it);
            if (wk < 0) break;
            const int gt = wk / p.n_ft, ft = wk - gt * p.n_ft;
            int slot, lt, cnt, e0;
            if (!tc_find_tile<TN>(p, gt, slot, lt, cnt, e0)) break;        // the loader publishes live tiles only
            const int widx = p.slot_index ? __ldg(p.slot_index + slot) : slot;
            const glq_weight_t W = p.table ? p.table[widx] : p.w;
            const int tile16 = ft * 8 + tl;
            const bool live = tile16 < (N + 15) / 16;
            const unsigned char* blk[NM];
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                const int d = SW ? tile16 * 2 + m : tile16;
                blk[m] = reinterpret_cast<const unsigned char*>(W.codes) + ((size_t)(d >> 1) * p.nkb * 2 + (d & 1)) * 576;
            }
            constexpr int D = 4;
            uint32_t cq[D][NM][2], csz[D][NM][2];     // word `wh` of row g and of row g+8; their (scale, zero) pairs
            auto fetch = [&](int st, uint32_t (&qv)[NM][2], uint32_t (&zv)[NM][2]) {
#pragma unroll
                for (int m = 0; m < NM; ++m) {
                    const bool in = live && st < p.nkb;
                    const unsigned char* src = blk[m] + (size_t)st * 2 * 576;
                    const uint32_t* wsrc = reinterpret_cast<const uint32_t*>(src) + lane * 4 + wh;
                    qv[m][0] = in ? __ldg(wsrc) : 0u;
                    qv[m][1] = in ? __ldg(wsrc + 2) : 0u;
                    const uint2 z = in ? __ldg(reinterpret_cast<const uint2*>(src + 512) + g) : make_uint2(0, 0);
                    zv[m][0] = z.x;
                    zv[m][1] = z.y;
                }
            };
#pragma unroll
            for (int d = 0; d < D; ++d) fetch(d, cq[d], csz[d]);

            bool ok = true;
            for (int st0 = 0; st0 < nst; st0 += D) {
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const int st = st0 + d;
                    if (st < nst) {
                        ok = __all_sync(0xffffffffu, ok && tc_wait(bar_empty + 8 * s, ph ^ 1u, dead, 100));
                        tc_fence_after();
                        const uint32_t acol = ring + (uint32_t)(s * NM * 64);
                        if (ok && st < p.nkb) {
#pragma unroll
                            for (int m = 0; m < NM; ++m) {
                                // regs of repeat n: {row g: positions 4t..4t+3 of k step 4*wh + n}, {row g+8: the same}
                                uint32_t r[16];
#pragma unroll
                                for (int hrow = 0; hrow < 2; ++hrow) {
                                    const TcAffine af(csz[d][m][hrow], 1024.f);
                                    const uint32_t w = cq[d][m][hrow];
#pragma unroll
                                    for (int n = 0; n < 4; ++n)
#pragma unroll
                                        for (int e = 0; e < 2; ++e) {
                                            const uint32_t h = and_or(w >> (2 * (2 * n + e)), 0x00030003u, 0x64006400u);
                                            r[4 * n + 2 * hrow + e] = af.integral ? af.exact(h) : af.general(h);
                                        }
                                }
                                tc_st_x4(acol + (uint32_t)(m * 64 + wh * 32) + lane_base, r);
                            }
                            fetch(st + D, cq[d], csz[d]);
                        } else if (ok) {
                            // low-rank stage: SV rows in natural K order; this warp stores k steps 2*wh, 2*wh+1
                            const int sl = st - p.nkb;
#pragma unroll
                            for (int m = 0; m < NM; ++m) {
                                const int dt = SW ? tile16 * 2 + m : tile16;
                                uint32_t r[8];
#pragma unroll
                                for (int n = 0; n < 2; ++n)
#pragma unroll
                                    for (int hrow = 0; hrow < 2; ++hrow) {
                                        const int row = g + 8 * hrow;
                                        const uint2* src = reinterpret_cast<const uint2*>(
                                            reinterpret_cast<const unsigned char*>(W.sv) +
                                            ((((size_t)(dt >> 1) * p.ns + sl) * 32) + (dt & 1) * 16 + row) * 128 +
                                            (2 * wh + n) * 32 + t * 8);
                                        const uint2 v = (live && W.sv) ? __ldg(src) : make_uint2(0, 0);
                                        r[4 * n + 2 * hrow] = v.x;
                                        r[4 * n + 2 * hrow + 1] = v.y;
                                    }
                                tc_st_x2(acol + (uint32_t)(m * 64 + wh * 16) + lane_base, r);
                            }
                        }
                        tc_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_full + 8 * s);
                        if (++s == S) {
                            s = 0;
                            ph ^= 1u;
                        }
                        // the ring is full again: the tensor pipe has work while the tile before goes to memory
                        if (pend > 0 && st == kFlushAt + kFlushGap * (P::NH - pend)) flush_pass();
                    }
                }
            }
            while (pend > 0) flush_pass();     // tiles with few stages

            // ---- accumulator -> registers (epilogue arithmetic, fp16 pairs); then it is free for the next tile ----
            const bool acc_ok = __all_sync(0xffffffffu, ok && tc_wait(bar_acc, (uint32_t)(it & 1), dead, 101));
            tc_fence_after();
            {
                const int f = ft * kTcFeat + q * 32 + lane;
                const __half* bias = reinterpret_cast<const __half*>(W.bias);
                const float bv = (!SW && bias && f < N) ? __half2float(__ldg(bias + f)) : 0.f;
#pragma unroll
                for (int h = 0; h < P::NH; ++h) {
#pragma unroll
                    for (int k = 0; k < P::TH / 64; ++k) {
                        const int c0 = h * P::TH + part * (P::TH / 4) + 16 * k;
                        uint32_t vg[16], vu[16];
                        tc_ld16(trow + (uint32_t)c0, vg);
                        if (SW) tc_ld16(trow + (uint32_t)(TN + c0), vu);
                        tc_ld_wait();
                        if (!SW && !bias && !p.entry_scale) {
                            // plain product: one rounding, two values per conversion
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const __half2 h2 = __floats2half2_rn(__uint_as_float(vg[2 * j]), __uint_as_float(vg[2 * j + 1]));
                                packed[h * (P::TH / 8) + 8 * k + j] = *reinterpret_cast<const uint32_t*>(&h2);
                            }
                        } else {
                            unsigned short hv[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int rr = lt * TN + c0 + j;
                                float v = round16(__uint_as_float(vg[j]));
                                if (SW) {
                                    v = round16(silu16(v) * round16(__uint_as_float(vu[j])));
                                } else {
                                    if (bias) v = round16(v + bv);
                                    if (p.entry_scale && rr < cnt) v = round16(__half2float(__ldg(p.entry_scale + e0 + rr)) * v);
                                }
                                hv[j] = __half_as_ushort(__float2half_rn(v));
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                packed[h * (P::TH / 8) + 8 * k + j] = (uint32_t)hv[2 * j] | ((uint32_t)hv[2 * j + 1] << 16);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_free);
            pend = P::NH;
            pv_ft = ft;
            pv_lt = lt;
            pv_cnt = cnt;
            pv_e0 = e0;
            ++it;
            if (!acc_ok || !st_ok) break;
        }
        while (pend > 0 && st_ok && !__any_sync(0xffffffffu, *dead != 0)) flush_pass();
        tc_fence_before();
    } else if (warp == kTcProducers) {
        // ================= MMA issuer =================
        constexpr uint32_t idesc = tc_idesc(TN);
        int s = 0;
        uint32_t ph = 0;
        int it = 0;
        for (;;) {
            const int wk = next_item(it);
            if (wk < 0) break;
            if (lane == 0) {
                bool ok = true;
                for (int st = 0; st < nst && ok; ++st) {
                    ok = tc_wait(bar_full + 8 * s, ph, dead, 103);
                    if (ok && st == 0 && it > 0) ok = tc_wait(bar_acc_free, (uint32_t)((it - 1) & 1), dead, 104);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t acol = ring + (uint32_t)(s * NM * 64);
                    const uint32_t bbase = sbase + (uint32_t)s * C::B_BYTES;
                    if (st < p.nkb) {
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const uint64_t bd = tc_smem_desc(bbase + (uint32_t)(kk >> 2) * (TN * 128) + (uint32_t)(kk & 3) * 32u);
                            tc_mma_f16_ts(tmem, acol + 8 * kk, bd, idesc, (st | kk) != 0);
                            if (SW) tc_mma_f16_ts(tmem + TN, acol + 64 + 8 * kk, bd, idesc, (st | kk) != 0);
                        }
                    } else {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            tc_mma_f16_ts(tmem, acol + 8 * kk, tc_smem_desc(bbase + (uint32_t)kk * 32u), idesc, 1);
                            if (SW) tc_mma_f16_ts(tmem + TN, acol + 64 + 8 * kk, tc_smem_desc(bbase + TN * 128 + (uint32_t)kk * 32u), idesc, 1);
                        }
                    }
                    tc_commit(bar_empty + 8 * s);
                    if (++s == S) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (ok) tc_commit(bar_acc);
            }
            // every lane keeps the ring position of lane 0
            s = __shfl_sync(0xffffffffu, s, 0);
            ph = __shfl_sync(0xffffffffu, ph, 0);
            ++it;
        }
    } else {
        // ================= loader of the token operand =================
        int s = 0;
        uint32_t ph = 0;
        int issued = 0;
        for (int n = 0;; ++n) {
            // draw the next live work item from the grid-wide counter and publish it to the other warps
            const int qi = n % kPsQueue;
            const bool room = __all_sync(0xffffffffu, tc_wait(bar_tq_empty + 8 * qi, (uint32_t)(((n / kPsQueue) & 1) ^ 1), dead, 109));
            int wk = -1, gt = 0;
            while (room) {
                int w = 0;
                if (lane == 0) w = atomicAdd(p.tile_ctr, 1);
                w = __shfl_sync(0xffffffffu, w, 0);
                if (w >= n_work) break;
                gt = w / p.n_ft;
                int slot, lt, cnt, e0;
                if (tc_find_tile<TN>(p, gt, slot, lt, cnt, e0)) {
                    wk = w;
                    break;
                }
            }
            if (lane == 0) {
                *reinterpret_cast<volatile int*>(&s_tile[qi]) = wk;
                mbar_arrive(bar_tq_full + 8 * qi);
            }
            __syncwarp();
            if (wk < 0) break;
            if (lane == 0) {
                const unsigned char* tile = p.xp + (size_t)gt * p.tile_bytes;
                for (int st = 0; st < nst; ++st) {
                    if (!tc_wait(bar_empty + 8 * s, ph ^ 1u, dead, 105)) break;
                    const uint32_t bbase = sbase + (uint32_t)s * C::B_BYTES;
                    const unsigned char* src;
                    uint32_t bytes;
                    if (st < p.nkb) {
                        src = tile + (size_t)st * TN * 256;
                        bytes = TN * 256;
                    } else {
                        src = tile + (size_t)p.nkb * TN * 256 + (size_t)(st - p.nkb) * p.na * TN * 128;
                        bytes = (uint32_t)p.na * TN * 128;
                    }
                    mbar_expect_tx(bar_full + 8 * s, bytes);
                    bulk_g2s(bbase, src, bytes, bar_full + 8 * s);
                    ++issued;
                    if (++s == S) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
            s = __shfl_sync(0xffffffffu, s, 0);
            ph = __shfl_sync(0xffffffffu, ph, 0);
        }
        if (lane == 0 && *dead) {      // do not leave while copies are in flight
            int s2 = s;
            uint32_t ph2 = ph;
            for (int i = 0; i < S && i < issued; ++i) {
                if (--s2 < 0) {
                    s2 = S - 1;
                    ph2 ^= 1u;
                }
                const unsigned long long t0 = global_ns();
                while (!mbar_test_wait(bar_full + 8 * s2, ph2) && global_ns() - t0 < 2000000ull) __nanosleep(64);
            }
        }
        __syncwarp();
    }

    __syncthreads();
    if (warp == kTcProducers) {
        tc_fence_after();
        tc_dealloc(tmem, 512);
    }
}

}  // namespace glq
