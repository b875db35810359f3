// Grouped dequant-GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM) for
// problems with many activation rows (prefill, large decode batches).
//
//   D[feature, token] = sum_k W[feature, k] * X[token, k]   (+ sum_r SV[feature, r] * a[token, r])
//
// The weights are the M operand ("swap AB"): a CTA owns 128 output features of one problem and TN
// tokens; producer warps unpack the 2-bit codes of the pair-interleaved tiled layout to the exact
// fp16 values fp16((q - z) * s) and store them as a K-major, 128-byte-swizzled UMMA operand in shared
// memory; the token operand arrives ready-made: a pre-pass (tc_pack_b_kernel) gathers the problem's
// activation rows, orders k like the unpack does and writes swizzled tiles, so the main kernel fetches
// each k stage of it with one bulk copy.  One thread issues the MMAs; the low-rank term is folded in
// as extra k steps (A = SV rows, B = the entries' x.U rows), so the epilogue only rounds, applies
// SwiGLU / routing weight / bias and stores.
//
// k order inside every group of 16 input channels: position 2j holds channel j, position 2j+1 holds
// channel j+8 (the order in which one shift-and-mask yields two codes); both operands use it, so the
// dot products are unchanged.
//
// Every mbarrier wait is bounded (about 2 ms); a wait that runs out records error 100/101, marks the
// CTA dead, and all roles fall through to the common exit, which frees the tensor memory.
#pragma once

#include "stream_mm.cuh"

namespace glq {

constexpr int kTcFeat = 128;          // output features per CTA (UMMA M)
constexpr int kTcProducers = 16;      // producer (and epilogue) warps: 8 tiles of 16 rows x 2 row halves
constexpr int kTcThreads = (kTcProducers + 2) * 32;

struct TcParams {
    glq_weight_t w;
    const glq_weight_t* table;
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
    unsigned char* xp;        // packed token operand: [token tile][k stages | low-rank stages]
    long long tile_bytes;     // bytes of one token tile in xp
    int n_problems, max_rows, rows_stride;
    int K, rank, nkb, ns, na; // ns: 64-wide low-rank slices, na: x.U operands per entry (1, or 2 for gate|up)
    int tiles_max;
    int x_vec;                // x rows allow 8-byte loads
    int fmt;                  // GLQ_FMT_*: fixes the channel order inside a group of 16
    int min_rows;             // only problems with more rows than this are this launch's
    int ts;                   // 1: K positions of a stage in the order of the tensor-memory variant
    int N, n_ft;              // output features of every problem; 128-feature tiles (persistent kernel)
    int y_vec;                // y rows allow 16-byte bulk stores
    int x_vec16;              // x rows allow 16-byte loads
    int* tile_ctr;            // work-item counter of the persistent kernel (in the workspace, zeroed by the pre-pass)
};

// ---- token tile -> (problem slot, local tile) -----------------------------------------------------
// Problem p (slot position) with entries [off_p, off_p + cnt_p) owns the global token tiles
// [off_p / TN + p, off_p / TN + p + ceil(cnt_p / TN)): disjoint for consecutive problems, and at most
// total / TN + P + 1 tiles in all.  Warp-uniform result; every warp scans the (few) slots itself.
template <int TN>
__device__ __forceinline__ bool tc_find_tile(const TcParams& p, int gt, int& slot, int& lt, int& cnt, int& e0) {
    const int lane = threadIdx.x & 31;
    int P = p.n_problems;
    if (p.n_slots) P = min(P, __ldg(p.n_slots));
    for (int base = 0; base < P; base += 32) {
        const int pp = base + lane;
        int off = 0, c = 0;
        if (pp < P) {
            c = p.slot_count ? __ldg(p.slot_count + pp) : p.max_rows;
            off = p.slot_offset ? __ldg(p.slot_offset + pp) : pp * p.rows_stride;
        }
        const int start = off / TN + pp;
        const bool hit = pp < P && c > p.min_rows && gt >= start && gt < start + (c + TN - 1) / TN;
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (m) {
            const int src = __ffs(m) - 1;
            slot = base + src;
            lt = gt - __shfl_sync(0xffffffffu, start, src);
            cnt = __shfl_sync(0xffffffffu, c, src);
            e0 = __shfl_sync(0xffffffffu, off, src);
            return true;
        }
    }
    return false;
}

// Order of the input channels inside a group of 16, per format (the order in which the format's
// unpack yields its values); the pre-pass stores the token operand in the same order.
__host__ __device__ __forceinline__ int tc_channel_of(int fmt, int pos) {
    switch (fmt) {
        case GLQ_FMT_Q2: return (pos >> 1) + 8 * (pos & 1);                              // (j, j+8)
        case GLQ_FMT_Q4: return (pos & 8) + ((pos & 7) >> 1) + 4 * (pos & 1);             // (j, j+4) per 8
        case GLQ_FMT_T2: return ((pos & 7) >> 1) * 4 + (pos & 1) * 2 + (pos >> 3);        // (0,2)(4,6)..(1,3)(5,7)..
        default: return 2 * (pos >> 2) + (pos & 1) + 8 * ((pos >> 1) & 1);                // F16 fragment order
    }
}

// K position -> channel of the tensor-memory variant (see tc_ts_kernel)
__host__ __device__ __forceinline__ int tc_ts_channel_of(int P) {
    const int w = P >> 6, n = (P >> 4) & 3, t = (P >> 2) & 3, i = P & 3;
    return 32 * t + 16 * w + 2 * n + (i >> 1) + 8 * (i & 1);
}

// ---- pre-pass: token operand in UMMA layout ---------------------------------------------------------
// Tile layout in xp (TN rows): per k stage (128 input channels) two atoms [TN][128 B], then per
// low-rank slice `na` atoms [TN][128 B].  Inside an atom row r keeps its 16-byte chunk c at chunk
// position c ^ (r & 7) (the 128-byte swizzle).  grid = (tiles_max, nkb + ns), 256 threads.
template <int TN>
__global__ void __launch_bounds__(256) tc_pack_b_kernel(const TcParams p) {
    if (p.tile_ctr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *p.tile_ctr = 0;
    int slot, lt, cnt, e0;
    if (!tc_find_tile<TN>(p, blockIdx.x, slot, lt, cnt, e0)) return;
    unsigned char* tile = p.xp + (size_t)blockIdx.x * p.tile_bytes;
    const int st = blockIdx.y;
    if (st < p.nkb && p.ts && p.x_vec16 && st * 128 + 128 <= p.K) {
        // tensor-memory order, whole stage inside K: a thread takes 16 consecutive channels (two 16-byte
        // loads) of one row, channels 32*t + 16*w + (0..15), and writes the four 8-byte pieces
        // {c, c+8, c+1, c+9}, c = 2n, that k step n of atom w holds for lane t
        unsigned char* sdst = tile + (size_t)st * TN * 256;
#pragma unroll 2
        for (int idx = threadIdx.x; idx < TN * 8; idx += 256) {
            const int r = idx >> 3, q8 = idx & 7, t = q8 >> 1, w = q8 & 1;
            const int rr = lt * TN + r;
            uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
            if (rr < cnt) {
                const long long row = p.entry_row ? __ldg(p.entry_row + e0 + rr) : (long long)(e0 + rr);
                const uint4* src = reinterpret_cast<const uint4*>(p.x + row * p.ldx + st * 128 + 32 * t + 16 * w);
                lo = __ldg(src);
                hi = __ldg(src + 1);
            }
            const uint32_t a[4] = {lo.x, lo.y, lo.z, lo.w}, b[4] = {hi.x, hi.y, hi.z, hi.w};
            unsigned char* rdst = sdst + (size_t)w * (TN * 128) + (size_t)r * 128 + (t & 1) * 8;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const int c = (2 * n + (t >> 1)) ^ (r & 7);
                *reinterpret_cast<uint2*>(rdst + c * 16) =
                    make_uint2(__byte_perm(a[n], b[n], 0x5410), __byte_perm(a[n], b[n], 0x7632));
            }
        }
    } else if (st < p.nkb) {
        uint4* dst = reinterpret_cast<uint4*>(tile + (size_t)st * TN * 256);
        for (int ci = threadIdx.x; ci < TN * 16; ci += 256) {
            const int atom = ci / (TN * 8), r = (ci >> 3) % TN, cpos = ci & 7;
            const int c = cpos ^ (r & 7);
            const int k0 = st * 128 + atom * 64 + (c >> 1) * 16, h = c & 1;
            const int rr = lt * TN + r;
            __align__(16) __half v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __float2half(0.f);
            if (rr < cnt) {
                const long long row = p.entry_row ? __ldg(p.entry_row + e0 + rr) : (long long)(e0 + rr);
                const __half* src = p.x + row * p.ldx;
                const int ka = k0 + 4 * h, kb = k0 + 8 + 4 * h;     // channels j and j+8, j = 4h..4h+3
                if (p.ts) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int k = st * 128 + tc_ts_channel_of(atom * 64 + c * 8 + i);
                        if (k < p.K) v[i] = __ldg(src + k);
                    }
                } else if (p.fmt != GLQ_FMT_Q2) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int k = k0 + tc_channel_of(p.fmt, 8 * h + i);
                        if (k < p.K) v[i] = __ldg(src + k);
                    }
                } else if (p.x_vec && kb + 4 <= p.K) {
                    __align__(8) __half lo[4], hi[4];
                    *reinterpret_cast<uint2*>(lo) = __ldg(reinterpret_cast<const uint2*>(src + ka));
                    *reinterpret_cast<uint2*>(hi) = __ldg(reinterpret_cast<const uint2*>(src + kb));
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        v[2 * i] = lo[i];
                        v[2 * i + 1] = hi[i];
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (ka + i < p.K) v[2 * i] = __ldg(src + ka + i);
                        if (kb + i < p.K) v[2 * i + 1] = __ldg(src + kb + i);
                    }
                }
            }
            dst[ci] = *reinterpret_cast<const uint4*>(v);
        }
    } else {
        const int sl = st - p.nkb;
        uint4* dst = reinterpret_cast<uint4*>(tile + (size_t)p.nkb * TN * 256 + (size_t)sl * p.na * TN * 128);
        for (int ci = threadIdx.x; ci < p.na * TN * 8; ci += 256) {
            const int ai = ci / (TN * 8), r = (ci >> 3) % TN, cpos = ci & 7;
            const int c = cpos ^ (r & 7);
            const int col = sl * 64 + c * 8;
            const int rr = lt * TN + r;
            __align__(16) __half v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __float2half(0.f);
            const __half* a = p.a[ai];
            if (rr < cnt && a != nullptr) {
                const __half* src = a + (long long)(e0 + rr) * p.lda + col;
                if (col + 8 <= p.rank) {
                    *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(src));   // lda % 8 == 0, a 16-byte aligned
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (col + i < p.rank) v[i] = __ldg(src + i);
                }
            }
            dst[ci] = *reinterpret_cast<const uint4*>(v);
        }
    }
}

// ---- tcgen05 primitives -----------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp gets lane (base lane + i)
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// K-major operand, 128-byte swizzle: rows 128 B apart, 8-row groups 1024 B apart, version 1
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// kind::f16: D fp32, A and B fp16, both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t tc_idesc(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTcFeat >> 4) << 24);
}

// bounded wait shared by all roles; `dead` lives in shared memory so that every role sees it
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* dead, int code) {
    if (*dead) return false;
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    // try_wait suspends the thread in hardware for a bounded time, so a waiting warp takes no issue slots
    // from the working ones; the loop only re-arms it and enforces the overall limit
    while (!mbar_try_wait(bar, parity)) {
        if (*dead) return false;
        if (global_ns() - t0 > 2000000ull) {
            glq_ok(false, code, bar, parity);
            *dead = 1;
            return false;
        }
    }
    return true;
}

template <int TN, bool SW> struct TcCfg {
    static constexpr int A_BYTES = (SW ? 2 : 1) * kTcFeat * 256;   // 128 rows x 128 channels fp16 (x2: gate, up)
    static constexpr int B_BYTES = TN * 256;
    static constexpr int STAGE = A_BYTES + B_BYTES;
    static constexpr int S = (200 * 1024) / STAGE >= 4 ? 4 : (200 * 1024) / STAGE;
    static constexpr int COLS = SW ? 2 * TN : TN;                 // fp32 accumulator columns in TMEM
    static constexpr size_t SMEM = (size_t)S * STAGE + 1024;
};

// (1024 + code) or (64 + code) pairs -> fp16(fp16(q - z) * s).  When offset + z is exact in fp16 (what
// integer zero points, the quantizer's output, always are) one subtraction of it from offset + code
// rounds once, to fp16(q - z), as the two-step form does; any other zero point takes
// (offset + code - offset) - z.
struct TcAffine {
    __half2 s2, z2, zc, koff;
    bool integral;
    __device__ __forceinline__ TcAffine(uint32_t sz, float off) {
        s2 = __half2half2(__ushort_as_half((unsigned short)(sz & 0xffffu)));
        z2 = __half2half2(__ushort_as_half((unsigned short)(sz >> 16)));
        koff = __float2half2_rn(off);
        zc = __hadd2(z2, koff);
        integral = __hbeq2(__hsub2(zc, koff), z2);      // offset + z kept every bit of z
    }
    __device__ __forceinline__ uint32_t exact(uint32_t h) const {
        const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&h), zc), s2);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    __device__ __forceinline__ uint32_t general(uint32_t h) const {
        const __half2 v = __hmul2(__hsub2(__hsub2(*reinterpret_cast<const __half2*>(&h), koff), z2), s2);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
};

template <int FMT, int TN, bool SW>
__global__ void __launch_bounds__(kTcThreads, 1) tc_kernel(const TcParams p) {
    using C = TcCfg<TN, SW>;
    constexpr int S = C::S;
    constexpr bool AFFINE = FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_Q4;
    static_assert(!(SW && FMT == GLQ_FMT_F16), "dense weights have no fused gate|up form");
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * S + 1];
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;

    int slot, lt, cnt, e0;
    if (!tc_find_tile<TN>(p, blockIdx.y, slot, lt, cnt, e0)) return;    // uniform: a padding tile
    const int widx = p.slot_index ? __ldg(p.slot_index + slot) : slot;
    const glq_weight_t W = p.table ? p.table[widx] : p.w;
    const int N = W.N;
    const int ft = blockIdx.x;
    if (ft * kTcFeat >= N) return;
    const bool has_lr = FMT != GLQ_FMT_F16 && p.rank > 0 && W.sv != nullptr && p.a[0] != nullptr;
    const int nst = p.nkb + (has_lr ? p.ns : 0);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sraw = smem_u32(tc_smem_raw);
    const uint32_t sbase = (sraw + 1023u) & ~1023u;
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * S, bar_acc = bar_full + 16 * S;
    volatile int* dead = &s_dead;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, kTcProducers + 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        s_dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTcProducers) tc_alloc(smem_u32(&s_tmem), C::COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    if (warp < kTcProducers) {
        // ================= producers: the weight operand =================
        // warp = (row half, 16-row tile): lane (g, t) owns row 8*hrow + g of tile `warp & 7`
        const int g = lane >> 2, t = lane & 3;
        const int hrow = warp >> 3;
        const int tile16 = ft * 8 + (warp & 7);                 // 16-row tile of the matrix (of gate and of up)
        constexpr int NM = SW ? 2 : 1;
        const int ntiles16 = (N + 15) / 16;
        const bool live = tile16 < ntiles16;                    // tiles past the matrix contribute zero rows
        // blocks of the tiled layouts per 128-channel stage, 32-bit words per lane, row and block
        constexpr int BPS = (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_T2) ? 1 : 2;
        constexpr int WPB = FMT == GLQ_FMT_F16 ? 8 : 2;
        constexpr int BB = FMT == GLQ_FMT_T2 ? 512 : 576;
        constexpr int REGS = NM * BPS * (WPB + (AFFINE ? 1 : 0));
        constexpr int D = REGS <= 6 ? 4 : (REGS <= 16 ? 2 : 1);    // register prefetch depth (stages)
        const int nblk = (FMT == GLQ_FMT_F16 || FMT == GLQ_FMT_Q4) ? (p.K + 63) / 64 : p.nkb;
        const unsigned char* blk[NM];
#pragma unroll
        for (int m = 0; m < NM; ++m) {
            if constexpr (FMT == GLQ_FMT_F16) {
                blk[m] = reinterpret_cast<const unsigned char*>(W.codes) + (size_t)tile16 * nblk * 2048;
            } else {
                // fused gate|up: destination tile d = 2 * tile16 + matrix; plain: d = tile16; pair d/2, slot d%2
                const int d = SW ? tile16 * 2 + m : tile16;
                blk[m] = reinterpret_cast<const unsigned char*>(W.codes) + ((size_t)(d >> 1) * nblk * 2 + (d & 1)) * BB;
            }
        }
        uint32_t TL[NM], TH[NM];
        if constexpr (FMT == GLQ_FMT_T2) {
#pragma unroll
            for (int m = 0; m < NM; ++m) make_t2_tables(W.centroids + 4 * m, TL[m], TH[m]);
        }
        uint32_t cq[D][NM][BPS][WPB];
        uint32_t csz[D][NM][BPS];
        auto fetch = [&](int st, uint32_t (&q)[NM][BPS][WPB], uint32_t (&z)[NM][BPS]) {
#pragma unroll
            for (int m = 0; m < NM; ++m)
#pragma unroll
                for (int b = 0; b < BPS; ++b) {
                    const int kb = st * BPS + b;
                    const bool in = live && st < p.nkb && kb < nblk;
                    if constexpr (FMT == GLQ_FMT_F16) {
                        // fragment (ks, lane): words 0,2 = row g (channels 2t,2t+1 | 2t+8,2t+9), words 1,3 = row g+8
                        const uint32_t* src = reinterpret_cast<const uint32_t*>(blk[m] + (size_t)kb * 2048) + lane * 4 + hrow;
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            q[m][b][2 * ks] = in ? __ldg(src + 128 * ks) : 0u;
                            q[m][b][2 * ks + 1] = in ? __ldg(src + 128 * ks + 2) : 0u;
                        }
                    } else {
                        // words 0,1 of the lane's 16 bytes = row g, words 2,3 = row g + 8
                        const unsigned char* src = blk[m] + (size_t)kb * 2 * BB;
                        const uint2 v = in ? __ldg(reinterpret_cast<const uint2*>(src) + 2 * lane + hrow) : make_uint2(0, 0);
                        q[m][b][0] = v.x;
                        q[m][b][1] = v.y;
                        if constexpr (AFFINE) z[m][b] = in ? __ldg(reinterpret_cast<const uint32_t*>(src + 512) + 2 * g + hrow) : 0u;
                    }
                }
        };
#pragma unroll
        for (int d = 0; d < D; ++d) fetch(d, cq[d], csz[d]);

        int s = 0;
        uint32_t ph = 0;
        // this lane's row of the A tile; its swizzle key (row & 7) is g
        const uint32_t row_off = (uint32_t)((warp & 7) * 16 + hrow * 8 + g) * 128u;
        for (int st0 = 0; st0 < nst; st0 += D) {
#pragma unroll
            for (int d = 0; d < D; ++d) {
                const int st = st0 + d;
                if (st < nst) {
                    const bool ok = tc_wait(bar_empty + 8 * s, ph ^ 1u, dead, 100);
                    const uint32_t abase = sbase + (uint32_t)s * C::STAGE;
                    if (ok && st < p.nkb) {
#pragma unroll
                        for (int m = 0; m < NM; ++m) {
                            const uint32_t mbase = abase + (uint32_t)m * (kTcFeat * 256) + row_off;
                            if constexpr (FMT == GLQ_FMT_Q2 || FMT == GLQ_FMT_T2) {
                                // lane t holds channels 32t .. 32t+31 of the stage: atom t/2, chunks 4(t%2) .. +3.
                                // Lanes of atom 1 take their two words in the other order, so that the lanes
                                // of one store instruction that differ only in the atom hit different banks.
                                const bool flip = (t >> 1) != 0;
                                const uint32_t wa = flip ? cq[d][m][0][1] : cq[d][m][0][0];
                                const uint32_t wb = flip ? cq[d][m][0][0] : cq[d][m][0][1];
                                uint32_t o[16];
                                if constexpr (FMT == GLQ_FMT_Q2) {
                                    const TcAffine af(csz[d][m][0], 1024.f);
                                    if (af.integral) {
#pragma unroll
                                        for (int j = 0; j < 8; ++j) {
                                            o[j] = af.exact(and_or(wa >> (2 * j), 0x00030003u, 0x64006400u));
                                            o[8 + j] = af.exact(and_or(wb >> (2 * j), 0x00030003u, 0x64006400u));
                                        }
                                    } else {
#pragma unroll
                                        for (int j = 0; j < 8; ++j) {
                                            o[j] = af.general(and_or(wa >> (2 * j), 0x00030003u, 0x64006400u));
                                            o[8 + j] = af.general(and_or(wb >> (2 * j), 0x00030003u, 0x64006400u));
                                        }
                                    }
                                } else {
                                    uint32_t h0[8], h1[8];
                                    unpack_t2(wa, TL[m], TH[m], h0);
                                    unpack_t2(wb, TL[m], TH[m], h1);
#pragma unroll
                                    for (int j = 0; j < 8; ++j) {
                                        o[j] = h0[j];
                                        o[8 + j] = h1[j];
                                    }
                                }
                                const uint32_t base = mbase + (uint32_t)(t >> 1) * (kTcFeat * 128);
                                const uint32_t fx = flip ? 2u : 0u;
#pragma unroll
                                for (int c = 0; c < 4; ++c) {
                                    const uint32_t chunk = ((uint32_t)(4 * (t & 1) + c) ^ fx) ^ (uint32_t)g;
                                    sts128(base + chunk * 16u, o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
                                }
                            } else if constexpr (FMT == GLQ_FMT_Q4) {
                                // block b = atom b; lane t holds channels 16t .. 16t+15 of it: chunks 2t, 2t+1
#pragma unroll
                                for (int b = 0; b < 2; ++b) {
                                    const TcAffine af(csz[d][m][b], kQ4Offset);
                                    uint32_t h0[4], h1[4];
                                    unpack_q4(cq[d][m][b][0], h0);
                                    unpack_q4(cq[d][m][b][1], h1);
                                    const uint32_t base = mbase + (uint32_t)b * (kTcFeat * 128);
                                    if (af.integral) {
                                        sts128(base + (uint32_t)((2 * t) ^ g) * 16u, af.exact(h0[0]), af.exact(h0[1]), af.exact(h0[2]),
                                               af.exact(h0[3]));
                                        sts128(base + (uint32_t)((2 * t + 1) ^ g) * 16u, af.exact(h1[0]), af.exact(h1[1]),
                                               af.exact(h1[2]), af.exact(h1[3]));
                                    } else {
                                        sts128(base + (uint32_t)((2 * t) ^ g) * 16u, af.general(h0[0]), af.general(h0[1]),
                                               af.general(h0[2]), af.general(h0[3]));
                                        sts128(base + (uint32_t)((2 * t + 1) ^ g) * 16u, af.general(h1[0]), af.general(h1[1]),
                                               af.general(h1[2]), af.general(h1[3]));
                                    }
                                }
                            } else {
                                // dense fp16 fragments: block b = atom b; (ks, lane) holds channels
                                // 16ks + {2t, 2t+1, 2t+8, 2t+9} of its row: 8 bytes at chunk 2ks + t/2, half t%2
#pragma unroll
                                for (int b = 0; b < 2; ++b)
#pragma unroll
                                    for (int ks = 0; ks < 4; ++ks) {
                                        const uint32_t a = mbase + (uint32_t)b * (kTcFeat * 128) +
                                                           (uint32_t)((2 * ks + (t >> 1)) ^ g) * 16u + (uint32_t)(t & 1) * 8u;
                                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a), "r"(cq[d][m][b][2 * ks]),
                                                     "r"(cq[d][m][b][2 * ks + 1])
                                                     : "memory");
                                    }
                            }
                        }
                        fetch(st + D, cq[d], csz[d]);
                    } else if (ok) {
                        // low-rank stage: rows of the packed SV slice -> atom 0 of the A buffer;
                        // four lanes per row, two 16-byte chunks each
                        const int sl = st - p.nkb;
#pragma unroll
                        for (int m = 0; m < NM; ++m) {
                            const int dt = SW ? tile16 * 2 + m : tile16;
                            const int r = hrow * 8 + g;                   // row of the tile
                            const uint4* src = reinterpret_cast<const uint4*>(
                                reinterpret_cast<const unsigned char*>(W.sv) +
                                ((((size_t)(dt >> 1) * p.ns + sl) * 32) + (dt & 1) * 16 + r) * 128 + t * 32);
                            const uint32_t base = abase + (uint32_t)m * (kTcFeat * 256) + row_off;
                            // codebook format: the accumulator is scaled by the row norm in the epilogue,
                            // so the low-rank rows go in divided by it
                            float inv = 1.f;
                            if constexpr (FMT == GLQ_FMT_T2) {
                                if (live) {
                                    const float nv = __ldg(W.norms + (size_t)dt * 16 + r);
                                    inv = nv != 0.f ? 1.f / nv : 0.f;
                                }
                            }
#pragma unroll
                            for (int c = 0; c < 2; ++c) {
                                uint4 v = make_uint4(0, 0, 0, 0);
                                if (live) v = __ldg(src + c);
                                if constexpr (FMT == GLQ_FMT_T2) {
                                    __half2* hp = reinterpret_cast<__half2*>(&v);
#pragma unroll
                                    for (int i = 0; i < 4; ++i) {
                                        const float2 f2 = __half22float2(hp[i]);
                                        hp[i] = __floats2half2_rn(f2.x * inv, f2.y * inv);
                                    }
                                }
                                const uint32_t chunk = (uint32_t)((2 * t + c) ^ g);
                                sts128(base + chunk * 16u, v.x, v.y, v.z, v.w);
                            }
                        }
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full + 8 * s);
                    if (++s == S) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }

        // ================= epilogue: TMEM -> registers -> global =================
        const bool acc_ok = tc_wait(bar_acc, 0, dead, 101);
        tc_fence_after();
        const int q = warp & 3, part = warp >> 2;      // TMEM lane quarter, quarter of the token columns
        const int f = ft * kTcFeat + q * 32 + lane;
        const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16);
        const __half* bias = reinterpret_cast<const __half*>(W.bias);
        const float bv = (!SW && bias && f < N) ? __half2float(__ldg(bias + f)) : 0.f;
        float nrm_g = 1.f, nrm_u = 1.f;     // codebook format: per-row norms, in tile order
        if constexpr (FMT == GLQ_FMT_T2) {
            if (f < N) {
                const int t16 = f >> 4, r16 = f & 15;
                nrm_g = __ldg(W.norms + (size_t)(SW ? 2 * t16 : t16) * 16 + r16);
                if (SW) nrm_u = __ldg(W.norms + (size_t)(2 * t16 + 1) * 16 + r16);
            }
        }
        for (int c0 = part * (TN / 4); c0 < (part + 1) * (TN / 4); c0 += 16) {
            uint32_t vg[16], vu[16];
            tc_ld16(trow + (uint32_t)c0, vg);
            if (SW) tc_ld16(trow + (uint32_t)(TN + c0), vu);
            tc_ld_wait();
            if (acc_ok && f < N) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int rr = lt * TN + c0 + j;
                    if (rr < cnt) {
                        float v = round16(__uint_as_float(vg[j]) * nrm_g);
                        if (SW) {
                            v = round16(silu16(v) * round16(__uint_as_float(vu[j]) * nrm_u));
                        } else {
                            if (bias) v = round16(v + bv);
                            if (p.entry_scale) v = round16(__half2float(__ldg(p.entry_scale + e0 + rr)) * v);
                        }
                        p.y[(size_t)(e0 + rr) * p.ldy + f] = __float2half_rn(v);
                    }
                }
            }
        }
        tc_fence_before();
    } else if (warp == kTcProducers) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t idesc = tc_idesc(TN);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int st = 0; st < nst && ok; ++st) {
                ok = tc_wait(bar_full + 8 * s, ph, dead, 100);
                if (!ok) break;
                tc_fence_after();
                const uint32_t abase = sbase + (uint32_t)s * C::STAGE, bbase = abase + C::A_BYTES;
                if (st < p.nkb) {
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint32_t ao = (uint32_t)(kk >> 2) * (kTcFeat * 128) + (uint32_t)(kk & 3) * 32u;
                        const uint32_t bo = (uint32_t)(kk >> 2) * (TN * 128) + (uint32_t)(kk & 3) * 32u;
                        const uint64_t bd = tc_smem_desc(bbase + bo);
                        tc_mma_f16(tmem, tc_smem_desc(abase + ao), bd, idesc, (st | kk) != 0);
                        if (SW) tc_mma_f16(tmem + TN, tc_smem_desc(abase + kTcFeat * 256 + ao), bd, idesc, (st | kk) != 0);
                    }
                } else {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint32_t o = (uint32_t)kk * 32u;
                        tc_mma_f16(tmem, tc_smem_desc(abase + o), tc_smem_desc(bbase + o), idesc, 1);
                        if (SW)
                            tc_mma_f16(tmem + TN, tc_smem_desc(abase + kTcFeat * 256 + o), tc_smem_desc(bbase + TN * 128 + o),
                                       idesc, 1);
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
        __syncwarp();
    } else {
        // ================= loader of the token operand =================
        if (lane == 0) {
            const unsigned char* tile = p.xp + (size_t)blockIdx.y * p.tile_bytes;
            int s = 0;
            uint32_t ph = 0;
            int issued = 0;
            for (int st = 0; st < nst; ++st) {
                if (!tc_wait(bar_empty + 8 * s, ph ^ 1u, dead, 100)) break;
                const uint32_t bbase = sbase + (uint32_t)s * C::STAGE + C::A_BYTES;
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
            // a CTA that gave up must not leave while its copies are in flight: wait (bounded) for the
            // barriers of the last copies issued
            if (*dead) {
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
        }
        __syncwarp();
    }

    __syncthreads();
    if (warp == kTcProducers) {
        tc_fence_after();
        tc_dealloc(tmem, C::COLS);
    }
}

// =====================================================================================================
// Variant with the weight operand in tensor memory (2-bit affine codes).
//
// An SS-operand MMA reads both operands from shared memory (8 KB per 128x128x16 instruction, the whole
// 128 B/clk port) while the producers store the unpacked weights and the bulk copy writes the token
// operand through the same port.  Here the producers write the unpacked fp16 values straight into
// tensor memory (tcgen05.st, 16 lanes x 256 bit shape, which matches the (g, t) ownership of the code
// tiles: lane (g, t) holds rows g and g+8 and four consecutive K positions of every 16) and the MMA
// takes A from there (tcgen05.mma with a TMEM A operand); only the token operand uses shared memory.
//
// Tensor memory (512 columns): accumulators first (TN columns, twice for gate|up), then a ring of S
// stages of 64 columns (128 K positions x fp16) per matrix.
//
// K positions of a 128-channel stage: position P = 64*w + 16*n + 4*t + i (w: word of the lane's 32
// channels, n: repeat of the store = k step inside the word's half, t: lane mod 4, i: 0..3) holds channel
// 32*t + 16*w + 2*n + (i >> 1) + 8*(i & 1); the pre-pass lays the token operand out the same way.
// =====================================================================================================
__device__ __forceinline__ void tc_st_x4(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tc_st_x2(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D (TMEM) += A (TMEM, 128 lanes x 8 columns = 16 fp16 per row) * B (shared memory descriptor)
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}

template <int TN, bool SW> struct TcTsCfg {
    static constexpr int NM = SW ? 2 : 1;
    static constexpr int ACC = NM * TN;                       // accumulator columns
    static constexpr int S = SW ? 2 : (TN > 128 ? 3 : 4);     // ring stages: tensor memory and shared memory both fit
    static constexpr int B_BYTES = TN * 256;
    static constexpr size_t SMEM = (size_t)S * B_BYTES + 1024;
    static_assert(ACC + S * NM * 64 <= 512, "tensor memory holds 512 columns");
};

template <int TN, bool SW>
__global__ void __launch_bounds__(kTcThreads, 1) tc_ts_kernel(const TcParams p) {
    using C = TcTsCfg<TN, SW>;
    constexpr int S = C::S, NM = C::NM;
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * S + 1];
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;

    int slot, lt, cnt, e0;
    if (!tc_find_tile<TN>(p, blockIdx.y, slot, lt, cnt, e0)) return;    // uniform: a padding tile
    const int widx = p.slot_index ? __ldg(p.slot_index + slot) : slot;
    const glq_weight_t W = p.table ? p.table[widx] : p.w;
    const int N = W.N;
    const int ft = blockIdx.x;
    if (ft * kTcFeat >= N) return;
    const bool has_lr = p.rank > 0 && W.sv != nullptr && p.a[0] != nullptr;
    const int nst = p.nkb + (has_lr ? p.ns : 0);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sbase = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * S, bar_acc = bar_full + 16 * S;
    volatile int* dead = &s_dead;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, kTcProducers + 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        s_dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTcProducers) tc_alloc(smem_u32(&s_tmem), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t ring = tmem + C::ACC;      // first column of the weight ring

    if (warp < kTcProducers) {
        // ================= producers: unpack into tensor memory =================
        // warp = (lane quarter q, sub): tiles 2q and 2q+1 of the CTA's eight 16-row tiles live in TMEM lanes
        // 32q .. 32q+31, the only ones this warp may touch; sub picks the tile and the word (K half)
        const int g = lane >> 2, t = lane & 3;
        const int q = warp & 3, sub = warp >> 2;
        const int tl = 2 * q + (sub & 1), wh = sub >> 1;
        const int tile16 = ft * 8 + tl;
        const bool live = tile16 < (N + 15) / 16;
        const uint32_t lane_base = (uint32_t)(16 * tl) << 16;
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

        int s = 0;
        uint32_t ph = 0;
        for (int st0 = 0; st0 < nst; st0 += D) {
#pragma unroll
            for (int d = 0; d < D; ++d) {
                const int st = st0 + d;
                if (st < nst) {
                    const bool ok = tc_wait(bar_empty + 8 * s, ph ^ 1u, dead, 100);
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
                                    const uint2 v = live ? __ldg(src) : make_uint2(0, 0);
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
                }
            }
        }

        // ================= epilogue: TMEM -> registers -> global =================
        const bool acc_ok = tc_wait(bar_acc, 0, dead, 101);
        tc_fence_after();
        const int part = warp >> 2;                                // quarter of the token columns
        const int f = ft * kTcFeat + q * 32 + lane;
        const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16);
        const __half* bias = reinterpret_cast<const __half*>(W.bias);
        const float bv = (!SW && bias && f < N) ? __half2float(__ldg(bias + f)) : 0.f;
        for (int c0 = part * (TN / 4); c0 < (part + 1) * (TN / 4); c0 += 16) {
            uint32_t vg[16], vu[16];
            tc_ld16(trow + (uint32_t)c0, vg);
            if (SW) tc_ld16(trow + (uint32_t)(TN + c0), vu);
            tc_ld_wait();
            if (acc_ok && f < N) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int rr = lt * TN + c0 + j;
                    if (rr < cnt) {
                        float v = round16(__uint_as_float(vg[j]));
                        if (SW) {
                            v = round16(silu16(v) * round16(__uint_as_float(vu[j])));
                        } else {
                            if (bias) v = round16(v + bv);
                            if (p.entry_scale) v = round16(__half2float(__ldg(p.entry_scale + e0 + rr)) * v);
                        }
                        p.y[(size_t)(e0 + rr) * p.ldy + f] = __float2half_rn(v);
                    }
                }
            }
        }
        tc_fence_before();
    } else if (warp == kTcProducers) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t idesc = tc_idesc(TN);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int st = 0; st < nst && ok; ++st) {
                ok = tc_wait(bar_full + 8 * s, ph, dead, 100);
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
        __syncwarp();
    } else {
        // ================= loader of the token operand =================
        if (lane == 0) {
            const unsigned char* tile = p.xp + (size_t)blockIdx.y * p.tile_bytes;
            int s = 0;
            uint32_t ph = 0;
            int issued = 0;
            for (int st = 0; st < nst; ++st) {
                if (!tc_wait(bar_empty + 8 * s, ph ^ 1u, dead, 100)) break;
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
            if (*dead) {      // do not leave while copies are in flight
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
