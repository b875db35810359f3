// One persistent kernel for the MoE block of a decode step (1..4 tokens, 2/4-bit integer codes).
//
// A decode token moves ~28 MB through a block in ~4 us of HBM time, but as ten dependent launches
// (router -> plan -> x.U -> gate|up -> h.U -> down -> combine, plus the shared expert's branch) the
// block took ~47 us: every launch pays its drain, the next launch's start and a cold pipeline.  Here the
// whole block up to the per-entry down outputs is ONE cooperative launch of one CTA (16 warps) per SM.
// Every CTA walks the same fixed sequence of steps; the steps of different CTAs meet through arrival
// counters in global memory (release: stores, fence, atomic add; acquire: bounded polling load), in an
// order in which a wait only ever depends on steps that come earlier in every CTA's sequence, so with
// all CTAs resident (cooperative launch) nothing can wait for itself:
//
//   S1  dense row tasks: router logits (+ shared gate logit, + the shared expert's x.U rows)        -> R
//   S0  stage x of the n tokens as int8 digit fragments (shared by both gate|up products)
//   S2  shared expert gate|up, streamed; epilogue (low-rank term, SwiGLU) needs R                   -> HS
//   S3  routing plan, computed by every CTA for itself from the logits (needs R)
//   S4  dense row tasks: x.U of the routed experts' gate and up clusters                            -> A[slot]
//   S5  routed gate|up, streamed; epilogue needs A[slot]                                            -> H[slot]
//   S6  dense row tasks: hs.U of the shared down projection (needs HS)                              -> BS
//   S7  shared down, streamed from hs (needs HS); epilogue needs BS                                 -> Y
//   S8  dense row tasks: h.U of the routed down clusters (needs H[slot])                            -> B[slot]
//   S9  routed down, streamed from h (needs H[slot]); epilogue needs B[slot], scales by the routing
//       weight                                                                                       -> Y
//   S10 (one device, no exchange) combine: CTA t sums token t's entries and the shared expert's row in the
//       reference's order, optionally adds the residual and applies the next RMS norm (needs Y)
//   end every CTA counts itself done; the last one clears all counters for the next call.
//
// The streamed products are the integer path of stream_mm.cuh (s8 tensor-core op on 16-bit block fixed
// point activations, exact integer dot products, scale / zero point per k block in fp32): a warp item is
// (tile pair, k split); the k splits of a pair are adjacent warps of one CTA, reduced through shared
// memory in a fixed order.  Every warp owns a ring of shared-memory stages filled by bulk asynchronous
// copies it issues itself, following its own item sequence ACROSS the steps: the codes of the routed
// experts are requested the moment the plan exists, the codes of the down projections while gate|up still
// computes, so the HBM latency of each product hides behind the step before it.
//
// Every wait (mbarrier, counter) is bounded by the global timer; a wait that runs out records an error
// word (glq_debug_error) and the CTA stops waiting, so the kernel always ends and the last CTA still
// clears the counters.  No cluster launch, no multicast.
#pragma once

#include "stream_mm.cuh"

namespace glq {

constexpr int kFW = 16;            // warps per CTA
constexpr int kFSW = 12;           // of them stream the quantized products; the other four run the dense row tasks,
                                   // the routing and the plan
constexpr int kFT = kFW * 32;      // threads per CTA
constexpr int kFRows = 4;          // activation rows (tokens, or entries of a slot) a product covers
constexpr int kFMaxEntries = 64;   // n_tokens * top_k
constexpr int kFMaxStages = 4;

// arrival counters (ints in global memory, zero between calls)
enum { FL_R = 0, FL_HS = 1, FL_BS = 2, FL_Y = 3, FL_DONE = 4, FL_A = 8, FL_H = FL_A + kFMaxEntries,
       FL_B = FL_H + kFMaxEntries, FL_COUNT = FL_B + kFMaxEntries };

// one streamed product
struct FusedPhase {
    const glq_weight_t* table;   // routed: the experts' descriptors; shared: nullptr
    glq_weight_t w;              // shared: the descriptor
    int N, K, nkb, npairs, swiglu;
    int sk, sk_log2, kb_per_split;
    int ppi;                     // tile pairs per iteration (16 warps / sk)
    int ipp;                     // iterations per problem
    int cta_base;                // iteration i runs on CTA (cta_base + i) mod grid
    int rank, ns;                // low-rank width of this product (0: none), 64-column slices of SV
    int live;                    // 0: the product does not exist (no shared expert)
};

struct FusedParams {
    int n, H, I, Is, E, k, R, renorm, ep_rank, ep_world;
    int ldl;                 // leading dimension of the logits buffer (dense rows)
    int dense_rows;          // rows of router_rm (router rows, padding, the shared expert's U^T rows)
    int sh_a_row;            // first row of the shared expert's U_gate^T in router_rm (U_up^T follows), or 0
    const __half* x;         // (n, H)
    const __half* router_rm; // (dense_rows, H) row-major
    const void* const* ut_rm_gate_up;   // [2E] row-major U^T (R x H): gate of expert e at e, up at E + e
    const void* const* ut_rm_down;      // [E]  row-major U^T (R x I)
    const __half* sh_ut_rm_down;        // row-major U^T (R x Is) of the shared down projection, or nullptr
    // global buffers
    __half* logits;          // (n, ldl)
    int* sel; __half* wts; int* active; int* n_active; int* slot_count; int* slot_offset; int* entry_row;
    __half* entry_scale; int* tok_entries;
    __half* a_gate; __half* a_up;   // (entries, R)
    __half* h;               // (entries, I)
    __half* b;               // (entries, R)
    __half* yd;              // (entries, H)
    __half* hs;              // (n, Is)
    __half* bs;              // (n, R)
    __half* ysh;             // (n, H)
    __half* logits_out; int* sel_out; __half* wts_out;
    int* flags;
    FusedPhase ph[4];        // 0 shared gate|up, 1 routed gate|up, 2 shared down, 3 routed down
    int stages, stage_bytes;
    int off_act, off_ox, off_red, off_ring, off_plan, off_tab, off_prob;   // shared memory carve-up (bytes)
    int g_shared;            // CTAs [0, g_shared) run the shared expert's chain, the others the routed experts' chain
    unsigned long long wait_ns;
    // S10: the combine inside this launch (0: the caller launches it, e.g. after an exchange between ranks)
    int combine, by_expert, gate_col;
    const __half* residual; const __half* norm_w; float norm_eps;
    __half* out; __half* normed;
    int trace;               // 1: thread 0 of every CTA records the global timer after each step (diagnostic)
    int s6_segs;             // adjacent warps sharing one row of the shared down projection's U^T (1, 2, 4, 8 or 16)
};

// step time stamps of the last traced launch: [CTA][16]
constexpr int kFTraceSlots = 16;
static __device__ unsigned long long g_fused_trace[256 * kFTraceSlots + 256];   // + the counters' final values

// what the kernel needs of one routed expert, copied to shared memory when the kernel starts (the routed
// products' first loads would otherwise wait for two dependent reads of the descriptor tables)
struct ExpertPtrs {
    const unsigned char* gu_codes; const unsigned char* gu_sv;
    const unsigned char* d_codes; const unsigned char* d_sv;
    const __half* ut_gate; const __half* ut_up; const __half* ut_down;
    long long pad;
};

struct FusedPlan {
    int n_valid, n_slots, dead, pad;
    unsigned sel_mask[8];    // experts chosen by any token (E <= 256)
    int sel[kFMaxEntries];
    __half wts[kFMaxEntries];
    int entry_tok[kFMaxEntries];
    int entry_e[kFMaxEntries];
    __half entry_w[kFMaxEntries];
    int tok_entry[kFMaxEntries];
    int slot_e[kFMaxEntries], slot_off[kFMaxEntries], slot_cnt[kFMaxEntries];
    int slot_tok_entry[kFMaxEntries][kFRows];   // entry of token t in the slot, -1: the token did not choose it
};

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait for an arrival counter, by one thread.  Returns false when the wait ran out.
__device__ __noinline__ bool flag_wait(const int* f, int target, unsigned long long limit_ns, int code) {
    if (ld_acquire(f) >= target) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        if (ld_acquire(f) >= target) return true;
        if (global_ns() - t0 > limit_ns) {
            glq_ok(false, code, (unsigned long long)ld_acquire(f), (unsigned long long)target);
            return false;
        }
        __nanosleep(20);
    }
}
// all stores of the warp before, one arrival after
__device__ __forceinline__ void warp_signal(int* f, int amount, int lane) {
    __syncwarp();
    if (lane == 0) asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(f), "r"(amount) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

__device__ __forceinline__ uint4 ldg_nc_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ float dot8(const uint4 a, const uint4 b, float acc) {
    const __half2* pa = reinterpret_cast<const __half2*>(&a);
    const __half2* pb = reinterpret_cast<const __half2*>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 fa = __half22float2(pa[i]), fb = __half22float2(pb[i]);
        acc = fmaf(fa.x, fb.x, acc);
        acc = fmaf(fa.y, fb.y, acc);
    }
    return acc;
}
// One warp: out[i] = <w_row[k0 .. k0 + klen), x_i[k0 ..)> for up to 4 vectors x_i (nullptr: skipped); k0, klen
// multiples of 8.  The first vector is requested together with the weights, so that the two latencies overlap.
// The vectors are read through L2 (they may have been written by other CTAs of this launch).
// Not inlined on purpose: the kernel runs every piece of its code once or twice per launch, so its time is
// bound by instruction fetch as much as by data; one shared copy of each routine stays in the instruction cache.
__device__ __noinline__ void dense_row_dots(const __half* __restrict__ wrow, int k0, int klen, const __half* x0p,
                                            const __half* x1p, const __half* x2p, const __half* x3p, int lane,
                                            float* out) {
    const uint4* wp = reinterpret_cast<const uint4*>(wrow + k0);
    const int nvec = klen >> 3;
    float acc[kFRows] = {0.f, 0.f, 0.f, 0.f};
    const __half* xr[kFRows] = {x0p, x1p, x2p, x3p};
    for (int base = 0; base < nvec; base += 32 * 8) {
        uint4 q[8], x0[8];
#pragma unroll
        for (int d = 0; d < 8; ++d) {
            const int idx = base + d * 32 + lane;
            const bool in = idx < nvec;
            x0[d] = (in && xr[0] != nullptr) ? __ldcg(reinterpret_cast<const uint4*>(xr[0] + k0) + idx) : make_uint4(0, 0, 0, 0);
            q[d] = in ? ldg_nc_stream(wp + idx) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int d = 0; d < 8; ++d) {
            const int idx = base + d * 32 + lane;
            if (idx < nvec) {
                acc[0] = dot8(q[d], x0[d], acc[0]);
#pragma unroll
                for (int i = 1; i < kFRows; ++i)
                    if (xr[i] != nullptr) acc[i] = dot8(q[d], __ldcg(reinterpret_cast<const uint4*>(xr[i] + k0) + idx), acc[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kFRows; ++i) out[i] = warp_sum(acc[i]);
}

// Activation rows -> int8 digit fragments of the integer path (the layout stage_x_i8 of stream_mm.cuh
// writes, for one tile of 4 rows = 8 digit columns), by the stream warps (the first kFSW * 32 threads).  Not inlined: one copy serves every product.  rows[i] == nullptr or i >= cnt:
// the row is not staged (its columns keep stale data, whose outputs are never stored).
template <int FMT>
__device__ __noinline__ void fused_stage_i8(uint4* xs, float2* ox, const __half* r0, const __half* r1, const __half* r2,
                                            const __half* r3, int cnt, int nkb, int K) {
    constexpr bool COHERENT = true;            // rows may have been written by other CTAs of this launch: read through L2
    constexpr int NTHREADS = kFSW * 32;
    const __half* rows[kFRows] = {r0, r1, r2, r3};
    using F = Fmt<FMT>;
    constexpr int P8 = F::UPK / 4;
    constexpr int ncol = 2 * kFRows;
    const int total = cnt * nkb * F::UPK;
    for (int base = 0; base < total; base += NTHREADS) {
        const int u = base + (int)threadIdx.x;
        const bool valid = u < total;
        const int row = valid ? u / (nkb * F::UPK) : 0;
        const int rem = valid ? u % (nkb * F::UPK) : 0;
        const int kb = rem / F::UPK, wi = rem % F::UPK;
        const int k0 = kb * F::KB + wi * 16;
        __align__(16) __half v[16];
        const __half* src = valid ? rows[row] : nullptr;
        if (src != nullptr && k0 < K) {
            src += k0;
            if (k0 + 16 <= K) {
                const uint4* sp = reinterpret_cast<const uint4*>(src);
                *reinterpret_cast<uint4*>(&v[0]) = COHERENT ? __ldcg(sp) : __ldg(sp);
                *reinterpret_cast<uint4*>(&v[8]) = COHERENT ? __ldcg(sp + 1) : __ldg(sp + 1);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    v[j] = (k0 + j < K) ? (COHERENT ? __ldcg(src + j) : src[j]) : __float2half(0.f);
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
        if (mx > 0.f) (void)frexpf(mx, &ex);
        const int sh = 14 - ex;
        const float scale = ldexpf(1.f, sh);
        int d0[16], d1[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int q = __float2int_rn(f[j] * scale);
            d1[j] = (q + 128) >> 8;
            d0[j] = q - (d1[j] << 8);
        }
        auto pack4 = [](const int* d, int c0, int c1, int c2, int c3) -> uint32_t {
            return (uint32_t)(d[c0] & 0xff) | ((uint32_t)(d[c1] & 0xff) << 8) | ((uint32_t)(d[c2] & 0xff) << 16) |
                   ((uint32_t)(d[c3] & 0xff) << 24);
        };
        if (valid && src != nullptr) {
            uint4 lo, hi;
            int t, piece;
            if constexpr (FMT == GLQ_FMT_Q2) {
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
            if (wi == 0) ox[kb * kFRows + row] = make_float2(ldexpf(1.f, -sh), sx);
        }
    }
}

// Probabilities of one token by one warp: softmax over the fp16 router logits in fp32 -- the arithmetic of
// moe_plan_kernel (a probability that is not a number counts as zero).  prob: E floats of shared memory.
__device__ __forceinline__ void softmax_token(const __half* row, int E, int lane, float* prob) {
    float lv[8], pv[8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        lv[i] = e < E ? __half2float(__ldcg(row + e)) : -INFINITY;
        mx = fmaxf(mx, lv[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        pv[i] = (lane + 32 * i) < E ? expf(lv[i] - mx) : 0.f;
        sum += pv[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        const float pr = pv[i] / sum;
        if (e < E) prob[e] = pr >= 0.f ? pr : 0.f;
    }
}

// bar.sync over a subset of the CTA's warps
__device__ __forceinline__ void stream_barrier() { named_bar_sync(15, kFSW * 32); }
__device__ __forceinline__ void dense_barrier() { named_bar_sync(14, (kFW - kFSW) * 32); }

template <int FMT>
__global__ void __launch_bounds__(kFT, 1) moe_fused_kernel(const FusedParams p) {
    using F = Fmt<FMT>;
    constexpr int BB = block_bytes<FMT>();
    constexpr int kPieces = F::UPK / 4;
    constexpr int ncol_i8 = 2 * kFRows;
    constexpr int kDW = kFW - kFSW;            // dense warps
    constexpr int kDT = kDW * 32;              // dense threads
    constexpr int kST = kFSW * 32;             // stream threads
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int cta = blockIdx.x, G = gridDim.x;
    const int n = p.n, S = p.stages;
    // the CTAs [0, Gs) carry the shared expert's chain, the CTAs [Gs, G) the routed experts' chain
    const int Gs = p.g_shared;
    const bool shared_cta = cta < Gs;
    const int sub_cta = shared_cta ? cta : cta - Gs;       // index and size of this CTA's subset
    const int sub_G = shared_cta ? Gs : G - Gs;
    const bool is_stream = w < kFSW;

    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem);
    uint4* xs = reinterpret_cast<uint4*>(smem + p.off_act);
    float2* ox = reinterpret_cast<float2*>(smem + p.off_ox);
    float2* red = reinterpret_cast<float2*>(smem + p.off_red);
    float* prob = reinterpret_cast<float*>(smem + p.off_prob);
    FusedPlan& plan = *reinterpret_cast<FusedPlan*>(smem + p.off_plan);
    ExpertPtrs* tab = reinterpret_cast<ExpertPtrs*>(smem + p.off_tab);
    const uint32_t xs_a = smem_u32(xs), ox_a = smem_u32(ox);
    const uint32_t ring_a = smem_u32(smem + p.off_ring) + (uint32_t)(w * S * p.stage_bytes);
    const uint32_t bar_a = smem_u32(bars) + (uint32_t)(w * kFMaxStages * 8);
    int* flags = p.flags;

    bool dead = false;        // a wait ran out somewhere in this CTA: no more waiting
    auto trace = [&](int slot) {
        if (p.trace && lane == 0 && (w == 0 || w == kFSW) && cta < 256)
            g_fused_trace[cta * kFTraceSlots + slot] = global_ns();
    };
    if (is_stream) trace(0);

    // every stream warp owns its barriers and its ring: its lane 0 initialises them and alone arms them
    if (is_stream && lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(bar_a + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (tid == kST) {
        plan.n_valid = 0;
        plan.n_slots = 0;
        plan.dead = 0;
    }
    __syncthreads();

    // ---- bounded waits -----------------------------------------------------------------------------------------
    // one warp (lane 0 polls)
    auto warp_wait = [&](const int* f, int target, int code) {
        int ok = 1;
        if (lane == 0 && !dead) ok = flag_wait(f, target, p.wait_ns, code) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) dead = true;
    };
    // all stream warps (thread 0 polls); also a barrier of the stream warps before and after
    auto stream_wait = [&](const int* f, int target, int code) {
        stream_barrier();
        if (tid == 0 && !dead && !flag_wait(f, target, p.wait_ns, code)) plan.dead = 1;
        stream_barrier();
        dead = dead || plan.dead != 0;
    };

    if (!is_stream) {
        // =========================================================================================================
        // dense warps: row tasks, routing, plan
        // =========================================================================================================
        const int dw = w - kFSW, dt = tid - kST;
        // ---------------- S1: dense rows of the router matrix (all CTAs) ----------------
        {
            const __half* xr[kFRows];
#pragma unroll
            for (int i = 0; i < kFRows; ++i) xr[i] = i < n ? p.x + (size_t)i * p.H : nullptr;
#pragma unroll 1
            for (int task = cta + G * dw; task < p.dense_rows; task += G * kDW) {
                float out[kFRows];
                dense_row_dots(p.router_rm + (size_t)task * p.H, 0, p.H, xr[0], xr[1], xr[2], xr[3], lane, out);
                if (lane == 0)
                    for (int i = 0; i < n; ++i) p.logits[(size_t)i * p.ldl + task] = __float2half_rn(out[i]);
                warp_signal(flags + FL_R, 1, lane);
            }
        }
        trace(1);
        // the routed experts' pointers -> shared memory (consumed after the plan; the loads overlap the wait for the logits)
        for (int e = dt; e < p.E; e += kDT) {
            ExpertPtrs ep;
            ep.gu_codes = reinterpret_cast<const unsigned char*>(p.ph[1].table[e].codes);
            ep.gu_sv = reinterpret_cast<const unsigned char*>(p.ph[1].table[e].sv);
            ep.d_codes = reinterpret_cast<const unsigned char*>(p.ph[3].table[e].codes);
            ep.d_sv = reinterpret_cast<const unsigned char*>(p.ph[3].table[e].sv);
            ep.ut_gate = p.R > 0 ? reinterpret_cast<const __half*>(p.ut_rm_gate_up[e]) : nullptr;
            ep.ut_up = p.R > 0 ? reinterpret_cast<const __half*>(p.ut_rm_gate_up[p.E + e]) : nullptr;
            ep.ut_down = p.R > 0 ? reinterpret_cast<const __half*>(p.ut_rm_down[e]) : nullptr;
            ep.pad = 0;
            tab[e] = ep;
        }
        // the U^T rows of the shared down projection's hs.U (S6): towards L2 now, needed after the shared gate|up
        const int s6_segs = p.s6_segs;
        if (shared_cta && p.ph[2].live && p.ph[2].rank > 0) {
            const int task = sub_cta * (kDW / s6_segs) + dw / s6_segs;
            if (task < p.R) {
                const int klen = p.Is / s6_segs;
                const char* row = reinterpret_cast<const char*>(p.sh_ut_rm_down + (size_t)task * p.Is + (dw % s6_segs) * klen);
                for (int off = lane * 128; off < klen * 2; off += 32 * 128) prefetch_l2(row + off);
            }
        }
        // ---------------- S3: routing plan (every CTA for itself) ----------------
        // Every dense warp polls the router's counter for itself (no barrier before the routing); warp dw routes
        // token dw alone; one barrier; then one thread per (token, slot) places its entry and, for the first
        // entry of an expert, the slot.
        for (int i = dt; i < kFMaxEntries * kFRows; i += kDT) (&plan.slot_tok_entry[0][0])[i] = -1;
        if (dt == 0) plan.n_slots = 0;
        if (dt < 8) plan.sel_mask[dt] = 0u;
        dense_barrier();
        {
            int ok = 1;
            if (lane == 0) ok = flag_wait(flags + FL_R, p.dense_rows, p.wait_ns, 201) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) dead = true, plan.dead = 1;
        }
        trace(2);
        {
            const int k = p.k, nk = n * k, E = p.E;
            constexpr int kProbLd = 256 + 16;
            if (dw < n) {
                // probabilities, then ranks: an expert's rank is the number of experts that beat it (ties to the lower
                // index); rank < k is selected as slot `rank`; the weights are the selected probabilities, optionally
                // divided by their sum taken in selection order (the arithmetic of moe_plan_kernel)
                float* pr = prob + dw * kProbLd;
                softmax_token(p.logits + (size_t)dw * p.ldl, E, lane, pr);
                __syncwarp();
                for (int e = lane; e < E; e += 32) {
                    const float pe = pr[e];
                    int rank = 0;
#pragma unroll 4
                    for (int j = 0; j < E; ++j) {
                        const float pj = pr[j];
                        rank += (pj > pe || (pj == pe && j < e)) ? 1 : 0;
                    }
                    if (rank < k) {
                        plan.sel[dw * k + rank] = e;
                        pr[256 + rank] = pe;
                        atomicOr(&plan.sel_mask[e >> 5], 1u << (e & 31));
                    }
                }
                __syncwarp();
                if (lane < k) {
                    float wsum = 0.f;
                    for (int s = 0; s < k; ++s) wsum += pr[256 + s];
                    const float pe = pr[256 + lane];
                    plan.wts[dw * k + lane] = __float2half_rn(p.renorm ? pe / wsum : pe);
                }
            }
            dense_barrier();
            // entries grouped by expert (ascending), in token order within an expert: every rank numbers them alike;
            // slots: the experts of this rank among them, in the same order
            if (dt < nk) {
                const int e = plan.sel[dt];
                int pos = 0, cnt = 0, slot = 0, first = 1;
                for (int j = 0; j < nk; ++j) {
                    const int ej = plan.sel[j];
                    pos += (ej < e || (ej == e && j < dt)) ? 1 : 0;
                    cnt += ej == e ? 1 : 0;
                    first &= !(ej == e && j < dt);
                }
                // this rank's chosen experts below e
                for (int e2 = p.ep_rank; e2 < e; e2 += p.ep_world) slot += (plan.sel_mask[e2 >> 5] >> (e2 & 31)) & 1u;
                plan.entry_tok[pos] = dt / k;
                plan.entry_e[pos] = e;
                plan.entry_w[pos] = plan.wts[dt];
                plan.tok_entry[dt] = pos;
                if (e % p.ep_world == p.ep_rank) {
                    plan.slot_tok_entry[slot][dt / k] = pos;
                    if (first) {
                        plan.slot_e[slot] = e;
                        plan.slot_off[slot] = pos;
                        plan.slot_cnt[slot] = cnt;
                        atomicAdd(&plan.n_slots, 1);
                    }
                }
                if (dt == 0) plan.n_valid = nk;
            }
        }
        // the plan is published to this CTA's stream warps (the routed CTAs' wait for it before their products, the
        // shared CTAs' before the combine)
        // (arrive only: the dense warps need nothing from the stream warps and must not wait for them)
        dense_barrier();            // the plan is complete for every dense warp too
        __threadfence_block();
        asm volatile("bar.arrive 13, %0;" ::"n"(kFT) : "memory");
        trace(3);
        const int n_slots = plan.n_slots;
        // ---------------- S4: x.U of the routed gate / up clusters (all CTAs) ----------------
        if (p.R > 0) {
            const int tasks = n_slots * 2 * p.R;
#pragma unroll 1
            for (int task = cta + G * dw; task < tasks; task += G * kDW) {
                const int slot = task / (2 * p.R), rem = task - slot * 2 * p.R;
                const int proj = rem / p.R, row = rem - proj * p.R;
                const int e = plan.slot_e[slot], e0 = plan.slot_off[slot], cnt = plan.slot_cnt[slot];
                const __half* ut = proj == 0 ? tab[e].ut_gate : tab[e].ut_up;
                const __half* xr[kFRows];
#pragma unroll
                for (int i = 0; i < kFRows; ++i) xr[i] = i < cnt ? p.x + (size_t)plan.entry_tok[e0 + i] * p.H : nullptr;
                float out[kFRows];
                dense_row_dots(ut + (size_t)row * p.H, 0, p.H, xr[0], xr[1], xr[2], xr[3], lane, out);
                if (lane == 0) {
                    __half* dst = proj == 0 ? p.a_gate : p.a_up;
                    for (int i = 0; i < cnt; ++i) dst[(size_t)(e0 + i) * p.R + row] = __float2half_rn(out[i]);
                }
                warp_signal(flags + FL_A + slot, 1, lane);
            }
        }
        trace(4);
        // CTA 0 leaves the plan in global memory for the combine (and the exchange) of a later launch
        if (cta == 0) {
            const int nk = n * p.k;
            for (int i = dt; i < nk; i += kDT) {
                p.sel[i] = plan.sel[i];
                p.wts[i] = plan.wts[i];
                p.tok_entries[i] = plan.tok_entry[i];
                if (p.sel_out) p.sel_out[i] = plan.sel[i];
                if (p.wts_out) p.wts_out[i] = plan.wts[i];
            }
            for (int q = dt; q < plan.n_valid; q += kDT) {
                p.entry_row[q] = plan.entry_tok[q];
                p.entry_scale[q] = plan.entry_w[q];
            }
            for (int s = dt; s < plan.n_slots; s += kDT) {
                p.active[s] = plan.slot_e[s];
                p.slot_count[s] = plan.slot_cnt[s];
                p.slot_offset[s] = plan.slot_off[s];
            }
            if (dt == 0) *p.n_active = plan.n_slots;
            if (p.logits_out)
                for (int i = dt; i < n * p.E; i += kDT)
                    p.logits_out[i] = __ldcg(p.logits + (size_t)(i / p.E) * p.ldl + (i % p.E));
        }
        if (shared_cta) {
            // ---------------- S6: hs.U of the shared down projection ----------------
            // a row of U^T is I_shared channels long: s6_segs adjacent dense warps share it
            if (p.ph[2].live && p.ph[2].rank > 0) {
                const int rows_per_cta = kDW / s6_segs;
                bool waited = false;
                float* rbuf = prob;      // idle after the plan
#pragma unroll 1
                for (int base = sub_cta * rows_per_cta; base < p.R; base += sub_G * rows_per_cta) {
                    if (!waited) warp_wait(flags + FL_HS, p.ph[0].npairs, 202), waited = true;
                    const int task = base + dw / s6_segs, seg = dw % s6_segs;
                    const int klen = p.Is / s6_segs;
                    const __half* xr[kFRows];
#pragma unroll
                    for (int i = 0; i < kFRows; ++i) xr[i] = (i < n && task < p.R) ? p.hs + (size_t)i * p.Is : nullptr;
                    float out[kFRows] = {0.f, 0.f, 0.f, 0.f};
                    if (task < p.R)
                        dense_row_dots(p.sh_ut_rm_down + (size_t)task * p.Is, seg * klen, klen, xr[0], xr[1], xr[2], xr[3], lane, out);
                    if (s6_segs > 1) {
                        dense_barrier();
                        if (seg != 0 && lane < kFRows) rbuf[dw * kFRows + lane] = out[lane];
                        dense_barrier();
                        if (seg == 0)
                            for (int s2 = 1; s2 < s6_segs; ++s2)
#pragma unroll
                                for (int i = 0; i < kFRows; ++i) out[i] += rbuf[(dw + s2) * kFRows + i];
                    }
                    if (seg == 0 && task < p.R) {
                        if (lane == 0)
                            for (int i = 0; i < n; ++i) p.bs[(size_t)i * p.R + task] = __float2half_rn(out[i]);
                        warp_signal(flags + FL_BS, 1, lane);
                    }
                }
            }
        } else if (p.R > 0) {
            // ---------------- S8: h.U of the routed down clusters ----------------
            const int tasks = n_slots * p.R;
            // the U^T rows towards L2 while gate|up still runs
#pragma unroll 1
            for (int task = sub_cta + sub_G * dw; task < tasks; task += sub_G * kDW) {
                const int slot = task / p.R, row = task - slot * p.R;
                const char* rowp = reinterpret_cast<const char*>(tab[plan.slot_e[slot]].ut_down + (size_t)row * p.I);
                for (int off = lane * 128; off < p.I * 2; off += 32 * 128) prefetch_l2(rowp + off);
            }
            int waited_slot = -1;
#pragma unroll 1
            for (int task = sub_cta + sub_G * dw; task < tasks; task += sub_G * kDW) {
                const int slot = task / p.R, row = task - slot * p.R;
                if (slot != waited_slot) warp_wait(flags + FL_H + slot, p.ph[1].npairs, 204), waited_slot = slot;
                const int e = plan.slot_e[slot], e0 = plan.slot_off[slot], cnt = plan.slot_cnt[slot];
                const __half* xr[kFRows];
#pragma unroll
                for (int i = 0; i < kFRows; ++i) xr[i] = i < cnt ? p.h + (size_t)(e0 + i) * p.I : nullptr;
                float out[kFRows];
                dense_row_dots(tab[e].ut_down + (size_t)row * p.I, 0, p.I, xr[0], xr[1], xr[2], xr[3], lane, out);
                if (lane == 0)
                    for (int i = 0; i < cnt; ++i) p.b[(size_t)(e0 + i) * p.R + row] = __float2half_rn(out[i]);
                warp_signal(flags + FL_B + slot, 1, lane);
            }
        }
        trace(5);
    } else {
        // =========================================================================================================
        // stream warps: the quantized products of this CTA's chain
        // =========================================================================================================
        bool plan_ready = false;
        const int ph_a = shared_cta ? 0 : 1, ph_b = shared_cta ? 2 : 3;     // this chain's gate|up and down
        // ---- items of a streamed product: (iteration j of this CTA) -> (slot, pair, split) --------------------
        struct Item {
            int slot, pair, s, kb_lo, kb_hi, ncode, nch;
            const unsigned char* codes;
            const unsigned char* sv;
            bool valid;
        };
        auto nslots_of = [&](int ph) -> int { return (ph & 1) ? plan.n_slots : (p.ph[ph].live ? 1 : 0); };
        auto first_iter = [&](int ph) -> int {
            int d = (sub_cta - p.ph[ph].cta_base) % sub_G;
            return d < 0 ? d + sub_G : d;
        };
        auto make_item = [&](Item& im, int ph, int it) {
            const FusedPhase& P = p.ph[ph];
            im.slot = it / P.ipp;
            const int r = it - im.slot * P.ipp;
            im.pair = r * P.ppi + (w >> P.sk_log2);
            im.s = w & (P.sk - 1);
            im.valid = im.pair < P.npairs;
            im.kb_lo = im.s * P.kb_per_split;
            im.kb_hi = min(P.nkb, im.kb_lo + P.kb_per_split);
            im.ncode = im.kb_hi > im.kb_lo ? (im.kb_hi - im.kb_lo + kStreamCB - 1) / kStreamCB : 0;
            if (ph & 1) {
                const ExpertPtrs& ep = tab[plan.slot_e[im.slot]];
                im.codes = ph == 1 ? ep.gu_codes : ep.d_codes;
                im.sv = P.rank > 0 ? (ph == 1 ? ep.gu_sv : ep.d_sv) : nullptr;
            } else {
                im.codes = reinterpret_cast<const unsigned char*>(P.w.codes);
                im.sv = P.rank > 0 ? reinterpret_cast<const unsigned char*>(P.w.sv) : nullptr;
            }
            im.nch = im.ncode + ((im.s == 0 && im.sv != nullptr) ? P.ns : 0);
        };

        // ---- fetch cursor: the warp's chunks in the order it consumes them, across the chain's two products -----
        int f_ph = ph_a, f_it = first_iter(ph_a), f_c = 0, f_stage = 0, f_inflight = 0;
        int c_stage = 0;
        uint32_t c_phase = 0;
        bool f_live = false, f_end = false;
        Item fi;
        auto fetch_seek = [&]() {
            f_live = false;
            while (!f_end) {
                if ((f_ph & 1) && !plan_ready) return;      // the routed products' items are known after the plan
                const int total = nslots_of(f_ph) * p.ph[f_ph].ipp;
                while (f_it < total) {
                    make_item(fi, f_ph, f_it);
                    if (fi.valid && fi.nch > 0) {
                        f_live = true;
                        return;
                    }
                    f_it += sub_G;
                }
                if (f_ph == ph_b) {
                    f_end = true;
                } else {
                    f_ph = ph_b;
                    f_it = first_iter(ph_b);
                }
            }
        };
        auto fetch_one = [&]() {
            if (lane == 0) {
                const FusedPhase& P = p.ph[f_ph];
                const uint32_t bar = bar_a + 8 * f_stage;
                const uint32_t dst = ring_a + (uint32_t)(f_stage * p.stage_bytes);
                const void* src;
                uint32_t bytes;
                if (f_c < fi.ncode) {
                    const int kb0 = fi.kb_lo + f_c * kStreamCB;
                    bytes = (uint32_t)(min(kStreamCB, fi.kb_hi - kb0) * 2 * BB);
                    src = fi.codes + ((size_t)fi.pair * P.nkb + kb0) * (2 * BB);
                } else {
                    bytes = 4096;
                    src = fi.sv + ((size_t)fi.pair * P.ns + (f_c - fi.ncode)) * 4096;
                }
                mbar_expect_tx(bar, bytes);
                bulk_g2s(dst, src, bytes, bar);
            }
            if (++f_stage == S) f_stage = 0;
            ++f_inflight;
            if (++f_c >= fi.nch) {
                f_c = 0;
                f_it += sub_G;
                fetch_seek();
            }
        };
        auto fetch_fill = [&]() {
            if (!f_live) fetch_seek();
            while (f_live && f_inflight < S) fetch_one();
        };
        auto ring_wait = [&]() -> uint32_t {
            mbar_wait(bar_a + 8 * c_stage, c_phase, dead);
            return ring_a + (uint32_t)(c_stage * p.stage_bytes);
        };
        auto ring_release = [&]() {
            __syncwarp();
            if (++c_stage == S) c_stage = 0, c_phase ^= 1u;
            --f_inflight;
            fetch_fill();
        };

        // ---- the chain's two products, one after the other, through ONE copy of the item loop ----------------------
        // RowMap of a problem: for activation column c (0..3): the output row (also the row of the low-rank operand),
        // and the output scale (negative: none).
        struct RowMap {
            int out_row[kFRows];
            float scale[kFRows];
        };
        auto stage = [&](const __half* base, long long ld, int e0, int cnt, int nkb, int K, const int* tokmap) {
            const __half* r[kFRows];
#pragma unroll
            for (int i = 0; i < kFRows; ++i) r[i] = i < cnt ? base + (size_t)(tokmap ? tokmap[i] : e0 + i) * ld : nullptr;
            fused_stage_i8<FMT>(xs, ox, r[0], r[1], r[2], r[3], cnt, nkb, K);
            stream_barrier();
        };
        fetch_fill();       // shared chain: the gate|up codes of this warp, on their way before anything else
        trace(6);
        int red_par = 0, n_slots = 0;
#pragma unroll 1
        for (int pi = 0; pi < 2; ++pi) {
            const int ph = pi ? ph_b : ph_a;
            const FusedPhase& P = p.ph[ph];
            // operands of the low-rank term, outputs and counters of this product
            const __half* a0;
            const __half* a1;
            long long lda;
            int a_col0, a_target;
            const int* a_flag_base;
            bool per_slot_a, per_slot_out;
            __half* y;
            long long ldy;
            int* out_flag_base;
            if (ph == 0) {          // S2: the shared expert's x.U sits in columns sh_a_row .. of the logits buffer
                a0 = p.logits, a1 = p.logits + p.R, lda = p.ldl, a_col0 = p.sh_a_row, a_flag_base = flags + FL_R,
                a_target = p.dense_rows, per_slot_a = false, y = p.hs, ldy = p.Is, out_flag_base = flags + FL_HS, per_slot_out = false;
            } else if (ph == 1) {   // S5
                a0 = p.a_gate, a1 = p.a_up, lda = p.R, a_col0 = 0, a_flag_base = flags + FL_A, a_target = 2 * p.R,
                per_slot_a = true, y = p.h, ldy = p.I, out_flag_base = flags + FL_H, per_slot_out = true;
            } else if (ph == 2) {   // S7
                a0 = a1 = p.bs, lda = p.R, a_col0 = 0, a_flag_base = flags + FL_BS, a_target = p.R, per_slot_a = false,
                y = p.ysh, ldy = p.H, out_flag_base = flags + FL_Y, per_slot_out = false;
            } else {                // S9
                a0 = a1 = p.b, lda = p.R, a_col0 = 0, a_flag_base = flags + FL_B, a_target = p.R, per_slot_a = true, y = p.yd,
                ldy = p.H, out_flag_base = flags + FL_Y, per_slot_out = false;
            }
            if (pi == 0) {
                // S0: x of the n tokens, staged once for the gate|up product of either chain
                stage(p.x, p.H, 0, n, p.ph[1].nkb, p.H, nullptr);
                if (!shared_cta) {
                    named_bar_sync(13, kFT);        // the plan, from this CTA's dense warps
                    plan_ready = true;
                    n_slots = plan.n_slots;
                    dead = dead || plan.dead != 0;
                    fetch_fill();           // the routed experts' gate|up codes
                }
                trace(7);
            }
            const int total = nslots_of(ph) * P.ipp;
            const int sk = P.sk;
            int staged_slot = -1;
#pragma unroll 1
            for (int it = first_iter(ph); it < total; it += sub_G) {
                Item im;
                make_item(im, ph, it);
                if (pi == 1 && im.slot != staged_slot) {
                    // the down product's activations: all of the chain's gate|up outputs for this problem must be there
                    if (ph == 2) {
                        stream_wait(flags + FL_HS, p.ph[0].npairs, 203);     // also: every stream warp is done with the staged x
                        stage(p.hs, p.Is, 0, n, P.nkb, p.Is, nullptr);
                    } else {
                        stream_wait(flags + FL_H + im.slot, p.ph[1].npairs, 205);
                        stage(p.h, p.I, plan.slot_off[im.slot], plan.slot_cnt[im.slot], P.nkb, p.I, nullptr);
                    }
                    staged_slot = im.slot;
                }
                float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};   // [tile in pair][weight row g / g+8], activation row t
                if (im.valid) {
#pragma unroll 1
                    for (int c = 0; c < im.ncode; ++c) {
                        const uint32_t st = ring_wait();
                        const int kb0 = im.kb_lo + c * kStreamCB;
                        const int nblk = min(kStreamCB, im.kb_hi - kb0);
#pragma unroll 1
                        for (int b = 0; b < nblk; ++b) {
                            const int kb = kb0 + b;
                            uint4 bx[1][2];
#pragma unroll
                            for (int i = 0; i < kPieces; ++i)
                                bx[0][i] = lds128(xs_a + (uint32_t)((((kb * kPieces + i) * ncol_i8) + g) * 4 + t) * 16u);
                            const uint2 ov = lds64(ox_a + (uint32_t)(kb * kFRows + t) * 8u);
                            const float o_s = __uint_as_float(ov.x), o_x = __uint_as_float(ov.y);
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const uint32_t blk = st + (uint32_t)((b * 2 + j) * BB);
                                const uint4 q = lds128(blk + lane * 16);
                                const uint2 szv = lds64(blk + 512 + g * 8);
                                int ci[1][4];
                                tile_block_i8<FMT, 1>(q, bx, ci);
                                const __half2 sz0 = *reinterpret_cast<const __half2*>(&szv.x);
                                const __half2 sz1 = *reinterpret_cast<const __half2*>(&szv.y);
                                const float s0 = __low2float(sz0), z0 = __high2float(sz0);
                                const float s1 = __low2float(sz1), z1 = __high2float(sz1);
                                const float f0 = (float)(ci[0][0] + (ci[0][1] << 8)) * o_s;
                                const float f1 = (float)(ci[0][2] + (ci[0][3] << 8)) * o_s;
                                acc[j][0] = fmaf(s0, fmaf(-z0, o_x, f0), acc[j][0]);
                                acc[j][1] = fmaf(s1, fmaf(-z1, o_x, f1), acc[j][1]);
                            }
                        }
                        ring_release();
                    }
                }
                // ---- k splits of a pair: adjacent warps, fixed-order sum through shared memory ----
                if (sk > 1) {
                    float2* rbuf = red + (size_t)red_par * (kFSW * 2 * 32);
                    if (im.s != 0) {
                        rbuf[(w * 2 + 0) * 32 + lane] = make_float2(acc[0][0], acc[0][1]);
                        rbuf[(w * 2 + 1) * 32 + lane] = make_float2(acc[1][0], acc[1][1]);
                    }
                    named_bar_sync(1 + (w >> P.sk_log2), sk * 32);
                    if (im.s == 0) {
                        for (int s2 = 1; s2 < sk; ++s2) {
                            const float2 v0 = rbuf[((w + s2) * 2 + 0) * 32 + lane];
                            const float2 v1 = rbuf[((w + s2) * 2 + 1) * 32 + lane];
                            acc[0][0] += v0.x;
                            acc[0][1] += v0.y;
                            acc[1][0] += v1.x;
                            acc[1][1] += v1.y;
                        }
                    }
                    red_par ^= 1;
                }
                if (im.s != 0 || !im.valid) continue;

                // ---- rows of this problem ----
                RowMap rm;
#pragma unroll
                for (int c = 0; c < kFRows; ++c) {
                    rm.scale[c] = -1.f;
                    if (ph == 1) {
                        rm.out_row[c] = plan.slot_tok_entry[im.slot][c];
                    } else if (ph == 3) {
                        const int e0 = plan.slot_off[im.slot], cnt = plan.slot_cnt[im.slot];
                        rm.out_row[c] = c < cnt ? e0 + c : -1;
                        if (c < cnt) rm.scale[c] = __half2float(plan.entry_w[e0 + c]);
                    } else {
                        rm.out_row[c] = c < n ? c : -1;
                    }
                }
                // ---- low-rank term: SV chunks from the ring, the operand rows from global memory (L2) ----
                float lo[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                const int nsv = im.nch - im.ncode;
                if (nsv > 0) warp_wait(a_flag_base + (per_slot_a ? im.slot : 0), a_target, 210 + ph);
#pragma unroll 1
                for (int c = 0; c < nsv; ++c) {
                    const uint32_t st = ring_wait();
                    const int cc0 = c * 64 + 16 * t;
                    const bool in_rank = cc0 < P.rank;
                    const uint4 z4 = make_uint4(0, 0, 0, 0);
                    // the op's column g is activation column g (only 0..3 exist)
                    const int arow = g < kFRows ? rm.out_row[g] : -1;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint32_t pa = st + (uint32_t)((j * 16 + g) * 128 + t * 32);
                        const uint4 sa0 = in_rank ? lds128(pa) : z4, sa1 = in_rank ? lds128(pa + 16) : z4;
                        const uint4 sb0 = in_rank ? lds128(pa + 8 * 128) : z4, sb1 = in_rank ? lds128(pa + 8 * 128 + 16) : z4;
                        uint4 av0 = z4, av1 = z4;
                        if (in_rank && arow >= 0) {
                            const __half* ap = (P.swiglu && j == 1 ? a1 : a0) + (size_t)arow * lda + a_col0 + cc0;
                            av0 = __ldcg(reinterpret_cast<const uint4*>(ap));
                            av1 = __ldcg(reinterpret_cast<const uint4*>(ap) + 1);
                        }
                        mma16816(lo[j], sa0.x, sb0.x, sa0.y, sb0.y, av0.x, av0.y);
                        mma16816(lo[j], sa0.z, sb0.z, sa0.w, sb0.w, av0.z, av0.w);
                        mma16816(lo[j], sa1.x, sb1.x, sa1.y, sb1.y, av1.x, av1.y);
                        mma16816(lo[j], sa1.z, sb1.z, sa1.w, sb1.w, av1.z, av1.w);
                    }
                    ring_release();
                }
                // ---- epilogue: activation column t, weight rows g and g + 8 of both tiles ----
                float val[2][2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    float v0 = round16(acc[j][0]);
                    float v1 = round16(acc[j][1]);
                    if (nsv > 0) {
                        // the low-rank op holds columns 2t', 2t'+1 in lane t': fetch this lane's column t
                        const int src = (g << 2) | (t >> 1);
                        const float a0v = __shfl_sync(0xffffffffu, lo[j][0], src);
                        const float a1v = __shfl_sync(0xffffffffu, lo[j][1], src);
                        const float b0v = __shfl_sync(0xffffffffu, lo[j][2], src);
                        const float b1v = __shfl_sync(0xffffffffu, lo[j][3], src);
                        v0 = round16(v0 + round16((t & 1) ? a1v : a0v));
                        v1 = round16(v1 + round16((t & 1) ? b1v : b0v));
                    }
                    val[j][0] = v0;
                    val[j][1] = v1;
                }
                const int orow = rm.out_row[t];
                if (orow >= 0) {
                    if (P.swiglu) {
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int nn = im.pair * kRowTile + g + 8 * hh;
                            if (nn < P.N) y[(size_t)orow * ldy + nn] = __float2half_rn(round16(silu16(val[0][hh]) * val[1][hh]));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j)
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh) {
                                const int nn = (im.pair * 2 + j) * kRowTile + g + 8 * hh;
                                if (nn < P.N) {
                                    float v = val[j][hh];
                                    if (rm.scale[t] >= 0.f) v = round16(rm.scale[t] * v);
                                    y[(size_t)orow * ldy + nn] = __float2half_rn(v);
                                }
                            }
                    }
                }
                warp_signal(out_flag_base + (per_slot_out ? im.slot : 0), 1, lane);
            }
            trace(8 + pi);
        }
        // ---------------- S10: combine (token t on CTA t) ----------------
        // out[t] = sum over the token's entries (already weighted, fp16), accumulated in fp16 in slot order or in
        // expert order, + sigmoid(shared gate logit) * shared expert row [+ residual]; normed = rms_norm(out) * weight.
        // The shared chain ends early, so its CTAs take the combine (they are already waiting when the last down
        // output lands); without a shared expert the first routed CTAs do.
        if (shared_cta) {
            named_bar_sync(13, kFT);        // the plan, from this CTA's dense warps
            n_slots = plan.n_slots;
            dead = dead || plan.dead != 0;
        }
        if (p.combine && cta < n) {
            const int tok = cta, k = p.k, H = p.H;
            const int y_target = (p.ph[2].live ? p.ph[2].npairs : 0) + n_slots * p.ph[3].npairs;
            stream_wait(flags + FL_Y, y_target, 206);
            int order[16];
            for (int s = 0; s < k; ++s) order[s] = s;
            if (p.by_expert)
                for (int i = 1; i < k; ++i) {
                    const int v = order[i];
                    const int ev = plan.sel[tok * k + v];
                    int j = i - 1;
                    while (j >= 0 && plan.sel[tok * k + order[j]] > ev) {
                        order[j + 1] = order[j];
                        --j;
                    }
                    order[j + 1] = v;
                }
            const float gate = (p.ysh && p.gate_col >= 0)
                                   ? sigmoid16(__half2float(__ldcg(p.logits + (size_t)tok * p.ldl + p.gate_col))) : 1.f;
            // 384 threads x 8 columns per step
            float ss = 0.f;
#pragma unroll 1
            for (int c0 = tid * 8; c0 < H; c0 += kST * 8) {
                float acc[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll 1
                for (int s = 0; s < k; ++s) {
                    const int entry = plan.tok_entry[tok * k + order[s]];
                    if (entry < 0) continue;     // dropped slot
                    __align__(16) __half v[8];
                    *reinterpret_cast<uint4*>(v) = __ldcg(reinterpret_cast<const uint4*>(p.yd + (size_t)entry * H + c0));
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = round16(acc[i] + __half2float(v[i]));
                }
                if (p.ysh) {
                    __align__(16) __half v[8];
                    *reinterpret_cast<uint4*>(v) = __ldcg(reinterpret_cast<const uint4*>(p.ysh + (size_t)tok * H + c0));
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = round16(acc[i] + round16(gate * __half2float(v[i])));
                }
                if (p.residual) {
                    __align__(16) __half v[8];
                    *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(p.residual + (size_t)tok * H + c0));
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = round16(__half2float(v[i]) + acc[i]);
                }
                __align__(16) __half o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    o[i] = __float2half_rn(acc[i]);       // exact: the sums above are already rounded to fp16
                    ss += acc[i] * acc[i];
                }
                *reinterpret_cast<uint4*>(p.out + (size_t)tok * H + c0) = *reinterpret_cast<const uint4*>(o);
            }
            if (p.normed) {
                float* rs = reinterpret_cast<float*>(red);
                ss = warp_sum(ss);
                stream_barrier();
                if (lane == 0) rs[w] = ss;
                stream_barrier();
                float tot = 0.f;
#pragma unroll
                for (int i = 0; i < kFSW; ++i) tot += rs[i];
                const float r = rsqrtf(tot / H + p.norm_eps);
#pragma unroll 1
                for (int c0 = tid * 8; c0 < H; c0 += kST * 8) {
                    // this thread's own outputs of the loop above (fp16, exactly the summed values)
                    __align__(16) __half v[8], o[8], wv[8];
                    *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(p.out + (size_t)tok * H + c0);
                    if (p.norm_w) *reinterpret_cast<uint4*>(wv) = __ldg(reinterpret_cast<const uint4*>(p.norm_w + c0));
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float nv = __half2float(v[i]) * r;
                        o[i] = __float2half_rn(p.norm_w ? __half2float(wv[i]) * nv : nv);
                    }
                    *reinterpret_cast<uint4*>(p.normed + (size_t)tok * H + c0) = *reinterpret_cast<const uint4*>(o);
                }
            }
            trace(10);
        }
    }

    // ================================================== end ===================================================
    if (dead) {
        // waits were cut short: give this CTA's copies in flight time to land before its shared memory is released
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    __syncthreads();
    if (is_stream) trace(15);
    if (tid == 0) {
        __threadfence();
        const int old = atomicAdd(flags + FL_DONE, 1);
        if (old == G - 1) {
            // every CTA is past its last wait: the counters go back to zero for the next call
            if (p.trace)
                for (int i = 0; i < FL_COUNT && i < 256; ++i) g_fused_trace[256 * kFTraceSlots + i] = (unsigned long long)flags[i];
            for (int i = 0; i < FL_COUNT; ++i) flags[i] = 0;
            __threadfence();
        }
    }
}

}  // namespace glq
