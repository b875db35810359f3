// MoE block forward on the device: routing plan, expert matmuls through glq_grouped_matmul, combine.
// Everything is enqueued on one stream with launch shapes that depend only on (desc, n_tokens), so
// the call is capturable into a CUDA graph; nothing is read back to the host.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "glq_common.cuh"
#include "moe_fused.cuh"

using namespace glq;

// error word of this translation unit (the fused kernel's timed-out waits), merged by glq_debug_error
int glq_moe_error_words(unsigned long long* out4, int clear) {
    if (cudaMemcpyFromSymbol(out4, g_glq_err, 4 * sizeof(unsigned long long)) != cudaSuccess) return GLQ_ERR_CUDA;
    if (clear) {
        unsigned long long z[4] = {0, 0, 0, 0};
        if (cudaMemcpyToSymbol(g_glq_err, z, sizeof(z)) != cudaSuccess) return GLQ_ERR_CUDA;
    }
    return GLQ_OK;
}

namespace {

inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }
inline bool share_sm() {
    static const bool v = std::getenv("GLQ_NO_SHARE_SM") == nullptr;
    return v;
}
inline bool no_dependent_launch() {
    static const bool v = std::getenv("GLQ_NO_PDL") != nullptr;
    return v;
}

// ---- workspace carve-up ---------------------------------------------------------------------------
struct MoeLayout {
    size_t logits, sel, wts, active, n_active, slot_count, slot_offset, entry_row, entry_scale, tok_entries;
    size_t active2, n_active2, slot_count2, slot_offset2;   // gate and up x.U as one launch: 2E slots
    size_t plan_blk;                                        // per-block expert counts of the many-token plan
    size_t a_gu, h, b, yd, a_sg, a_su, hs, bs, ysh, xr, hr, hsr, mm, mm2;
    size_t total, mm_bytes, mm_counters;
};

// Rows per problem slot of the routed products.  With 9 or more tokens but few rows per expert on
// average, an expert's entries are cut into slots of at most 8 rows (consecutive entries, so nothing
// else changes): every routed product then stays on the integer streaming path in one launch, and the
// repeated reads of an expert's weights are served by L2.  0: one slot per expert.
inline int moe_chunk(const glq_moe_desc_t* d, int n) {
    static const bool off = std::getenv("GLQ_NO_CHUNK") != nullptr;
    const long long nk = (long long)n * d->top_k;
    const bool affine = d->fmt == GLQ_FMT_Q2 || d->fmt == GLQ_FMT_Q4;
    return (!off && affine && n > 8 && nk <= 24ll * d->E) ? 8 : 0;
}
inline int moe_slots(const glq_moe_desc_t* d, int n) {
    const long long nk = (long long)n * d->top_k;
    const int chunk = moe_chunk(d, n);
    return (int)std::min<long long>(nk, chunk ? d->E + nk / chunk : d->E);
}

void set_mm(glq_mm_args_t* m, int fmt, int group_size, int epi, int P, int rows, int N, int K, int rank,
            int total_rows = 0) {
    std::memset(m, 0, sizeof(*m));
    m->fmt = fmt;
    m->group_size = group_size;
    m->epilogue = epi;
    m->n_problems = P;
    m->max_rows = rows;
    m->rows_stride = rows;
    m->N = N;
    m->K = K;
    m->rank = rank;
    m->total_rows = total_rows;   // entries of all problems together (0: P * rows)
}

MoeLayout moe_layout(const glq_moe_desc_t* d, int n) {
    MoeLayout L{};
    const size_t nk = (size_t)n * d->top_k, R = (size_t)std::max(d->rank, 16);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += up256(bytes);
        return o;
    };
    L.logits = take((size_t)n * d->dense0_rows * 2);
    L.sel = take(nk * 4);
    L.wts = take(nk * 2);
    const size_t PS = (size_t)moe_slots(d, n);
    L.active = take(PS * 4);
    L.n_active = take(4);
    L.slot_count = take(PS * 4);
    L.slot_offset = take(PS * 4);
    L.entry_row = take(2 * nk * 4);   // second copy for the up half of the x.U launch
    L.entry_scale = take(nk * 2);
    L.tok_entries = take(nk * 4);
    L.active2 = take(2 * PS * 4);
    L.n_active2 = take(4);
    L.slot_count2 = take(2 * PS * 4);
    L.slot_offset2 = take(2 * PS * 4);
    L.plan_blk = take(((nk + 511) / 512) * (size_t)d->E * 4);
    L.a_gu = take(2 * nk * R * 2);
    L.h = take(nk * d->I * 2);
    L.b = take(nk * R * 2);
    L.yd = take(nk * d->H * 2);
    if (d->I_shared > 0) {
        L.a_sg = take((size_t)n * R * 2);
        L.a_su = take((size_t)n * R * 2);
        L.hs = take((size_t)n * d->I_shared * 2);
        L.bs = take((size_t)n * R * 2);
        L.ysh = take((size_t)n * d->H * 2);
    }
    if (d->rot_in || d->rht_in) L.xr = take((size_t)n * d->H * 2);
    if (d->rot_mid || d->rht_mid) L.hr = take(nk * d->I * 2);
    if ((d->sh_rot_mid || d->sh_rht_mid) && d->I_shared > 0) L.hsr = take((size_t)n * d->I_shared * 2);
    // scratch / counters of the matmul calls: they run one after the other, so they share
    const int P = moe_slots(d, n);
    const int rows = moe_chunk(d, n) ? std::min(n, moe_chunk(d, n)) : n;   // rows per routed slot
    glq_mm_args_t m;
    size_t wb = 0, wc = 0;
    auto acc = [&]() {
        wb = std::max(wb, glq_mm_workspace_bytes(&m));
        wc = std::max(wc, glq_mm_counters(&m));
    };
    set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 1, n, d->dense0_rows, d->H, 0); acc();
    if (d->rot_in) { set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 1, n, d->H, d->H, 0); acc(); }
    if (d->rot_mid) { set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 1, (int)nk, d->I, d->I, 0); acc(); }
    if (d->sh_rot_mid && d->I_shared > 0) { set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 1, n, d->I_shared, d->I_shared, 0); acc(); }
    if (d->rank > 0) {
        set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 2 * P, rows, d->rank, d->H, 0, (int)(2 * nk)); acc();
        set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, P, rows, d->rank, d->I, 0, (int)nk); acc();
    }
    set_mm(&m, d->fmt, d->group_size, GLQ_EPI_SWIGLU, P, rows, d->I, d->H, d->rank, (int)nk); acc();
    set_mm(&m, d->fmt, d->group_size, GLQ_EPI_LINEAR, P, rows, d->H, d->I, d->rank, (int)nk); acc();
    if (d->I_shared > 0) {
        if (d->rank > 0) {
            set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 1, n, d->rank, d->H, 0); acc();
            set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 1, n, d->rank, d->I_shared, 0); acc();
        }
        set_mm(&m, d->fmt, d->group_size, GLQ_EPI_SWIGLU, 1, n, d->I_shared, d->H, d->rank); acc();
        set_mm(&m, d->fmt, d->group_size, GLQ_EPI_LINEAR, 1, n, d->H, d->I_shared, d->rank); acc();
    }
    L.mm_bytes = up256(wb);
    L.mm_counters = wc;
    L.mm = take(L.mm_bytes);
    L.mm2 = take(L.mm_bytes);   // the shared expert's branch may run concurrently on a second stream
    L.total = off;
    return L;
}

// ---- routing plan -----------------------------------------------------------------------------------
// One CTA.  Phase A, warp per token: softmax over the fp16 router logits in fp32, top-k (ties to
// the lower expert index), optional renormalisation, weights rounded to fp16.  Phase B, warp per
// expert: entry counts, offsets and the expert's entry list in token order (ballot scans:
// deterministic), and the compacted list of live experts.
// Routing of one token by one warp: soft-max over the experts (lanes over experts, E <= 256), top-k by
// repeated arg-max (first maximum wins), optional renormalisation, fp16 weights.
__device__ __forceinline__ void route_token(int t, int lane, const __half* __restrict__ logits, int ldl, int E, int k, int renorm,
                                            int* __restrict__ sel, __half* __restrict__ wts, __half* __restrict__ logits_out,
                                            int* __restrict__ sel_out, __half* __restrict__ wts_out) {
    const __half* row = logits + (size_t)t * ldl;
    float lv[8], pv[8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        lv[i] = e < E ? __half2float(row[e]) : -INFINITY;
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
    // a probability that is not a number (non-finite hidden state) counts as zero: the top-k below then
    // still selects k distinct experts and no index leaves the tables
    for (int i = 0; i < 8; ++i) {
        const float pr = pv[i] / sum;
        pv[i] = (lane + 32 * i) < E ? (pr >= 0.f ? pr : 0.f) : -1.f;
    }
    float wk[16];
    int ek[16];
    float wsum = 0.f;
    for (int s = 0; s < k; ++s) {
        float best = -1.f;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (pv[i] > best) {   // increasing i = increasing expert index: first maximum wins
                best = pv[i];
                be = lane + 32 * i;
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ob > best || (ob == best && oe < be)) {
                best = ob;
                be = oe;
            }
        }
        wk[s] = best;
        ek[s] = be;
        wsum += best;
        if ((be & 31) == lane) pv[be >> 5] = -1.f;   // taken
    }
    if (lane == 0) {
        for (int s = 0; s < k; ++s) {
            const float wv = renorm ? wk[s] / wsum : wk[s];
            const __half wh = __float2half_rn(wv);
            sel[t * k + s] = ek[s];
            wts[t * k + s] = wh;
            if (sel_out) sel_out[t * k + s] = ek[s];
            if (wts_out) wts_out[t * k + s] = wh;
        }
    }
    if (logits_out)
        for (int e = lane; e < E; e += 32) logits_out[(size_t)t * E + e] = row[e];
}

// Warp 0 of a CTA: exclusive prefix of the per-expert counts in sm_cnt (entry offsets are global: every rank
// numbers the entries alike) into sm_off, and the compacted lists of the live experts this rank holds.
__device__ __forceinline__ void plan_lists(int lane, const int* sm_cnt, int* sm_off, int E, int nk, int chunk, int ep_rank,
                                           int ep_world, int* __restrict__ active, int* __restrict__ n_active,
                                           int* __restrict__ slot_count, int* __restrict__ slot_offset,
                                           int* __restrict__ active2, int* __restrict__ n_active2,
                                           int* __restrict__ slot_count2, int* __restrict__ slot_offset2) {
    int base = 0, j = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
        const int e = e0 + lane;
        const int c = e < E ? sm_cnt[e] : 0;
        int v = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int tv = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += tv;
        }
        const int off = base + v - c;
        if (e < E) sm_off[e] = off;
        const bool act = e < E && c > 0 && e % ep_world == ep_rank;
        // slots of this expert: one, or ceil(c / chunk) of at most `chunk` consecutive entries each
        const int ns = act ? (chunk > 0 ? (c + chunk - 1) / chunk : 1) : 0;
        int sv = ns;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int tv = __shfl_up_sync(0xffffffffu, sv, o);
            if (lane >= o) sv += tv;
        }
        for (int i = 0; i < ns; ++i) {
            const int pos = j + sv - ns + i;
            const int cc = chunk > 0 ? min(chunk, c - i * chunk) : c;
            const int oo = off + (chunk > 0 ? i * chunk : 0);
            active[pos] = e;
            slot_count[pos] = cc;
            slot_offset[pos] = oo;
            // the same lists twice, for gate (table entry e, entries 0..nk) and up (entry E+e, entries nk..2nk)
            active2[pos] = e;
            slot_count2[pos] = cc;
            slot_offset2[pos] = oo;
        }
        j += __shfl_sync(0xffffffffu, sv, 31);
        base += __shfl_sync(0xffffffffu, v, 31);
    }
    __syncwarp();
    for (int i = lane; i < j; i += 32) {
        active2[j + i] = E + active[i];
        slot_count2[j + i] = slot_count[i];
        slot_offset2[j + i] = nk + slot_offset[i];
    }
    if (lane == 0) {
        *n_active = j;
        *n_active2 = 2 * j;
    }
}

__global__ void __launch_bounds__(1024) moe_plan_kernel(const __half* __restrict__ logits, int ldl, int n, int E, int k,
                                                        int renorm, int* __restrict__ sel, __half* __restrict__ wts,
                                                        int* __restrict__ active, int* __restrict__ n_active,
                                                        int* __restrict__ slot_count, int* __restrict__ slot_offset,
                                                        int* __restrict__ entry_row, __half* __restrict__ entry_scale,
                                                        int* __restrict__ tok_entries, __half* __restrict__ logits_out,
                                                        int* __restrict__ sel_out, __half* __restrict__ wts_out,
                                                        int* __restrict__ active2, int* __restrict__ n_active2,
                                                        int* __restrict__ slot_count2, int* __restrict__ slot_offset2,
                                                        int ep_rank, int ep_world, const int* __restrict__ sel_in,
                                                        const __half* __restrict__ wts_in, int chunk) {
    extern __shared__ int sm_cnt[];  // [E] counts, then [E] offsets
    int* sm_off = sm_cnt + E;
    asm volatile("griddepcontrol.wait;" ::: "memory");              // no-ops for a plain launch
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // Phase A: one warp per token, lanes over experts (E <= 256)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (sel_in) {
        // routing decided by the caller: copy it; an index outside [0, E) marks a dropped slot
        for (int i = threadIdx.x; i < n * k; i += blockDim.x) {
            const int e = sel_in[i];
            sel[i] = e;
            wts[i] = wts_in[i];
            if (e < 0 || e >= E) tok_entries[i] = -1;
        }
    }
    for (int t = warp; t < n && !sel_in; t += nwarps)
        route_token(t, lane, logits, ldl, E, k, renorm, sel, wts, logits_out, sel_out, wts_out);
    __syncthreads();
    const int nk = n * k;
    const unsigned lt = (1u << lane) - 1u;
    // Phase B1: entries per expert, one warp per expert (ballot counts: no atomics, any order gives the same sum)
    for (int e = warp; e < E; e += nwarps) {
        int c = 0;
        for (int i0 = 0; i0 < nk; i0 += 32) {
            const int i = i0 + lane;
            c += __popc(__ballot_sync(0xffffffffu, i < nk && sel[i] == e));
        }
        if (lane == 0) sm_cnt[e] = c;
    }
    __syncthreads();
    // Phase B2, warp 0: exclusive prefix of the counts (entry offsets are global: every rank numbers the
    // entries alike) and the compacted list of live experts this rank holds (e mod world == rank)
    if (warp == 0)
        plan_lists(lane, sm_cnt, sm_off, E, nk, chunk, ep_rank, ep_world, active, n_active, slot_count, slot_offset, active2,
                   n_active2, slot_count2, slot_offset2);
    __syncthreads();
    // Phase B3: each expert's entries in token order, one warp per expert
    for (int e = warp; e < E; e += nwarps) {
        if (sm_cnt[e] == 0) continue;
        int pos = sm_off[e];
        for (int i0 = 0; i0 < nk; i0 += 32) {
            const int i = i0 + lane;
            const bool hit = i < nk && sel[i] == e;
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const int q = pos + __popc(m & lt);
                entry_row[q] = i / k;
                entry_row[nk + q] = i / k;
                entry_scale[q] = wts[i];
                tok_entries[i] = q;
            }
            pos += __popc(m);
        }
    }
}

// ---- the same plan for many tokens, spread over the SMs -----------------------------------------------------
// moe_plan_kernel is one CTA (the decode step wants one short launch); with thousands of tokens its scans over
// all entries per expert take a millisecond.  Four small launches give the identical plan: (a) one warp per
// token routes; (b) one warp per block of kPlanChunk consecutive entries counts its entries per expert;
// (c) one CTA sums the counts, builds the lists (plan_lists) and turns the per-block counts into per-block
// bases; (d) every block scatters its entries in entry order from its bases -- a stable counting sort, so each
// expert's entries come out in token order exactly as in the one-CTA kernel.
constexpr int kPlanChunk = 512;
constexpr long long kPlanParallelFrom = 2048;   // entries (tokens x top-k) from which the plan runs as four launches

__global__ void __launch_bounds__(256) moe_route_kernel(const __half* __restrict__ logits, int ldl, int n, int E, int k, int renorm,
                                                        int* __restrict__ sel, __half* __restrict__ wts,
                                                        int* __restrict__ tok_entries, __half* __restrict__ logits_out,
                                                        int* __restrict__ sel_out, __half* __restrict__ wts_out,
                                                        const int* __restrict__ sel_in, const __half* __restrict__ wts_in) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (sel_in) {   // routing decided by the caller: copy it; an index outside [0, E) marks a dropped slot
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n * k; i += gridDim.x * blockDim.x) {
            const int e = sel_in[i];
            sel[i] = e;
            wts[i] = wts_in[i];
            if (e < 0 || e >= E) tok_entries[i] = -1;
        }
        return;
    }
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t < n) route_token(t, lane, logits, ldl, E, k, renorm, sel, wts, logits_out, sel_out, wts_out);
}

// one warp per block: blk[b][e] = entries of expert e among the block's kPlanChunk entries
__global__ void __launch_bounds__(32) moe_plan_count_kernel(const int* __restrict__ sel, int nk, int E, int* __restrict__ blk) {
    extern __shared__ int sm_c[];
    const int lane = threadIdx.x, b = blockIdx.x;
    for (int e = lane; e < E; e += 32) sm_c[e] = 0;
    __syncwarp();
    const int i_end = min(nk, (b + 1) * kPlanChunk);
    for (int i0 = b * kPlanChunk; i0 < i_end; i0 += 32) {
        const int i = i0 + lane;
        const int e = i < i_end ? sel[i] : -1;
        const bool valid = e >= 0 && e < E;
        const unsigned m = __match_any_sync(0xffffffffu, valid ? e : E + lane);
        if (valid && lane == __ffs(m) - 1) sm_c[e] += __popc(m);
        __syncwarp();
    }
    for (int e = lane; e < E; e += 32) blk[(size_t)b * E + e] = sm_c[e];
}

__global__ void __launch_bounds__(1024) moe_plan_lists_kernel(int* __restrict__ blk, int nb, int nk, int E, int chunk, int ep_rank,
                                                              int ep_world, int* __restrict__ active, int* __restrict__ n_active,
                                                              int* __restrict__ slot_count, int* __restrict__ slot_offset,
                                                              int* __restrict__ active2, int* __restrict__ n_active2,
                                                              int* __restrict__ slot_count2, int* __restrict__ slot_offset2) {
    extern __shared__ int sm_cnt[];  // [E] counts, then [E] offsets
    int* sm_off = sm_cnt + E;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int c = 0;
        for (int b = 0; b < nb; ++b) c += blk[(size_t)b * E + e];
        sm_cnt[e] = c;
    }
    __syncthreads();
    if (warp == 0)
        plan_lists(lane, sm_cnt, sm_off, E, nk, chunk, ep_rank, ep_world, active, n_active, slot_count, slot_offset, active2,
                   n_active2, slot_count2, slot_offset2);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {   // counts -> first entry number of (block, expert)
        int run = sm_off[e];
        for (int b = 0; b < nb; ++b) {
            const int c = blk[(size_t)b * E + e];
            blk[(size_t)b * E + e] = run;
            run += c;
        }
    }
}

__global__ void __launch_bounds__(32) moe_plan_scatter_kernel(const int* __restrict__ sel, const __half* __restrict__ wts, int nk,
                                                              int E, int k, const int* __restrict__ blk,
                                                              int* __restrict__ entry_row, __half* __restrict__ entry_scale,
                                                              int* __restrict__ tok_entries) {
    extern __shared__ int sm_b[];
    const int lane = threadIdx.x, b = blockIdx.x;
    const unsigned lt = (1u << lane) - 1u;
    for (int e = lane; e < E; e += 32) sm_b[e] = blk[(size_t)b * E + e];
    __syncwarp();
    const int i_end = min(nk, (b + 1) * kPlanChunk);
    for (int i0 = b * kPlanChunk; i0 < i_end; i0 += 32) {
        const int i = i0 + lane;
        const int e = i < i_end ? sel[i] : -1;
        const bool valid = e >= 0 && e < E;
        const unsigned m = __match_any_sync(0xffffffffu, valid ? e : E + lane);
        if (valid) {
            const int q = sm_b[e] + __popc(m & lt);
            entry_row[q] = i / k;
            entry_row[nk + q] = i / k;
            entry_scale[q] = wts[i];
            tok_entries[i] = q;
        }
        __syncwarp();
        if (valid && lane == __ffs(m) - 1) sm_b[e] += __popc(m);
        __syncwarp();
    }
}

// ---- exchange over peer memory ---------------------------------------------------------------------------
// One CTA.  Step e = *epoch + 1 uses half (e & 1) of every rank's exchange buffer.  The rows of this rank's
// slots (the plan's active list holds only its own experts) go from the local staging buffer to the same
// rows of every rank's buffer, this rank's included, as 16-byte stores; after a system-wide fence the step
// number is published in word [rank] of every rank's flags, and the CTA waits until its own flag words
// all show step e.  The wait is bounded by the global timer; when it runs out *error is set and the
// kernel returns (the step's result is then incomplete, the context stays usable).
__global__ void __launch_bounds__(1024) moe_exchange_kernel(const __half* __restrict__ staged, const int* __restrict__ n_active,
                                                            const int* __restrict__ slot_count,
                                                            const int* __restrict__ slot_offset, int n_entries, int H,
                                                            int rank, int world, void* const* __restrict__ bufs,
                                                            int* const* __restrict__ flags, int* epoch, int* error,
                                                            size_t half_elems, unsigned long long limit_ns) {
    __shared__ int s_step;
    if (threadIdx.x == 0) s_step = *epoch + 1;
    __syncthreads();
    const int step = s_step;
    const size_t half = (size_t)(step & 1) * half_elems;
    const int nact = min(*n_active, n_entries);
    const int vec_per_row = H / 8;
    for (int s = 0; s < nact; ++s) {
        const int off = slot_offset[s], cnt = slot_count[s];
        if (off < 0 || cnt <= 0 || off + cnt > n_entries) continue;
        const int nvec = cnt * vec_per_row;
        const uint4* src = reinterpret_cast<const uint4*>(staged + (size_t)off * H);
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            const uint4 v = src[i];
            for (int p = 0; p < world; ++p)
                reinterpret_cast<uint4*>(reinterpret_cast<__half*>(bufs[p]) + half + (size_t)off * H)[i] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) {
        int* theirs = flags[threadIdx.x] + rank;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(step) : "memory");
        const int* mine = flags[rank] + threadIdx.x;
        const unsigned long long t0 = global_ns();
        for (;;) {
            int seen;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if (seen - step >= 0) break;
            if (global_ns() - t0 > limit_ns) {
                atomicCAS(error, 0, step);      // the first wait that ran out stays on record
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) *epoch = step;
}

// ---- combine ------------------------------------------------------------------------------------------
// out[t] = sum over the token's experts of (already weighted, fp16) down outputs, accumulated in fp16
// in slot order or in expert order, + sigmoid(shared gate) * shared expert output.  8 columns/thread.
__global__ void moe_combine_kernel(const __half* __restrict__ yd, const int* __restrict__ tok_entries, int n_entries,
                                   const int* __restrict__ sel, int k, int H, int by_expert,
                                   const __half* __restrict__ ysh, const __half* __restrict__ logits, int ldl,
                                   int gate_col, __half* __restrict__ out, const int* __restrict__ epoch,
                                   size_t half_elems) {
    asm volatile("griddepcontrol.wait;" ::: "memory");              // no-op for a plain launch
    if (epoch) yd += (size_t)(*epoch & 1) * half_elems;            // the half the last exchange filled
    const int t = blockIdx.y;
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c0 >= H) return;
    int order[16];
    for (int s = 0; s < k; ++s) order[s] = s;
    if (by_expert) {
        for (int i = 1; i < k; ++i) {
            const int v = order[i];
            const int ev = sel[t * k + v];
            int j = i - 1;
            while (j >= 0 && sel[t * k + order[j]] > ev) {
                order[j + 1] = order[j];
                --j;
            }
            order[j + 1] = v;
        }
    }
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int s = 0; s < k; ++s) {
        const int entry = tok_entries[t * k + order[s]];
        if (entry < 0 || entry >= n_entries) continue;     // dropped slot
        __align__(16) __half v[8];
        *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(yd + (size_t)entry * H + c0);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = round16(acc[i] + __half2float(v[i]));
    }
    if (ysh) {
        const float gate = gate_col >= 0 ? sigmoid16(__half2float(logits[(size_t)t * ldl + gate_col])) : 1.f;
        __align__(16) __half v[8];
        *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(ysh + (size_t)t * H + c0);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = round16(acc[i] + round16(gate * __half2float(v[i])));
    }
    __align__(16) __half o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = __float2half_rn(acc[i]);
    *reinterpret_cast<uint4*>(out + (size_t)t * H + c0) = *reinterpret_cast<const uint4*>(o);
}

// Combine with the decoder's next steps folded in: out = residual + block output (when a residual is given),
// and normed = rms_norm(out) * weight.  One CTA per token, 8 columns per thread and step, up to 4 steps
// (H <= 8192); the sum of squares goes through shared memory.
__global__ void __launch_bounds__(256) moe_combine_norm_kernel(const __half* __restrict__ yd, const int* __restrict__ tok_entries,
                                                               int n_entries, const int* __restrict__ sel, int k, int H,
                                                               int by_expert, const __half* __restrict__ ysh,
                                                               const __half* __restrict__ logits, int ldl, int gate_col,
                                                               const __half* __restrict__ residual,
                                                               const __half* __restrict__ norm_w, float eps,
                                                               __half* __restrict__ out, __half* __restrict__ normed,
                                                               const int* __restrict__ epoch, size_t half_elems) {
    const int t = blockIdx.x;
    if (epoch) yd += (size_t)(*epoch & 1) * half_elems;
    int order[16];
    for (int s = 0; s < k; ++s) order[s] = s;
    if (by_expert) {
        for (int i = 1; i < k; ++i) {
            const int v = order[i];
            const int ev = sel[t * k + v];
            int j = i - 1;
            while (j >= 0 && sel[t * k + order[j]] > ev) {
                order[j + 1] = order[j];
                --j;
            }
            order[j + 1] = v;
        }
    }
    const float gate = (ysh && gate_col >= 0) ? sigmoid16(__half2float(logits[(size_t)t * ldl + gate_col])) : 1.f;
    float val[4][8];
    float ss = 0.f;
#pragma unroll
    for (int step = 0; step < 4; ++step) {
        const int c0 = (step * 256 + threadIdx.x) * 8;
        if (c0 >= H) continue;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        for (int s = 0; s < k; ++s) {
            const int entry = tok_entries[t * k + order[s]];
            if (entry < 0 || entry >= n_entries) continue;
            __align__(16) __half v[8];
            *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(yd + (size_t)entry * H + c0);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = round16(acc[i] + __half2float(v[i]));
        }
        if (ysh) {
            __align__(16) __half v[8];
            *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(ysh + (size_t)t * H + c0);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = round16(acc[i] + round16(gate * __half2float(v[i])));
        }
        if (residual) {
            __align__(16) __half v[8];
            *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(residual + (size_t)t * H + c0);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = round16(__half2float(v[i]) + acc[i]);
        }
        __align__(16) __half o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            o[i] = __float2half_rn(acc[i]);
            val[step][i] = acc[i];
            ss += acc[i] * acc[i];
        }
        *reinterpret_cast<uint4*>(out + (size_t)t * H + c0) = *reinterpret_cast<const uint4*>(o);
    }
    __shared__ float red[8];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float r = rsqrtf(tot / H + eps);
#pragma unroll
    for (int step = 0; step < 4; ++step) {
        const int c0 = (step * 256 + threadIdx.x) * 8;
        if (c0 >= H) continue;
        __align__(16) __half o[8], wv[8];
        if (norm_w) *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(norm_w + c0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float nv = val[step][i] * r;
            o[i] = __float2half_rn(norm_w ? __half2float(wv[i]) * nv : nv);
        }
        *reinterpret_cast<uint4*>(normed + (size_t)t * H + c0) = *reinterpret_cast<const uint4*>(o);
    }
}

// ---- the fused decode kernel: eligibility, geometry, launch ---------------------------------------------------
inline bool fused_disabled() {
    static const bool v = std::getenv("GLQ_NO_FUSED_MOE") != nullptr;
    return v;
}
inline int fused_sms() {
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (sms[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        sms[dev] = v;
    }
    return sms[dev];
}
inline int cdiv_i(int a, int b) { return (a + b - 1) / b; }

// true when the block with n tokens runs as the one persistent kernel; fills the launch parameters that do not
// depend on the call's buffers
bool plan_fused(const glq_moe_desc_t* d, int n, FusedParams* out, size_t* smem_bytes) {
    if (fused_disabled() || n < 1 || n > kFRows) return false;
    if (d->fmt != GLQ_FMT_Q2 && d->fmt != GLQ_FMT_Q4) return false;
    if (!d->router_rm || !d->router_t) return false;
    if (d->rank < 0 || d->rank % 16 != 0 || (d->rank > 0 && (!d->ut_rm_gate_up || !d->ut_rm_down))) return false;
    if (d->top_k > 16 || n * d->top_k > kFMaxEntries || d->E > 256) return false;
    if (d->H % 8 != 0 || d->I % 8 != 0 || d->I_shared % 8 != 0) return false;
    const int KB = d->fmt == GLQ_FMT_Q2 ? 128 : 64;
    if (d->group_size <= 0 || d->group_size % KB != 0) return false;
    const int gb = d->group_size / KB;
    const bool shared = d->I_shared > 0 && d->sh_gate_up.codes != nullptr;
    const int R = d->rank;
    int sh_rank = 0;
    if (shared) {
        if (!d->sh_down.codes) return false;
        sh_rank = d->sh_gate_up.sv ? d->sh_gate_up.rank : 0;
        if (sh_rank > 0) {
            // the shared expert's x.U must come out of the router product, and its h.U needs the row-major U^T
            if (sh_rank != R || d->sh_a_row <= 0 || d->dense0_rows < d->sh_a_row + 2 * R || !d->sh_ut_rm_down ||
                !d->sh_down.sv || d->sh_down.rank != R || d->dense0_rows % 8 != 0)
                return false;
        } else if (d->sh_down.sv && d->sh_down.rank > 0) {
            return false;
        }
    }
    FusedParams P{};
    const int sms = fused_sms();
    P.n = n;
    P.H = d->H;
    P.I = d->I;
    P.Is = shared ? d->I_shared : 0;
    P.E = d->E;
    P.k = d->top_k;
    P.R = R;
    P.renorm = d->norm_topk_prob;
    P.ldl = d->dense0_rows;
    P.dense_rows = d->dense0_rows;
    P.sh_a_row = d->sh_a_row;
    // CTAs of the shared expert's chain: in proportion to its bytes, between an eighth and a half of the SMs
    const int est = n * d->top_k;
    int gs = 0;
    if (shared) {
        const double fs = (double)d->I_shared / ((double)d->I_shared + (double)est * d->I);
        // (the shared chain has slack -- nothing in it waits for the routing -- so it gets half its share)
        static const char* gse = std::getenv("GLQ_FUSED_GSHARE");
        gs = (int)((gse ? std::atof(gse) : 0.5) * fs * sms + 0.5);
        gs = std::max(sms / 8, std::min(sms / 2, gs));
        gs = std::max(gs, kFRows);
    }
    if (sms - gs < kFRows) return false;        // the combine needs one CTA per token
    P.g_shared = gs;
    int max_nkb = 0;
    int base[2] = {0, 0};      // rotation of the iteration -> CTA map, per subset
    auto set_phase = [&](int idx, bool live, int N, int K, int swiglu, int rank, int problems) {
        FusedPhase& ph = P.ph[idx];
        const int sub = (idx & 1) ? 1 : 0, sub_G = sub ? sms - gs : std::max(gs, 1);
        ph.live = live ? 1 : 0;
        ph.N = N;
        ph.K = K;
        ph.swiglu = swiglu;
        ph.rank = rank;
        ph.ns = rank > 0 ? cdiv_i(rank, 64) : 0;
        ph.nkb = cdiv_i(std::max(K, 1), KB);
        const int units = cdiv_i(ph.nkb, gb);
        const int ntiles = cdiv_i(std::max(N, 1), kRowTile);
        ph.npairs = swiglu ? ntiles : cdiv_i(ntiles, 2);
        // k splits per pair (1, 2 or 4 adjacent warps): the fewest rounds of iterations over the subset's CTAs, then
        // the shortest items (every round ends in an epilogue with its own chain of waits)
        int sk = 1;
        long best = -1;
        static const char* ske = std::getenv("GLQ_FUSED_SK");
        const int sk_lo = ske ? std::atoi(ske) : 1;
        for (int c = sk_lo; c <= 4; c *= 2) {
            if (c > sk_lo && units < c) break;
            const long rounds = cdiv_i(problems * cdiv_i(ph.npairs, kFSW / c), sub_G);
            const long cost = rounds * 1000 + cdiv_i(units, c);
            if (best < 0 || cost < best) best = cost, sk = c;
        }
        ph.sk = sk;
        ph.sk_log2 = sk == 1 ? 0 : (sk == 2 ? 1 : 2);
        ph.kb_per_split = cdiv_i(units, sk) * gb;
        ph.ppi = kFSW / sk;
        ph.ipp = cdiv_i(ph.npairs, ph.ppi);
        ph.cta_base = base[sub] % sub_G;
        if (live) {
            base[sub] += problems * ph.ipp;
            max_nkb = std::max(max_nkb, ph.nkb);
        }
    };
    set_phase(0, shared, d->I_shared, d->H, 1, sh_rank, 1);
    set_phase(1, true, d->I, d->H, 1, R, est);
    set_phase(2, shared, d->H, d->I_shared, 0, sh_rank, 1);
    set_phase(3, true, d->H, d->I, 0, R, est);
    P.ph[0].w = d->sh_gate_up;
    P.ph[2].w = d->sh_down;
    P.ph[1].table = d->gate_up;
    P.ph[3].table = d->down;
    // shared memory
    const int pieces = d->fmt == GLQ_FMT_Q2 ? 2 : 1;
    size_t off = (size_t)kFW * kFMaxStages * 8;
    off = (off + 127) / 128 * 128;
    P.off_act = (int)off;
    off += (size_t)max_nkb * pieces * 512;
    P.off_ox = (int)off;
    off += (size_t)max_nkb * kFRows * 8;
    off = (off + 15) / 16 * 16;
    P.off_red = (int)off;
    off += (size_t)2 * kFSW * 2 * 32 * sizeof(float2);     // k-split sums (two parities)
    P.off_prob = (int)off;
    off += (size_t)kFRows * (256 + 16) * sizeof(float);    // the routing's probabilities
    off = (off + 15) / 16 * 16;
    P.off_plan = (int)off;
    off += sizeof(FusedPlan);
    off = (off + 15) / 16 * 16;
    P.off_tab = (int)off;
    off += (size_t)d->E * sizeof(ExpertPtrs);
    off = (off + 127) / 128 * 128;
    P.off_ring = (int)off;
    P.stage_bytes = std::max(kStreamCB * 2 * block_bytes_of(d->fmt), 4096);
    const size_t cap = 227 * 1024;
    if (off + (size_t)kFSW * P.stage_bytes > cap) return false;
    P.stages = (int)std::min<size_t>((cap - off) / ((size_t)kFSW * P.stage_bytes), 3);
    // long reductions (an intermediate size in the ten thousands) leave room for one stage only: without a second
    // one nothing overlaps the copies, and the separate launches with their deeper rings stream better
    if (P.stages < 2) return false;
    *smem_bytes = off + (size_t)kFSW * P.stages * P.stage_bytes;
    // dense warps sharing one row of the shared down projection's U^T: segments of at most 2048 channels
    P.s6_segs = 1;
    while (P.s6_segs < kFW - kFSW && P.Is / P.s6_segs > 2048 && P.Is % (16 * P.s6_segs) == 0) P.s6_segs *= 2;
    static const bool tr = std::getenv("GLQ_FUSED_TRACE") != nullptr;
    P.trace = tr ? 1 : 0;
    static const char* wl = std::getenv("GLQ_FUSED_WAIT_US");
    P.wait_ns = wl ? (unsigned long long)std::atoll(wl) * 1000ull : 4000000ull;
    *out = P;
    return true;
}

template <int FMT>
int launch_fused_t(const FusedParams& P, size_t smem, cudaStream_t st) {
    auto kern = moe_fused_kernel<FMT>;
    static size_t configured[64] = {0};
    static int resident[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return GLQ_ERR_CUDA;
    if (dev < 0 || dev >= 64) return GLQ_ERR_UNSUPPORTED;
    if (configured[dev] < smem) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return GLQ_ERR_CUDA;
        int nb = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, kFT, smem) != cudaSuccess) return GLQ_ERR_CUDA;
        resident[dev] = nb;
        configured[dev] = smem;
    }
    if (resident[dev] < 1) return GLQ_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(fused_sms());
    cfg.blockDim = dim3(kFT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeCooperative;      // all CTAs resident at once: they wait on one another
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, P) != cudaSuccess) return GLQ_ERR_CUDA;
    return GLQ_OK;
}

}  // namespace

extern "C" size_t glq_moe_workspace_bytes(const glq_moe_desc_t* d, int n_tokens) {
    if (!d || n_tokens <= 0) return 0;
    return moe_layout(d, n_tokens).total;
}
extern "C" size_t glq_moe_counters(const glq_moe_desc_t* d, int n_tokens) {
    if (!d || n_tokens <= 0) return 0;
    // the matmul launches' arrival counters (two concurrent branches), or the fused kernel's
    return std::max<size_t>(2 * moe_layout(d, n_tokens).mm_counters, (size_t)FL_COUNT);
}

// Diagnostic: with GLQ_FUSED_TRACE set in the environment, thread 0 of every CTA of the persistent kernel records
// the GPU's global timer (ns) after each step; this copies the stamps of the last launch, [CTA][16], to the host.
extern "C" int glq_moe_fused_trace(unsigned long long* out, int n_words) {
    if (!out || n_words <= 0 || n_words > 256 * kFTraceSlots + 256) return GLQ_ERR_ARG;
    return cudaMemcpyFromSymbol(out, g_fused_trace, (size_t)n_words * sizeof(unsigned long long)) == cudaSuccess
               ? GLQ_OK : GLQ_ERR_CUDA;
}

extern "C" int glq_moe_uses_fused_kernel(const glq_moe_desc_t* d, int n_tokens) {
    if (!d) return 0;
    FusedParams fp;
    size_t smem = 0;
    return plan_fused(d, n_tokens, &fp, &smem) ? 1 : 0;
}

extern "C" int glq_moe_forward(const glq_moe_desc_t* d, const void* x, int n, void* out, void* router_logits,
                               int32_t* sel_out, void* weight_out, void* workspace, size_t workspace_bytes,
                               int32_t* counters, size_t n_counters, void* stream, void* aux_stream, void* ev_fork,
                               void* ev_join) {
    return glq_moe_forward_ep(d, x, n, out, router_logits, sel_out, weight_out, workspace, workspace_bytes, counters,
                              n_counters, stream, aux_stream, ev_fork, ev_join, nullptr);
}

extern "C" int glq_moe_forward_ep(const glq_moe_desc_t* d, const void* x, int n, void* out, void* router_logits,
                                  int32_t* sel_out, void* weight_out, void* workspace, size_t workspace_bytes,
                                  int32_t* counters, size_t n_counters, void* stream, void* aux_stream, void* ev_fork,
                                  void* ev_join, const glq_moe_ep_t* ep) {
    if (!d || !x || !out || n < 0) return GLQ_ERR_ARG;
    const int ep_rank = ep ? ep->rank : 0, ep_world = ep ? ep->world : 1, phase = ep ? ep->phase : GLQ_MOE_PHASE_ALL;
    if (ep_world < 1 || ep_rank < 0 || ep_rank >= ep_world || phase < GLQ_MOE_PHASE_ALL || phase > GLQ_MOE_PHASE_EXCHANGE)
        return GLQ_ERR_ARG;
    const glq_ep_peers_t* px = ep ? ep->peers : nullptr;
    if (phase == GLQ_MOE_PHASE_EXCHANGE &&
        (!px || !px->entry_bufs || !px->flags || !px->epoch || !px->error || ep_world > 1024 ||
         px->half_elems < (size_t)n * d->top_k * d->H))
        return GLQ_ERR_ARG;
    if (phase == GLQ_MOE_PHASE_EXPERTS && px) return GLQ_ERR_ARG;     // the staging buffer is not exchanged
    const int* px_epoch = (phase == GLQ_MOE_PHASE_COMBINE && px) ? px->epoch : nullptr;
    const size_t px_half = px ? px->half_elems : 0;
    if (ep_world > 1 && (phase == GLQ_MOE_PHASE_ALL || !ep->entry_out)) return GLQ_ERR_ARG;   // the exchange is the caller's
    if (n == 0) return GLQ_OK;
    if (d->top_k < 1 || d->top_k > 16 || d->E < d->top_k || d->E > 256 || d->H % 8 != 0 || d->I % 8 != 0)
        return GLQ_ERR_UNSUPPORTED;
    const bool given = ep && ep->sel_in != nullptr;     // routing supplied by the caller: no router, no shared expert
    if (given && (!ep->weight_in || d->I_shared > 0 || router_logits)) return GLQ_ERR_ARG;
    if ((!given && !d->router_t) || !d->gate_up || !d->down) return GLQ_ERR_ARG;
    if (d->rank > 0 && (!d->ut_gate_up || !d->ut_down)) return GLQ_ERR_ARG;
    if (!given && (d->dense0_rows < d->router_rows || (d->sh_a_row > 0 && (d->sh_a_row % 16 != 0 || d->sh_a_row < d->router_rows))))
        return GLQ_ERR_ARG;
    const MoeLayout L = moe_layout(d, n);
    if (!workspace || workspace_bytes < L.total) return GLQ_ERR_WORKSPACE;
    if (L.mm_counters > 0 && (!counters || n_counters < 2 * L.mm_counters)) return GLQ_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return GLQ_ERR_ALIGN;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    char* ws = reinterpret_cast<char*>(workspace);
    const int k = d->top_k, nk = n * k, R = d->rank;
    const int P = moe_slots(d, n), chunk = moe_chunk(d, n);
    const int rows = chunk ? std::min(n, chunk) : n;     // rows per routed slot
    // per-entry down-projection outputs: in the workspace, or in the caller's exchange buffer
    char* p_yd = ep && ep->entry_out ? reinterpret_cast<char*>(ep->entry_out) : ws + L.yd;
    const bool shared = d->I_shared > 0 && d->sh_gate_up.codes != nullptr;

    auto p_logits = reinterpret_cast<__half*>(ws + L.logits);
    auto p_sel = reinterpret_cast<int*>(ws + L.sel);
    auto p_wts = reinterpret_cast<__half*>(ws + L.wts);
    auto p_active = reinterpret_cast<int*>(ws + L.active);
    auto p_nact = reinterpret_cast<int*>(ws + L.n_active);
    auto p_cnt = reinterpret_cast<int*>(ws + L.slot_count);
    auto p_off = reinterpret_cast<int*>(ws + L.slot_offset);
    auto p_erow = reinterpret_cast<int*>(ws + L.entry_row);
    auto p_escale = reinterpret_cast<__half*>(ws + L.entry_scale);
    auto p_tok = reinterpret_cast<int*>(ws + L.tok_entries);
    const int ldl = d->dense0_rows;

    if (phase == GLQ_MOE_PHASE_EXCHANGE) {
        moe_exchange_kernel<<<1, 1024, 0, st>>>(reinterpret_cast<const __half*>(p_yd), p_nact, p_cnt, p_off, nk, d->H,
                                                ep_rank, ep_world, px->entry_bufs, px->flags, px->epoch, px->error,
                                                px->half_elems, px->wait_limit_ns ? px->wait_limit_ns : 1000000000ull);
        return cudaGetLastError() == cudaSuccess ? GLQ_OK : GLQ_ERR_CUDA;
    }
    FusedParams fp;
    size_t fused_smem = 0;
    const bool fused = !given && plan_fused(d, n, &fp, &fused_smem) && counters != nullptr && n_counters >= (size_t)FL_COUNT;
    if (phase != GLQ_MOE_PHASE_COMBINE && fused) {
        // rows of remote experts' entries stay zero, so that summing the ranks' buffers is exact
        if (ep_world > 1 && !(ep->flags & GLQ_MOE_EP_NO_ZERO_FILL) &&
            cudaMemsetAsync(p_yd, 0, (size_t)nk * d->H * 2, st) != cudaSuccess)
            return GLQ_ERR_CUDA;
        fp.ep_rank = ep_rank;
        fp.ep_world = ep_world;
        fp.x = reinterpret_cast<const __half*>(x);
        fp.router_rm = reinterpret_cast<const __half*>(d->router_rm);
        fp.ut_rm_gate_up = d->ut_rm_gate_up;
        fp.ut_rm_down = d->ut_rm_down;
        fp.sh_ut_rm_down = reinterpret_cast<const __half*>(d->sh_ut_rm_down);
        fp.logits = p_logits;
        fp.sel = p_sel;
        fp.wts = p_wts;
        fp.active = p_active;
        fp.n_active = p_nact;
        fp.slot_count = p_cnt;
        fp.slot_offset = p_off;
        fp.entry_row = p_erow;
        fp.entry_scale = p_escale;
        fp.tok_entries = p_tok;
        fp.a_gate = reinterpret_cast<__half*>(ws + L.a_gu);
        fp.a_up = fp.a_gate + (size_t)nk * std::max(R, 16);
        fp.h = reinterpret_cast<__half*>(ws + L.h);
        fp.b = reinterpret_cast<__half*>(ws + L.b);
        fp.yd = reinterpret_cast<__half*>(p_yd);
        fp.hs = shared ? reinterpret_cast<__half*>(ws + L.hs) : nullptr;
        fp.bs = shared ? reinterpret_cast<__half*>(ws + L.bs) : nullptr;
        fp.ysh = shared ? reinterpret_cast<__half*>(ws + L.ysh) : nullptr;
        fp.logits_out = reinterpret_cast<__half*>(router_logits);
        fp.sel_out = sel_out;
        fp.wts_out = reinterpret_cast<__half*>(weight_out);
        fp.flags = counters;
        // one device, whole block: the combine runs inside the same launch
        if (phase == GLQ_MOE_PHASE_ALL && ep_world == 1 && d->H <= 8192 && !(ep && ep->residual && !ep->normed_out)) {
            fp.combine = 1;
            fp.by_expert = n > d->slot_order_max_tokens ? 1 : 0;
            fp.gate_col = d->router_rows > d->E ? d->E : -1;
            fp.out = reinterpret_cast<__half*>(out);
            if (ep && ep->normed_out) {
                fp.normed = reinterpret_cast<__half*>(ep->normed_out);
                fp.residual = reinterpret_cast<const __half*>(ep->residual);
                fp.norm_w = reinterpret_cast<const __half*>(ep->norm_weight);
                fp.norm_eps = ep->norm_eps;
            }
        }
        const int rc = d->fmt == GLQ_FMT_Q2 ? launch_fused_t<GLQ_FMT_Q2>(fp, fused_smem, st)
                                            : launch_fused_t<GLQ_FMT_Q4>(fp, fused_smem, st);
        if (rc != GLQ_OK) return rc;
        if (fp.combine) return GLQ_OK;
    } else if (phase != GLQ_MOE_PHASE_COMBINE) {
    glq_mm_args_t m;
    // the shared expert's chain runs on aux_stream (forked after the first dense product, joined before
    // the combine) when the caller provides a stream and two events; it has its own scratch and counters
    const bool forked = aux_stream != nullptr && ev_fork != nullptr && ev_join != nullptr;
    bool on_aux = false;
    // programmatic dependent launches: allowed when the previous operation on the stream was one of this
    // library's launches (not the first launch of the call, not after an event wait)
    bool after_kernel[2] = {false, false};
    auto finish = [&](glq_mm_args_t& mm) {
        // (chaining every launch this way, GLQ_MM_AFTER_KERNEL, measured no faster than plain launches
        // inside a graph: only the two x.U edges, whose consumers have real independent work, are used)
        if (!after_kernel[on_aux ? 1 : 0]) mm.flags &= ~GLQ_MM_A_FROM_PREVIOUS_LAUNCH;
        if (on_aux && forked && share_sm()) mm.flags |= GLQ_MM_SHARE_SM;      // the routed products run beside it
        after_kernel[on_aux ? 1 : 0] = true;
        mm.workspace = ws + (on_aux ? L.mm2 : L.mm);
        mm.workspace_bytes = L.mm_bytes;
        mm.counters = counters ? counters + (on_aux ? L.mm_counters : 0) : nullptr;
        mm.n_counters = L.mm_counters;
        return glq_grouped_matmul(&mm, on_aux && forked ? aux_stream : stream);
    };
    int rc;
    // y = x . Pi^T for a tiled dense Pi (rows x dim -> rows x dim)
    auto rotate = [&](const void* pi_t, const float* signs, const void* src, int rows, int dim, void* dst) {
        if (signs)
            return glq_rht_forward(src, 0, dim, signs, rows, dim, 1.0f / sqrtf((float)dim), dst, 0, dim,
                                   on_aux && forked ? aux_stream : stream);
        set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 1, rows, dim, dim, 0);
        m.w.codes = pi_t;
        m.w.N = dim;
        m.w.K = dim;
        m.x = src;
        m.ldx = dim;
        m.y = dst;
        m.ldy = dim;
        return finish(m);
    };
    const void* xq = x;  // input of the quantized gate/up products
    if (d->rot_in || d->rht_in) {
        if ((rc = rotate(d->rot_in, d->rht_in, x, n, d->H, ws + L.xr)) != GLQ_OK) return rc;
        xq = ws + L.xr;
    }

    // 1. router logits (and the shared expert's gate logit): dense fp16 matmul
    //    when the shared expert's U_gate^T / U_up^T are appended to the router rows, the same product
    //    also yields the shared expert's x.U (columns sh_a_row .. +2R of the output)
    const bool sh_a_fused = d->sh_a_row > 0 && d->dense0_rows >= d->sh_a_row + 2 * R;
    if (!given) {
        set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 1, n, ldl, d->H, 0);
        m.w.codes = d->router_t;
        m.w.N = ldl;
        m.w.K = d->H;
        m.x = x;
        m.ldx = d->H;
        m.y = p_logits;
        m.ldy = ldl;
        if ((rc = finish(m)) != GLQ_OK) return rc;
    }

    if (forked && cudaEventRecord(reinterpret_cast<cudaEvent_t>(ev_fork), st) != cudaSuccess) return GLQ_ERR_CUDA;

    // 2. routing plan
    if ((long long)nk >= kPlanParallelFrom) {
        // many tokens: routing, per-block counts, lists and scatter as four launches over the SMs
        const int nb = (nk + kPlanChunk - 1) / kPlanChunk;
        int* blk = reinterpret_cast<int*>(ws + L.plan_blk);
        const int* s_in = given ? (const int*)ep->sel_in : (const int*)nullptr;
        const __half* w_in = given ? reinterpret_cast<const __half*>(ep->weight_in) : (const __half*)nullptr;
        moe_route_kernel<<<given ? std::min(1024, (nk + 255) / 256) : (n + 7) / 8, 256, 0, st>>>(
            (const __half*)p_logits, ldl, n, (int)d->E, k, (int)d->norm_topk_prob, p_sel, p_wts, p_tok,
            reinterpret_cast<__half*>(router_logits), (int*)sel_out, reinterpret_cast<__half*>(weight_out), s_in, w_in);
        moe_plan_count_kernel<<<nb, 32, d->E * sizeof(int), st>>>(p_sel, nk, (int)d->E, blk);
        moe_plan_lists_kernel<<<1, 1024, 2 * d->E * sizeof(int), st>>>(
            blk, nb, nk, (int)d->E, chunk, ep_rank, ep_world, p_active, p_nact, p_cnt, p_off,
            reinterpret_cast<int*>(ws + L.active2), reinterpret_cast<int*>(ws + L.n_active2),
            reinterpret_cast<int*>(ws + L.slot_count2), reinterpret_cast<int*>(ws + L.slot_offset2));
        moe_plan_scatter_kernel<<<nb, 32, d->E * sizeof(int), st>>>(p_sel, p_wts, nk, (int)d->E, k, blk, p_erow, p_escale, p_tok);
        if (cudaGetLastError() != cudaSuccess) return GLQ_ERR_CUDA;
        after_kernel[0] = true;
    } else {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(1);
        cfg.blockDim = dim3(1024);
        cfg.dynamicSmemBytes = 2 * d->E * sizeof(int);
        cfg.stream = st;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 0;   // plain launch (a dependent launch after the router product measured no faster)
        if (cudaLaunchKernelEx(&cfg, moe_plan_kernel, (const __half*)p_logits, ldl, n, (int)d->E, k, (int)d->norm_topk_prob,
                               p_sel, p_wts, p_active, p_nact, p_cnt, p_off, p_erow, p_escale, p_tok,
                               reinterpret_cast<__half*>(router_logits), (int*)sel_out, reinterpret_cast<__half*>(weight_out),
                               reinterpret_cast<int*>(ws + L.active2), reinterpret_cast<int*>(ws + L.n_active2),
                               reinterpret_cast<int*>(ws + L.slot_count2), reinterpret_cast<int*>(ws + L.slot_offset2),
                               ep_rank, ep_world, given ? (const int*)ep->sel_in : (const int*)nullptr,
                               given ? reinterpret_cast<const __half*>(ep->weight_in) : (const __half*)nullptr, chunk) != cudaSuccess)
            return GLQ_ERR_CUDA;
        after_kernel[0] = true;
    }
    // rows of remote experts' entries stay zero, so that summing the ranks' buffers is exact
    if (ep_world > 1 && !(ep->flags & GLQ_MOE_EP_NO_ZERO_FILL) &&
        cudaMemsetAsync(p_yd, 0, (size_t)nk * d->H * 2, st) != cudaSuccess)
        return GLQ_ERR_CUDA;

    auto routed = [&](glq_mm_args_t& mm) {
        mm.slot_index = p_active;
        mm.n_slots = p_nact;
        mm.slot_count = p_cnt;
        mm.slot_offset = p_off;
    };

    // 3. x.U of the routed experts' gate and up clusters: one launch over 2 x (live experts) slots,
    //    rows 0..nk of the output for gate, nk..2nk for up
    char* a_gate = ws + L.a_gu;
    char* a_up = a_gate + (size_t)nk * R * 2;
    if (R > 0) {
        set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 2 * P, rows, R, d->H, 0, 2 * nk);
        m.w_table = d->ut_gate_up;
        m.slot_index = reinterpret_cast<int*>(ws + L.active2);
        m.n_slots = reinterpret_cast<int*>(ws + L.n_active2);
        m.slot_count = reinterpret_cast<int*>(ws + L.slot_count2);
        m.slot_offset = reinterpret_cast<int*>(ws + L.slot_offset2);
        m.entry_row = p_erow;
        m.x = x;
        m.ldx = d->H;
        m.y = a_gate;
        m.ldy = R;
        if ((rc = finish(m)) != GLQ_OK) return rc;
    }
    // 4. h = silu(gate x) * (up x), one row per (token, expert) entry
    set_mm(&m, d->fmt, d->group_size, GLQ_EPI_SWIGLU, P, rows, d->I, d->H, R, nk);
    m.w_table = d->gate_up;
    routed(m);
    m.entry_row = p_erow;
    m.x = xq;
    m.ldx = d->H;
    if (R > 0) {
        m.a0 = a_gate;
        m.a1 = a_up;
        m.lda = R;
        m.flags = GLQ_MM_A_FROM_PREVIOUS_LAUNCH;    // the x.U launch directly before; x and the lists are older
    }
    m.y = ws + L.h;
    m.ldy = d->I;
    if ((rc = finish(m)) != GLQ_OK) return rc;
    // 5. h.U of the down clusters
    if (R > 0) {
        set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, P, rows, R, d->I, 0, nk);
        m.w_table = d->ut_down;
        routed(m);
        m.x = ws + L.h;
        m.ldx = d->I;
        m.y = ws + L.b;
        m.ldy = R;
        if ((rc = finish(m)) != GLQ_OK) return rc;
    }
    // 6. down projection, scaled by the routing weight
    const void* hq = ws + L.h;
    if (d->rot_mid || d->rht_mid) {
        // rotates every entry row (rows beyond the live entries hold stale but finite data)
        if ((rc = rotate(d->rot_mid, d->rht_mid, ws + L.h, nk, d->I, ws + L.hr)) != GLQ_OK) return rc;
        hq = ws + L.hr;
    }
    set_mm(&m, d->fmt, d->group_size, GLQ_EPI_LINEAR, P, rows, d->H, d->I, R, nk);
    m.w_table = d->down;
    routed(m);
    m.entry_scale = p_escale;
    m.x = hq;
    m.ldx = d->I;
    if (R > 0) {
        m.a0 = ws + L.b;
        m.lda = R;
        if (hq == ws + L.h) m.flags = GLQ_MM_A_FROM_PREVIOUS_LAUNCH;   // h.U directly before; not when a rotation sits between
    }
    m.y = p_yd;
    m.ldy = d->H;
    if ((rc = finish(m)) != GLQ_OK) return rc;

    // 7. shared expert (every rank computes it: no exchange)
    if (shared) {
        if (forked) {
            if (cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(aux_stream), reinterpret_cast<cudaEvent_t>(ev_fork), 0) !=
                cudaSuccess)
                return GLQ_ERR_CUDA;
            on_aux = true;
        }
        const bool lr = R > 0 && d->sh_ut_down && (sh_a_fused || (d->sh_ut_gate && d->sh_ut_up));
        const void* a_sg = ws + L.a_sg;
        const void* a_su = ws + L.a_su;
        long long lda_s = R;
        if (lr && sh_a_fused) {
            a_sg = reinterpret_cast<const __half*>(p_logits) + d->sh_a_row;
            a_su = reinterpret_cast<const __half*>(p_logits) + d->sh_a_row + R;
            lda_s = ldl;
        }
        if (lr && !sh_a_fused) {
            for (int which = 0; which < 2; ++which) {
                set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 1, n, R, d->H, 0);
                m.w.codes = which == 0 ? d->sh_ut_gate : d->sh_ut_up;
                m.w.N = R;
                m.w.K = d->H;
                m.x = x;
                m.ldx = d->H;
                m.y = ws + (which == 0 ? L.a_sg : L.a_su);
                m.ldy = R;
                if ((rc = finish(m)) != GLQ_OK) return rc;
            }
        }
        set_mm(&m, d->fmt, d->group_size, GLQ_EPI_SWIGLU, 1, n, d->I_shared, d->H, lr ? R : 0);
        m.w = d->sh_gate_up;
        if (!lr) m.w.rank = 0;
        m.x = xq;
        m.ldx = d->H;
        if (lr) {
            m.a0 = a_sg;
            m.a1 = a_su;
            m.lda = lda_s;
        }
        m.y = ws + L.hs;
        m.ldy = d->I_shared;
        if ((rc = finish(m)) != GLQ_OK) return rc;
        if (lr) {
            set_mm(&m, GLQ_FMT_F16, 0, GLQ_EPI_LINEAR, 1, n, R, d->I_shared, 0);
            m.w.codes = d->sh_ut_down;
            m.w.N = R;
            m.w.K = d->I_shared;
            m.x = ws + L.hs;
            m.ldx = d->I_shared;
            m.y = ws + L.bs;
            m.ldy = R;
            if ((rc = finish(m)) != GLQ_OK) return rc;
        }
        const void* hsq = ws + L.hs;
        if (d->sh_rot_mid || d->sh_rht_mid) {
            if ((rc = rotate(d->sh_rot_mid, d->sh_rht_mid, ws + L.hs, n, d->I_shared, ws + L.hsr)) != GLQ_OK) return rc;
            hsq = ws + L.hsr;
        }
        set_mm(&m, d->fmt, d->group_size, GLQ_EPI_LINEAR, 1, n, d->H, d->I_shared, lr ? R : 0);
        m.w = d->sh_down;
        if (!lr) m.w.rank = 0;
        m.x = hsq;
        m.ldx = d->I_shared;
        if (lr) {
            m.a0 = ws + L.bs;
            m.lda = R;
            if (hsq == ws + L.hs) m.flags = GLQ_MM_A_FROM_PREVIOUS_LAUNCH;
        }
        m.y = ws + L.ysh;
        m.ldy = d->H;
        if ((rc = finish(m)) != GLQ_OK) return rc;
        if (forked) {
            on_aux = false;
            if (cudaEventRecord(reinterpret_cast<cudaEvent_t>(ev_join), reinterpret_cast<cudaStream_t>(aux_stream)) != cudaSuccess)
                return GLQ_ERR_CUDA;
        }
    }
    }   // phases before the combine
    if (phase == GLQ_MOE_PHASE_EXPERTS) return GLQ_OK;
    // the shared expert's branch joins only here: with expert parallelism the caller's exchange of the entry
    // buffer, issued between the two phases, overlaps the rest of that branch
    if (!fused && aux_stream != nullptr && ev_fork != nullptr && ev_join != nullptr && shared &&
        cudaStreamWaitEvent(st, reinterpret_cast<cudaEvent_t>(ev_join), 0) != cudaSuccess)
        return GLQ_ERR_CUDA;

    // 8. combine
    if (ep && ep->normed_out) {
        if (d->H > 8192) return GLQ_ERR_UNSUPPORTED;
        moe_combine_norm_kernel<<<n, 256, 0, st>>>(
            reinterpret_cast<const __half*>(p_yd), p_tok, nk, p_sel, k, d->H, n > d->slot_order_max_tokens ? 1 : 0,
            shared ? reinterpret_cast<const __half*>(ws + L.ysh) : nullptr, p_logits, ldl, d->router_rows > d->E ? d->E : -1,
            reinterpret_cast<const __half*>(ep->residual), reinterpret_cast<const __half*>(ep->norm_weight), ep->norm_eps,
            reinterpret_cast<__half*>(out), reinterpret_cast<__half*>(ep->normed_out), px_epoch, px_half);
        return cudaGetLastError() == cudaSuccess ? GLQ_OK : GLQ_ERR_CUDA;
    }
    if (ep && ep->residual) return GLQ_ERR_ARG;     // a residual needs the fused form (normed_out)
    const dim3 grid((d->H / 8 + 255) / 256, n);
    moe_combine_kernel<<<grid, 256, 0, st>>>(
        reinterpret_cast<const __half*>(p_yd), p_tok, nk, p_sel, k, d->H, n > d->slot_order_max_tokens ? 1 : 0,
        shared ? reinterpret_cast<const __half*>(ws + L.ysh) : nullptr, p_logits, ldl,
        d->router_rows > d->E ? d->E : -1, reinterpret_cast<__half*>(out), px_epoch, px_half);
    if (cudaGetLastError() != cudaSuccess) return GLQ_ERR_CUDA;
    return GLQ_OK;
}
