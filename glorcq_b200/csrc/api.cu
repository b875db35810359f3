// extern "C" entry points of libglorcq_b200: argument checks, launch geometry, launches.
// No torch types, no allocation: the caller owns every buffer.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "aux_kernels.cuh"
#include "skinny_mm.cuh"
#include "stream_mm.cuh"
#include "tc_mm.cuh"
#include "tc_ps.cuh"

using namespace glq;

static thread_local int g_last_cuda_error = 0;

#define GLQ_CUDA(call)                                   \
    do {                                                 \
        cudaError_t e__ = (call);                        \
        if (e__ != cudaSuccess) {                        \
            g_last_cuda_error = (int)e__;                \
            return GLQ_ERR_CUDA;                         \
        }                                                \
    } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline bool aligned_to(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
static inline int cdiv(int a, int b) { return (a + b - 1) / b; }
static inline int pow2ceil(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

extern "C" int glq_version(void) { return 100; }

extern "C" const char* glq_status_string(int status) {
    switch (status) {
        case GLQ_OK: return "ok";
        case GLQ_ERR_ARG: return "invalid argument (null pointer or inconsistent size)";
        case GLQ_ERR_ALIGN: return "pointer or leading dimension not aligned to 16 bytes";
        case GLQ_ERR_UNSUPPORTED: return "shape, group size or rank not supported by the sm_100a kernels";
        case GLQ_ERR_CUDA: return "CUDA call failed (see glq_last_cuda_error)";
        case GLQ_ERR_WORKSPACE: return "workspace too small (or, for the *_static entry point, the problem needs more scratch than the fixed array holds)";
        default: return "unknown status";
    }
}

extern "C" int glq_last_cuda_error(void) { return g_last_cuda_error; }

// ---------------------------------------------------------------------------------------------
// tiled layout sizes
// ---------------------------------------------------------------------------------------------
static inline int fmt_kb(int fmt) { return (fmt == GLQ_FMT_Q2 || fmt == GLQ_FMT_T2) ? 128 : 64; }
static inline int dest_pairs(int n_rows, int count) { return (cdiv(n_rows, 16) * count + 1) / 2; }

extern "C" size_t glq_tiled_bytes(int fmt, int n_rows, int K, int count) {
    if (fmt < 0 || fmt > 2 || n_rows <= 0 || K <= 0 || count < 1 || count > 2) return 0;
    return (size_t)dest_pairs(n_rows, count) * cdiv(K, fmt_kb(fmt)) * 2 * block_bytes_of(fmt);
}
extern "C" size_t glq_sv_bytes(int n_rows, int rank, int count) {
    if (n_rows <= 0 || rank <= 0 || count < 1 || count > 2) return 0;
    return (size_t)dest_pairs(n_rows, count) * cdiv(rank, 64) * 4096;
}
extern "C" size_t glq_rows_f32_count(int n_rows, int count) {
    if (n_rows <= 0 || count < 1 || count > 2) return 0;
    return (size_t)dest_pairs(n_rows, count) * 32;
}
extern "C" size_t glq_tiled_f16_bytes(int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    return (size_t)cdiv(N, 16) * cdiv(K, 64) * 4 * 512;
}

// ---------------------------------------------------------------------------------------------
// launch geometry of the skinny kernel (shared by the workspace query and the launcher)
// ---------------------------------------------------------------------------------------------
struct Geometry {
    int nw, ntt, ntc, nkb, group_blocks, tile_groups, sk, kb_per_split, kb_chunk, max_passes;
    size_t smem, n_counters, scratch_bytes;
};

// SM count of the current device (cached per device: the planned splits follow the GPU the call runs on)
static int num_sms() {
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

static int plan_geometry(int fmt, int epilogue, int N, int K, int group_size, int n_problems, int max_rows,
                         bool allow_split, Geometry* out) {
    if (fmt < 0 || fmt > 3 || N <= 0 || K <= 0 || n_problems <= 0 || max_rows <= 0) return GLQ_ERR_ARG;
    Geometry g{};
    g.nw = (epilogue == GLQ_EPI_SWIGLU) ? 2 : 1;
    if (g.nw == 2 && fmt == GLQ_FMT_F16) return GLQ_ERR_UNSUPPORTED;
    const int kb = fmt_kb(fmt);
    g.nkb = cdiv(K, kb);
    g.group_blocks = 1;
    if (fmt == GLQ_FMT_Q2 || fmt == GLQ_FMT_Q4) {
        if (group_size <= 0 || group_size % kb != 0) return GLQ_ERR_UNSUPPORTED;
        g.group_blocks = group_size / kb;
    }
    if (max_rows <= 8) g.ntt = 1;
    else if (max_rows <= 16 || g.nw == 2) g.ntt = 2;
    else g.ntt = 4;
    g.ntc = g.ntt == 1 ? std::max(2, pow2ceil(max_rows)) : 8 * g.ntt;
    g.max_passes = cdiv(max_rows, 8 * g.ntt);
    g.tile_groups = cdiv(cdiv(N, kRowTile), kRW);

    // CTA-level k split: fill the machine about twice over while every warp keeps >= 1 k block
    const long ctas = (long)n_problems * g.tile_groups;
    const int units = cdiv(g.nkb, g.group_blocks);  // split granularity = one scale group
    int sk = 1;
    if (allow_split) {
        const long want = 2L * num_sms();
        if (ctas < want) sk = (int)std::min<long>((want + ctas - 1) / ctas, std::max(1, units / kKW));
    }
    g.kb_per_split = cdiv(units, sk) * g.group_blocks;
    g.sk = cdiv(g.nkb, g.kb_per_split);
    // shared memory holds kb_chunk blocks of staged activations at a time (two CTAs per SM)
    const size_t per_kb = skinny_smem_bytes(fmt, 1, g.ntc, g.nw, g.ntt) - skinny_smem_bytes(fmt, 0, g.ntc, g.nw, g.ntt);
    const size_t fixed = skinny_smem_bytes(fmt, 0, g.ntc, g.nw, g.ntt);
    const size_t smem_cap = 100 * 1024;
    g.kb_chunk = (int)std::max<size_t>(1, std::min<size_t>((size_t)std::min(g.kb_per_split, g.nkb),
                                                             (smem_cap - fixed) / per_kb));
    g.smem = skinny_smem_bytes(fmt, g.kb_chunk, g.ntc, g.nw, g.ntt);
    const size_t tiles = (size_t)n_problems * g.tile_groups * g.max_passes;
    g.n_counters = g.sk > 1 ? tiles : 0;
    g.scratch_bytes = g.sk > 1 ? tiles * g.sk * (size_t)(kRW * g.nw * g.ntt * 32) * sizeof(float4) : 0;
    *out = g;
    return GLQ_OK;
}

// launch with programmatic stream serialization: the grid may be scheduled while the previous kernel of
// the stream still runs; the kernels wait for it (griddepcontrol.wait) before they read its results
static thread_local bool t_dependent_launch = false;
static thread_local bool t_share_sm = false;
template <typename Kern, typename Params>
static int launch_dependent(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, const Params& p) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    GLQ_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return GLQ_OK;
}

template <int FMT, int NW, int NTT, bool RM>
static int launch_one(const SkinnyParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kern = skinny_kernel<FMT, NW, NTT, RM>;
    if (smem > 48 * 1024) {
        static size_t configured[16] = {0};
        int dev = 0;
        GLQ_CUDA(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 16 || configured[dev] < smem) {
            GLQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            if (dev >= 0 && dev < 16) configured[dev] = smem;
        }
    }
    if (t_dependent_launch) return launch_dependent(kern, dim3(grid), dim3(kThreads), smem, st, p);
    kern<<<grid, kThreads, smem, st>>>(p);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

template <int FMT, bool RM>
static int launch_fmt(const SkinnyParams& p, const Geometry& g, int grid, cudaStream_t st) {
    if (g.nw == 2) {
        if constexpr (FMT == GLQ_FMT_F16 || RM) {
            return GLQ_ERR_UNSUPPORTED;
        } else {
            if (g.ntt == 1) return launch_one<FMT, 2, 1, false>(p, grid, g.smem, st);
            return launch_one<FMT, 2, 2, false>(p, grid, g.smem, st);
        }
    }
    if (g.ntt == 1) return launch_one<FMT, 1, 1, RM>(p, grid, g.smem, st);
    if (g.ntt == 2) return launch_one<FMT, 1, 2, RM>(p, grid, g.smem, st);
    return launch_one<FMT, 1, 4, RM>(p, grid, g.smem, st);
}

static int launch_skinny(int fmt, bool rowmajor, const SkinnyParams& p, const Geometry& g, int n_problems,
                         cudaStream_t st) {
    const long grid = (long)n_problems * g.tile_groups * g.sk;
    if (grid <= 0 || grid > 0x7fffffffL) return GLQ_ERR_UNSUPPORTED;
    if (rowmajor) {
        if (fmt != GLQ_FMT_T2) return GLQ_ERR_UNSUPPORTED;
        return launch_fmt<GLQ_FMT_T2, true>(p, g, (int)grid, st);
    }
    switch (fmt) {
        case GLQ_FMT_Q2: return launch_fmt<GLQ_FMT_Q2, false>(p, g, (int)grid, st);
        case GLQ_FMT_Q4: return launch_fmt<GLQ_FMT_Q4, false>(p, g, (int)grid, st);
        case GLQ_FMT_T2: return launch_fmt<GLQ_FMT_T2, false>(p, g, (int)grid, st);
        case GLQ_FMT_F16: return launch_fmt<GLQ_FMT_F16, false>(p, g, (int)grid, st);
    }
    return GLQ_ERR_ARG;
}

static void fill_geometry(SkinnyParams& p, const Geometry& g) {
    p.tile_groups = g.tile_groups;
    p.sk = g.sk;
    p.kb_per_split = g.kb_per_split;
    p.kb_chunk = g.kb_chunk;
    p.group_blocks = g.group_blocks;
    p.nkb = g.nkb;
    p.ntc = g.ntc;
    p.max_passes = g.max_passes;
}

// ---------------------------------------------------------------------------------------------
// streaming kernel: eligibility, geometry, launch
// ---------------------------------------------------------------------------------------------
struct StreamGeom {
    int i8, nt, ntc, nkb, sk, kb_per_split, npairs, ips, stages, stage_bytes, swiglu;
    int off_xs, off_ox, off_as, off_ring, off_red;
    size_t smem;
    int grid;
};

static bool pdl_disabled() {
    static const bool v = std::getenv("GLQ_NO_PDL") != nullptr;
    return v;
}
static bool stream_disabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("GLQ_NO_STREAM");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}
static bool i8_disabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("GLQ_NO_I8");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// returns true when the streaming kernel covers this call
static bool plan_stream(int fmt, int epilogue, int N, int K, int rank, int group_size, int n_problems, int max_rows,
                        StreamGeom* out) {
    if (stream_disabled()) return false;
    if (fmt != GLQ_FMT_Q2 && fmt != GLQ_FMT_Q4 && fmt != GLQ_FMT_T2) return false;
    if (N <= 0 || K <= 0 || n_problems <= 0 || max_rows <= 0 || rank < 0 || rank % 16 != 0) return false;
    StreamGeom g{};
    g.swiglu = (epilogue == GLQ_EPI_SWIGLU) ? 1 : 0;
    const int kb = fmt_kb(fmt);
    g.nkb = cdiv(K, kb);
    int group_blocks = 1;
    if (fmt != GLQ_FMT_T2) {
        if (group_size <= 0 || group_size % kb != 0) return false;
        group_blocks = group_size / kb;
    }
    int rows;
    if (max_rows <= 8 && !i8_disabled()) {
        g.i8 = 1;
        g.nt = max_rows <= 4 ? 1 : 2;
        rows = 4 * g.nt;
        g.ntc = 8 * g.nt;
    } else {
        g.i8 = 0;
        if (max_rows <= 8) g.nt = 1;
        else if (max_rows <= 16) g.nt = 2;
        else if (max_rows <= 32) g.nt = 4;
        else return false;
        rows = 8 * g.nt;
        g.ntc = g.nt == 1 ? std::max(2, pow2ceil(max_rows)) : 8 * g.nt;
    }
    const int ntiles = cdiv(N, kRowTile);
    g.npairs = g.swiglu ? ntiles : cdiv(ntiles, 2);
    // k splits (warps of one CTA): enough iterations to give every SM one; splits on group boundaries
    const int units = cdiv(g.nkb, group_blocks);
    int sk = 1;
    const long want_iters = (long)kStreamCtasPerSm * num_sms();
    while (sk < 8 && (long)n_problems * cdiv(g.npairs * sk, kWarpsPerCta) < want_iters && units >= 2 * sk) sk *= 2;
    int ctas_per_sm = kStreamCtasPerSm;
    for (;; sk /= 2) {
        g.sk = sk;
        g.kb_per_split = cdiv(units, sk) * group_blocks;
        g.ips = cdiv(g.npairs * sk, kWarpsPerCta);
        g.stage_bytes = std::max(kStreamCB * 2 * block_bytes_of(fmt), 4096);
        size_t off = kWarpsPerCta * kMaxStages * 8;
        off = (off + 127) / 128 * 128;
        g.off_xs = (int)off;
        if (g.i8) {
            const int p8 = fmt == GLQ_FMT_Q4 ? 1 : 2;
            off += (size_t)g.nkb * p8 * (2 * rows) * 4 * 16;
            g.off_ox = (int)off;
            off += (size_t)g.nkb * rows * 8;
        } else {
            const int xs_u4 = (fmt == GLQ_FMT_Q4) ? 8 : 16;
            off += (size_t)g.nkb * xs_u4 * g.ntc * 16;
            g.off_ox = (int)off;
            off += (size_t)g.nkb * g.ntc * 8;
        }
        off = (off + 15) / 16 * 16;
        g.off_as = (int)off;
        off += (size_t)(g.swiglu ? 2 : 1) * rows * std::max(rank, 16) * 2;
        off = (off + 127) / 128 * 128;
        g.off_ring = (int)off;
        const size_t red = sk > 1 ? (size_t)2 * kWarpsPerCta * 2 * g.nt * 32 * 16 : 0;
        // two CTAs per SM when the staged activations leave room for it, else one
        size_t cap = (size_t)(kStreamCtasPerSm == 1 ? 220 : 110) * 1024;
        ctas_per_sm = kStreamCtasPerSm;
        if (off + red + (size_t)kWarpsPerCta * 2 * g.stage_bytes > cap) {
            cap = 220 * 1024;
            ctas_per_sm = 1;
        }
        if (off + red + (size_t)kWarpsPerCta * 2 * g.stage_bytes > cap) {
            if (sk > 1) continue;
            return false;
        }
        int stages = (int)((cap - off - red) / ((size_t)kWarpsPerCta * g.stage_bytes));
        g.stages = std::min(stages, kMaxStages);
        off += (size_t)kWarpsPerCta * g.stages * g.stage_bytes;
        g.off_red = (int)off;
        off += red;
        g.smem = off;
        // the k-split reduction buffer may be what pushes the CTA over half an SM's shared memory: fewer
        // splits with two CTAs per SM stream better, as long as every SM still gets work
        if (ctas_per_sm == 1 && sk > 1 && kStreamCtasPerSm == 2 &&
            (size_t)g.off_ring + (size_t)kWarpsPerCta * 2 * g.stage_bytes <= (size_t)110 * 1024 &&
            (long)n_problems * cdiv(g.npairs, kWarpsPerCta) >= num_sms()) {
            sk = 2;      // -> one split: no reduction buffer
            continue;
        }
        break;
    }
    const long iters = (long)n_problems * g.ips;
    g.grid = (int)std::min<long>(iters, (long)ctas_per_sm * num_sms());
    *out = g;
    return g.grid > 0;
}

template <int FMT, bool I8, int NT>
static int launch_stream_one(const StreamParams& sp, const StreamGeom& g, cudaStream_t st) {
    auto kern = stream_kernel<FMT, I8, NT>;
    static size_t configured[16] = {0};
    int dev = 0;
    GLQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16 || configured[dev] < g.smem) {
        GLQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem));
        if (dev >= 0 && dev < 16) configured[dev] = g.smem;
    }
    if (sp.a_late || sp.dependent) return launch_dependent(kern, dim3(g.grid), dim3(kThreads), g.smem, st, sp);
    kern<<<g.grid, kThreads, g.smem, st>>>(sp);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

template <int FMT>
static int launch_stream_fmt(const StreamParams& sp, const StreamGeom& g, cudaStream_t st) {
    if (g.i8) {
        if (g.nt == 1) return launch_stream_one<FMT, true, 1>(sp, g, st);
        return launch_stream_one<FMT, true, 2>(sp, g, st);
    }
    if (g.nt == 1) return launch_stream_one<FMT, false, 1>(sp, g, st);
    if (g.nt == 2) return launch_stream_one<FMT, false, 2>(sp, g, st);
    return launch_stream_one<FMT, false, 4>(sp, g, st);
}

static int launch_stream(int fmt, SkinnyParams& p, const StreamGeom& g, int N, int K, int rank, int n_problems,
                         cudaStream_t st, bool a_late = false, bool dependent = false, int cnt_lo = 0,
                         int cnt_hi = 0x7fffffff) {
    StreamParams sp{};
    sp.cnt_lo = cnt_lo;
    sp.cnt_hi = cnt_hi;
    sp.a_late = (a_late && rank > 0 && p.a[0] != nullptr && !pdl_disabled()) ? 1 : 0;
    sp.dependent = ((dependent || a_late) && !pdl_disabled()) ? 1 : 0;
    p.nkb = g.nkb;
    p.ntc = g.ntc;
    p.kb_chunk = g.nkb;
    p.kb_per_split = g.nkb;
    p.sk = 1;
    sp.b = p;
    sp.N = N;
    sp.K = K;
    sp.rank = rank;
    sp.n_problems = n_problems;
    sp.swiglu = g.swiglu;
    sp.sk = g.sk;
    sp.sk_log2 = g.sk == 1 ? 0 : (g.sk == 2 ? 1 : (g.sk == 4 ? 2 : 3));
    sp.kb_per_split = g.kb_per_split;
    sp.npairs = g.npairs;
    sp.ips = g.ips;
    sp.stages = g.stages;
    sp.stage_bytes = g.stage_bytes;
    sp.off_xs = g.off_xs;
    sp.off_ox = g.off_ox;
    sp.off_as = g.off_as;
    sp.off_ring = g.off_ring;
    sp.off_red = g.off_red;
    StreamGeom gl = g;
    // a concurrent stream runs grouped products too: two thirds of the CTA slots, so that its kernels find room
    // (measured on the MoE block: the shared expert's branch beside the routed experts')
    if (t_share_sm && gl.grid > 4 * num_sms() / 3) gl.grid = 4 * num_sms() / 3;
    switch (fmt) {
        case GLQ_FMT_Q2: return launch_stream_fmt<GLQ_FMT_Q2>(sp, gl, st);
        case GLQ_FMT_Q4: return launch_stream_fmt<GLQ_FMT_Q4>(sp, gl, st);
        case GLQ_FMT_T2: return launch_stream_fmt<GLQ_FMT_T2>(sp, gl, st);
    }
    return GLQ_ERR_ARG;
}

// ---------------------------------------------------------------------------------------------
// glq_grouped_matmul
// ---------------------------------------------------------------------------------------------
// ---------------------------------------------------------------------------------------------
// tensor-core path (tc_mm.cuh): many rows per problem
// ---------------------------------------------------------------------------------------------
struct TcGeom {
    int tn, nkb, ns, na, tiles_max;
    bool hybrid;
    long long tile_bytes;
    size_t xp_bytes;
};
static bool ts_disabled() {
    static const bool v = std::getenv("GLQ_NO_TS") != nullptr;
    return v;
}
static bool hybrid_disabled() {
    static const bool v = std::getenv("GLQ_NO_HYBRID") != nullptr;
    return v;
}
static bool tc_disabled() {
    static const bool v = std::getenv("GLQ_NO_TC") != nullptr;
    return v;
}
// true when the tcgen05 kernel takes the call: 2-bit affine codes, more rows than the streaming kernel stages
static bool plan_tc(const glq_mm_args_t* a, TcGeom* out) {
    if (tc_disabled() || a->max_rows <= 32) return false;
    if (a->N <= 0 || a->K <= 0 || a->n_problems <= 0 || a->rank < 0 || a->rank % 16 != 0) return false;
    if (a->fmt == GLQ_FMT_Q2 || a->fmt == GLQ_FMT_Q4) {
        if (a->group_size <= 0 || a->group_size % fmt_kb(a->fmt) != 0) return false;
    } else if (a->fmt == GLQ_FMT_F16) {
        if (a->epilogue != GLQ_EPI_LINEAR) return false;
    } else if (a->fmt != GLQ_FMT_T2) {
        return false;
    }
    TcGeom g{};
    const long long stride = a->rows_stride > 0 ? a->rows_stride : a->max_rows;
    long long total = a->total_rows > 0 ? a->total_rows : (long long)a->n_problems * (a->slot_offset ? a->max_rows : stride);
    if (!a->slot_offset) total = std::max(total, (long long)(a->n_problems - 1) * stride + a->max_rows);
    g.tn = (total / a->n_problems > 64) ? 128 : 64;
    // 256-token tiles: tensor-memory variant, plain epilogue (2-bit codes), long problems only
    static const char* tn_env = std::getenv("GLQ_TC_TN");
    const bool wide_ok = a->fmt == GLQ_FMT_Q2 && a->epilogue == GLQ_EPI_LINEAR && !ts_disabled();
    const int wide_from = tn_env ? std::atoi(tn_env) : 512;      // rows per problem from which the wide tile is used
    if (wide_ok && wide_from > 0 && total / a->n_problems >= wide_from) g.tn = 256;
    g.nkb = cdiv(a->K, 128);
    g.ns = a->rank > 0 ? cdiv(a->rank, 64) : 0;
    g.na = a->epilogue == GLQ_EPI_SWIGLU ? 2 : 1;
    const long long tiles = total / g.tn + a->n_problems + 1;
    if (tiles > 65535) return false;
    g.tiles_max = (int)tiles;
    g.tile_bytes = (long long)g.nkb * g.tn * 256 + (long long)g.ns * g.na * g.tn * 128;
    g.xp_bytes = (size_t)g.tiles_max * (size_t)g.tile_bytes + 256;   // + the work-item counter of the persistent kernel
    // device-side row counts with few rows per problem on average: the streaming kernels take the
    // problems with up to 32 rows (one launch for <= 8 rows on the integer path, one for 9..32), this
    // kernel only the larger ones
    g.hybrid = a->slot_count != nullptr && a->fmt != GLQ_FMT_F16 && total / a->n_problems <= 24 && !hybrid_disabled();
    *out = g;
    return true;
}

template <int FMT, int TN, bool SW>
static int launch_tc_t(const TcParams& p, int N, cudaStream_t st) {
    using C = TcCfg<TN, SW>;
    static bool configured[64] = {};
    int dev = 0;
    GLQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        GLQ_CUDA(cudaFuncSetAttribute(tc_kernel<FMT, TN, SW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    tc_pack_b_kernel<TN><<<dim3(p.tiles_max, p.nkb + p.ns), 256, 0, st>>>(p);
    GLQ_CUDA(cudaGetLastError());
    tc_kernel<FMT, TN, SW><<<dim3(cdiv(N, kTcFeat), p.tiles_max), kTcThreads, C::SMEM, st>>>(p);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

// variant with the weight operand in tensor memory (2-bit affine codes)
template <int TN, bool SW>
static int launch_tc_ts_t(const TcParams& p, int N, cudaStream_t st) {
    using C = TcTsCfg<TN, SW>;
    static bool configured[64] = {};
    int dev = 0;
    GLQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        GLQ_CUDA(cudaFuncSetAttribute(tc_ts_kernel<TN, SW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    tc_pack_b_kernel<TN><<<dim3(p.tiles_max, p.nkb + p.ns), 256, 0, st>>>(p);
    GLQ_CUDA(cudaGetLastError());
    tc_ts_kernel<TN, SW><<<dim3(cdiv(N, kTcFeat), p.tiles_max), kTcThreads, C::SMEM, st>>>(p);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

// persistent form of the tensor-memory variant: one CTA per SM over all (token tile, feature tile) items
static bool ps_disabled() {
    static const bool v = std::getenv("GLQ_NO_TC_PERSISTENT") != nullptr;
    return v;
}
template <int TN, bool SW>
static int launch_tc_ps_t(const TcParams& p, cudaStream_t st) {
    using C = TcPsCfg<TN, SW>;
    static bool configured[64] = {};
    int dev = 0;
    GLQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        GLQ_CUDA(cudaFuncSetAttribute(tc_ps_kernel<TN, SW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    tc_pack_b_kernel<TN><<<dim3(p.tiles_max, p.nkb + p.ns), 256, 0, st>>>(p);
    GLQ_CUDA(cudaGetLastError());
    const long work = (long)p.n_ft * p.tiles_max;
    const int grid = (int)std::min<long>(work, num_sms());
    tc_ps_kernel<TN, SW><<<grid, kTcThreads, C::SMEM, st>>>(p);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

static int launch_tc(const glq_mm_args_t* a, const TcGeom& g, cudaStream_t st, int min_rows = 0) {
    if (!a->workspace || a->workspace_bytes < g.xp_bytes) return GLQ_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(a->workspace) & 127u) != 0) return GLQ_ERR_ALIGN;
    TcParams p{};
    p.w = a->w;
    p.table = a->w_table;
    p.slot_index = a->slot_index;
    p.n_slots = a->n_slots;
    p.slot_count = a->slot_count;
    p.slot_offset = a->slot_offset;
    p.entry_row = a->entry_row;
    p.entry_scale = reinterpret_cast<const __half*>(a->entry_scale);
    p.x = reinterpret_cast<const __half*>(a->x);
    p.ldx = a->ldx;
    p.a[0] = reinterpret_cast<const __half*>(a->a0);
    p.a[1] = reinterpret_cast<const __half*>(a->a1);
    p.lda = a->lda;
    p.y = reinterpret_cast<__half*>(a->y);
    p.ldy = a->ldy;
    p.xp = reinterpret_cast<unsigned char*>(a->workspace);
    p.tile_bytes = g.tile_bytes;
    p.n_problems = a->n_problems;
    p.max_rows = a->max_rows;
    p.rows_stride = a->rows_stride > 0 ? a->rows_stride : a->max_rows;
    p.K = a->K;
    p.rank = (a->a0 != nullptr) ? a->rank : 0;
    p.nkb = g.nkb;
    p.ns = p.rank > 0 ? g.ns : 0;
    p.na = g.na;
    p.tiles_max = g.tiles_max;
    p.x_vec = ((reinterpret_cast<uintptr_t>(a->x) & 7u) == 0 && a->ldx % 4 == 0) ? 1 : 0;
    p.fmt = a->fmt;
    p.min_rows = min_rows;
    const bool sw = a->epilogue == GLQ_EPI_SWIGLU;
    const bool big = g.tn == 128;
    p.N = a->N;
    p.n_ft = cdiv(a->N, kTcFeat);
    p.y_vec = ((reinterpret_cast<uintptr_t>(a->y) & 15u) == 0 && a->ldy % 8 == 0 && a->N % 8 == 0) ? 1 : 0;
    p.x_vec16 = ((reinterpret_cast<uintptr_t>(a->x) & 15u) == 0 && a->ldx % 8 == 0) ? 1 : 0;
    p.tile_ctr = nullptr;
    if (a->fmt == GLQ_FMT_Q2 && !ts_disabled()) {
        p.ts = 1;
        if (!ps_disabled()) {
            p.tile_ctr = reinterpret_cast<int*>(p.xp + (g.xp_bytes - 256));
            if (g.tn == 256) return launch_tc_ps_t<256, false>(p, st);
            if (big) return sw ? launch_tc_ps_t<128, true>(p, st) : launch_tc_ps_t<128, false>(p, st);
            return sw ? launch_tc_ps_t<64, true>(p, st) : launch_tc_ps_t<64, false>(p, st);
        }
        if (g.tn == 256) return launch_tc_ts_t<256, false>(p, a->N, st);
        if (big) return sw ? launch_tc_ts_t<128, true>(p, a->N, st) : launch_tc_ts_t<128, false>(p, a->N, st);
        return sw ? launch_tc_ts_t<64, true>(p, a->N, st) : launch_tc_ts_t<64, false>(p, a->N, st);
    }
    switch (a->fmt) {
#define GLQ_TC_CASE(F)                                                                                       \
    case F:                                                                                                  \
        if (big) return sw ? launch_tc_t<F, 128, true>(p, a->N, st) : launch_tc_t<F, 128, false>(p, a->N, st); \
        return sw ? launch_tc_t<F, 64, true>(p, a->N, st) : launch_tc_t<F, 64, false>(p, a->N, st);
        GLQ_TC_CASE(GLQ_FMT_Q2)
        GLQ_TC_CASE(GLQ_FMT_Q4)
        GLQ_TC_CASE(GLQ_FMT_T2)
#undef GLQ_TC_CASE
        case GLQ_FMT_F16:
            return big ? launch_tc_t<GLQ_FMT_F16, 128, false>(p, a->N, st) : launch_tc_t<GLQ_FMT_F16, 64, false>(p, a->N, st);
    }
    return GLQ_ERR_UNSUPPORTED;
}

extern "C" size_t glq_mm_workspace_bytes(const glq_mm_args_t* a) {
    if (!a) return 0;
    TcGeom tg;
    if (plan_tc(a, &tg)) return tg.xp_bytes;
    StreamGeom sg;
    if (plan_stream(a->fmt, a->epilogue, a->N, a->K, a->rank, a->group_size, a->n_problems, a->max_rows, &sg)) return 0;
    Geometry g;
    if (plan_geometry(a->fmt, a->epilogue, a->N, a->K, a->group_size, a->n_problems, a->max_rows, true, &g) != GLQ_OK)
        return 0;
    return g.scratch_bytes;
}

extern "C" size_t glq_mm_counters(const glq_mm_args_t* a) {
    if (!a) return 0;
    TcGeom tg;
    if (plan_tc(a, &tg)) return 0;
    StreamGeom sg;
    if (plan_stream(a->fmt, a->epilogue, a->N, a->K, a->rank, a->group_size, a->n_problems, a->max_rows, &sg)) return 0;
    Geometry g;
    if (plan_geometry(a->fmt, a->epilogue, a->N, a->K, a->group_size, a->n_problems, a->max_rows, true, &g) != GLQ_OK)
        return 0;
    return g.n_counters;
}

extern "C" int glq_grouped_matmul(const glq_mm_args_t* a, void* stream) {
    if (!a || !a->x || !a->y) return GLQ_ERR_ARG;
    if (a->n_problems == 0 || a->max_rows == 0) return GLQ_OK;
    if (a->epilogue != GLQ_EPI_LINEAR && a->epilogue != GLQ_EPI_SWIGLU) return GLQ_ERR_ARG;
    if (a->rank < 0 || a->rank % 16 != 0) return GLQ_ERR_UNSUPPORTED;
    if (a->rank > 0 && (a->a0 || a->a1) && (a->lda % 8 != 0 || !aligned16(a->a0) || !aligned16(a->a1)))
        return GLQ_ERR_ALIGN;
    t_share_sm = (a->flags & GLQ_MM_SHARE_SM) != 0;
    TcGeom tg;
    const bool use_tc = plan_tc(a, &tg);
    if (use_tc && !tg.hybrid) {
        if (!a->w_table && !a->w.codes) return GLQ_ERR_ARG;
        return launch_tc(a, tg, reinterpret_cast<cudaStream_t>(stream));
    }
    // 9..32 rows of the same problems, counts known on the host: the integer path stages at most 8 rows (4 when the
    // staged activations of a long reduction leave no room for 8) and streams at a multiple of the fp16 path's rate,
    // so it runs over chunks of rows; after the first chunk the weights come from L2 where they fit
    if (!use_tc && !a->slot_count && !a->slot_offset && a->max_rows > 8 && a->max_rows <= 32 && !i8_disabled() &&
        (a->fmt == GLQ_FMT_Q2 || a->fmt == GLQ_FMT_Q4)) {
        int chunk = 0;
        for (int c : {8, 4}) {
            StreamGeom cg;
            if (plan_stream(a->fmt, a->epilogue, a->N, a->K, a->rank, a->group_size, a->n_problems, c, &cg) && cg.i8) {
                chunk = c;
                break;
            }
        }
        if (chunk) {
            for (int r0 = 0; r0 < a->max_rows; r0 += chunk) {
                glq_mm_args_t b = *a;
                b.max_rows = std::min(chunk, a->max_rows - r0);
                b.rows_stride = a->rows_stride > 0 ? a->rows_stride : a->max_rows;
                if (a->entry_row) b.entry_row = a->entry_row + r0;
                else b.x = static_cast<const char*>(a->x) + (size_t)r0 * a->ldx * 2;
                if (a->entry_scale) b.entry_scale = static_cast<const char*>(a->entry_scale) + (size_t)r0 * 2;
                if (a->a0) b.a0 = static_cast<const char*>(a->a0) + (size_t)r0 * a->lda * 2;
                if (a->a1) b.a1 = static_cast<const char*>(a->a1) + (size_t)r0 * a->lda * 2;
                b.y = static_cast<char*>(a->y) + (size_t)r0 * a->ldy * 2;
                const int rc = glq_grouped_matmul(&b, stream);
                if (rc != GLQ_OK) return rc;
            }
            return GLQ_OK;
        }
    }
    StreamGeom sg;
    // Row-count classes (device-side counts): slots with <= 8 rows go to the integer path, 9..16 to the
    // fp16 path with two activation tiles, and above that to the tcgen05 kernel when the call may have
    // more than 32 rows per slot, else to the fp16 path with four tiles.  Each class is one launch that
    // skips the slots of the others.
    StreamGeom sg8, sg16;
    const int cap = use_tc ? 16 : std::min(a->max_rows, 32);
    bool use_stream = plan_stream(a->fmt, a->epilogue, a->N, a->K, a->rank, a->group_size, a->n_problems, cap, &sg);
    const bool classes = use_stream && a->slot_count != nullptr && a->max_rows > 8 && !sg.i8 && !hybrid_disabled();
    const bool split8 = classes && plan_stream(a->fmt, a->epilogue, a->N, a->K, a->rank, a->group_size, a->n_problems, 8, &sg8) &&
                        sg8.i8;
    const bool split16 = classes && cap > 16 &&
                         plan_stream(a->fmt, a->epilogue, a->N, a->K, a->rank, a->group_size, a->n_problems, 16, &sg16);
    if (use_tc && !use_stream) {
        if (!a->w_table && !a->w.codes) return GLQ_ERR_ARG;
        return launch_tc(a, tg, reinterpret_cast<cudaStream_t>(stream));
    }
    Geometry g{};
    int rc = use_stream ? GLQ_OK
                        : plan_geometry(a->fmt, a->epilogue, a->N, a->K, a->group_size, a->n_problems, a->max_rows,
                                        true, &g);
    if (rc != GLQ_OK) return rc;
    if (!use_stream && g.sk > 1) {
        if (!a->workspace || a->workspace_bytes < g.scratch_bytes) return GLQ_ERR_WORKSPACE;
        if (!a->counters || a->n_counters < g.n_counters) return GLQ_ERR_WORKSPACE;
        if (!aligned16(a->workspace)) return GLQ_ERR_ALIGN;
    }
    if (!a->w_table && !a->w.codes) return GLQ_ERR_ARG;

    SkinnyParams p{};
    p.w = a->w;
    p.table = a->w_table;
    p.sv_slices = cdiv(std::max(a->rank, 1), 64);
    p.slot_index = a->slot_index;
    p.n_slots = a->n_slots;
    p.slot_count = a->slot_count;
    p.slot_offset = a->slot_offset;
    p.entry_row = a->entry_row;
    p.entry_scale = reinterpret_cast<const __half*>(a->entry_scale);
    p.x = reinterpret_cast<const __half*>(a->x);
    p.ldx = a->ldx;
    p.a[0] = reinterpret_cast<const __half*>(a->a0);
    p.a[1] = reinterpret_cast<const __half*>(a->a1);
    p.lda = a->lda;
    p.y = reinterpret_cast<__half*>(a->y);
    p.ldy = a->ldy;
    p.counters = a->counters;
    p.scratch = reinterpret_cast<float4*>(a->workspace);
    p.max_rows = a->max_rows;
    p.rows_stride = a->rows_stride > 0 ? a->rows_stride : a->max_rows;
    p.epilogue = a->epilogue;
    p.x_vec = (aligned16(a->x) && a->ldx % 8 == 0) ? 1 : 0;
    if (use_stream) {
        cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
        const bool a_late = (a->flags & GLQ_MM_A_FROM_PREVIOUS_LAUNCH) != 0, dep = (a->flags & GLQ_MM_AFTER_KERNEL) != 0;
        if (!split8 && !split16 && !use_tc) return launch_stream(a->fmt, p, sg, a->N, a->K, a->rank, a->n_problems, st, a_late, dep);
        // one launch per class; only the first may depend programmatically on the producer of x.U (the
        // later ones start after it has finished)
        int lo = 0;
        bool first = true;
        auto one = [&](const StreamGeom& gg, int rows, int hi) {
            SkinnyParams pp = p;
            pp.max_rows = rows;
            const int r2 = launch_stream(a->fmt, pp, gg, a->N, a->K, a->rank, a->n_problems, st, first && a_late, first && dep,
                                         lo, hi);
            first = false;
            lo = hi;
            return r2;
        };
        if (split8 && (rc = one(sg8, 8, 8)) != GLQ_OK) return rc;
        if (split16 && (rc = one(sg16, 16, 16)) != GLQ_OK) return rc;
        if ((rc = one(sg, cap, cap)) != GLQ_OK) return rc;
        if (use_tc) return launch_tc(a, tg, st, cap);
        return GLQ_OK;
    }
    fill_geometry(p, g);
    t_dependent_launch = (a->flags & (GLQ_MM_AFTER_KERNEL | GLQ_MM_A_FROM_PREVIOUS_LAUNCH)) != 0 && !pdl_disabled();
    rc = launch_skinny(a->fmt, false, p, g, a->n_problems, reinterpret_cast<cudaStream_t>(stream));
    t_dependent_launch = false;
    return rc;
}

// ---------------------------------------------------------------------------------------------
// glq_linear_forward
// ---------------------------------------------------------------------------------------------
static void linear_args(int fmt, int group_size, const glq_weight_t* w, int B, glq_mm_args_t* m) {
    std::memset(m, 0, sizeof(*m));
    m->fmt = fmt;
    m->group_size = group_size;
    m->epilogue = GLQ_EPI_LINEAR;
    m->n_problems = 1;
    m->max_rows = B;
    m->rows_stride = B;
    m->N = w->N;
    m->K = w->K;
    m->rank = w->rank;
    m->w = *w;
}
static void xu_args(const glq_weight_t* w, const void* ut, int B, glq_mm_args_t* m) {
    std::memset(m, 0, sizeof(*m));
    m->fmt = GLQ_FMT_F16;
    m->epilogue = GLQ_EPI_LINEAR;
    m->n_problems = 1;
    m->max_rows = B;
    m->rows_stride = B;
    m->N = w->rank;
    m->K = w->K;
    m->w.codes = ut;
    m->w.N = w->rank;
    m->w.K = w->K;
}
static inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }

extern "C" size_t glq_linear_workspace_bytes(int fmt, int group_size, const glq_weight_t* w, int B) {
    if (!w || B <= 0) return 0;
    glq_mm_args_t m;
    linear_args(fmt, group_size, w, B, &m);
    size_t total = up256(glq_mm_workspace_bytes(&m));
    if (w->rank > 0) {
        glq_mm_args_t u;
        xu_args(w, w->codes, B, &u);
        total += up256((size_t)B * w->rank * sizeof(__half)) + up256(glq_mm_workspace_bytes(&u));
    }
    return total;
}

extern "C" size_t glq_linear_counters(int fmt, int group_size, const glq_weight_t* w, int B) {
    if (!w || B <= 0) return 0;
    glq_mm_args_t m;
    linear_args(fmt, group_size, w, B, &m);
    size_t total = glq_mm_counters(&m);
    if (w->rank > 0) {
        glq_mm_args_t u;
        xu_args(w, w->codes, B, &u);
        total += glq_mm_counters(&u);
    }
    return total;
}

extern "C" int glq_linear_forward(int fmt, int group_size, const glq_weight_t* w, const void* ut, const void* x,
                                  int64_t ldx, const void* a, void* y, int64_t ldy, int B, void* workspace,
                                  size_t workspace_bytes, int32_t* counters, size_t n_counters, void* stream) {
    if (!w || !x || !y || B < 0) return GLQ_ERR_ARG;
    if (B == 0 || w->N == 0) return GLQ_OK;
    glq_mm_args_t m;
    linear_args(fmt, group_size, w, B, &m);
    char* ws = reinterpret_cast<char*>(workspace);
    const size_t main_ws = up256(glq_mm_workspace_bytes(&m));
    const size_t main_ctr = glq_mm_counters(&m);
    const void* a_use = a;
    if (!a && ut && w->rank > 0 && w->sv) {
        glq_mm_args_t u;
        xu_args(w, ut, B, &u);
        const size_t a_bytes = up256((size_t)B * w->rank * sizeof(__half));
        const size_t u_ws = up256(glq_mm_workspace_bytes(&u));
        const size_t u_ctr = glq_mm_counters(&u);
        if (!ws || workspace_bytes < main_ws + a_bytes + u_ws) return GLQ_ERR_WORKSPACE;
        if (u_ctr > 0 && (!counters || n_counters < main_ctr + u_ctr)) return GLQ_ERR_WORKSPACE;
        u.x = x;
        u.ldx = ldx;
        u.y = ws + main_ws;
        u.ldy = w->rank;
        u.workspace = ws + main_ws + a_bytes;
        u.workspace_bytes = u_ws;
        u.counters = counters ? counters + main_ctr : nullptr;
        u.n_counters = u_ctr;
        int rc = glq_grouped_matmul(&u, stream);
        if (rc != GLQ_OK) return rc;
        a_use = ws + main_ws;
    }
    if (main_ws > 0 && (!ws || workspace_bytes < main_ws)) return GLQ_ERR_WORKSPACE;
    if (main_ctr > 0 && (!counters || n_counters < main_ctr)) return GLQ_ERR_WORKSPACE;
    m.x = x;
    m.ldx = ldx;
    m.a0 = a_use;
    m.lda = w->rank;
    m.y = y;
    m.ldy = ldy;
    m.workspace = ws;
    m.workspace_bytes = main_ws;
    m.counters = counters;
    m.n_counters = main_ctr;
    if (!a_use) m.w.rank = 0, m.rank = 0;
    // x.U was just launched above and is needed only in the epilogue; x itself is older
    if (a_use != nullptr && a_use != a) m.flags = GLQ_MM_A_FROM_PREVIOUS_LAUNCH;
    return glq_grouped_matmul(&m, stream);
}

// ---------------------------------------------------------------------------------------------
// Drop-ins for the reference's native modules
// ---------------------------------------------------------------------------------------------
static int turbo_rowmajor(const void* x, const uint8_t* packed, const float* norms, const float* centroids, void* y,
                          int n_problems, int rows, int N, int K, int slot_rows, void* stream) {
    if (!x || !packed || !norms || !centroids || !y) return GLQ_ERR_ARG;
    if (K <= 0 || K % 4 != 0) return GLQ_ERR_UNSUPPORTED;
    if (!aligned_to(x, 2) || !aligned_to(y, 2) || !aligned_to(norms, 4) || !aligned_to(centroids, 4)) return GLQ_ERR_ALIGN;
    Geometry g;
    int rc = plan_geometry(GLQ_FMT_T2, GLQ_EPI_LINEAR, N, K, 0, n_problems, rows, false, &g);
    if (rc != GLQ_OK) return rc;
    SkinnyParams p{};
    p.w.codes = packed;
    p.w.reserved = aligned_to(packed, 8) ? 1 : 0;   // 8-byte loads of the codes only from an 8-byte aligned base
    p.w.norms = norms;
    p.w.centroids = centroids;
    p.w.N = N;
    p.w.K = K;
    p.sv_slices = 1;
    p.x = reinterpret_cast<const __half*>(x);
    p.ldx = K;
    p.y = reinterpret_cast<__half*>(y);
    p.ldy = N;
    p.max_rows = rows;
    p.rows_stride = rows;
    p.x_vec = (aligned16(x) && K % 8 == 0) ? 1 : 0;
    p.slot_rows = slot_rows;
    p.x_extent = (long long)n_problems * rows * K;
    p.y_extent = (long long)n_problems * rows * N;
    fill_geometry(p, g);
    return launch_skinny(GLQ_FMT_T2, true, p, g, n_problems, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int glq_turbo_dequant_matmul(const void* x_rot, const uint8_t* packed, const float* norms,
                                        const float* centroids, void* y, int B, int N, int K, void* stream) {
    if (B < 0 || N < 0) return GLQ_ERR_ARG;
    if (B == 0 || N == 0) return GLQ_OK;
    return turbo_rowmajor(x_rot, packed, norms, centroids, y, 1, B, N, K, 0, stream);
}

extern "C" int glq_turbo_dequant_grouped_gemv(const void* x_grouped, const uint8_t* packed_cat, const float* norms_cat,
                                              const float* centroids, void* y, int E, int N_out, int K,
                                              void* stream) {
    if (E < 0 || N_out < 0) return GLQ_ERR_ARG;
    if (E == 0 || N_out == 0) return GLQ_OK;
    return turbo_rowmajor(x_grouped, packed_cat, norms_cat, centroids, y, E, 1, N_out, K, N_out, stream);
}

extern "C" int glq_gptq_dequant_matmul(const float* x, const int8_t* q, const void* scales, const void* zeros,
                                       const float* lora_out, float* y, int B, int N, int K, int groupsize,
                                       int n_groups, int sym, void* stream) {
    if (B < 0 || N < 0 || K < 0) return GLQ_ERR_ARG;
    if (B == 0 || N == 0) return GLQ_OK;
    if (!x || !q || !scales || !y || (!sym && !zeros)) return GLQ_ERR_ARG;
    if (groupsize <= 0 || n_groups <= 0 || (long)n_groups * groupsize < K) return GLQ_ERR_ARG;
    if (!aligned_to(x, 4) || !aligned_to(y, 4) || !aligned_to(lora_out, 4) || !aligned_to(scales, 2) || !aligned_to(zeros, 2))
        return GLQ_ERR_ALIGN;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const size_t smem = (size_t)K * sizeof(float);
    // activation rows per pass over the codes: up to 8, as many as the staged rows leave room for (one pass for a
    // decode batch; a long prompt re-reads the int8 matrix once per 8 rows)
    int per = 8;
    while (per > 1 && smem * per > 200 * 1024) per /= 2;
    if (smem > 200 * 1024) return GLQ_ERR_UNSUPPORTED;
    static size_t configured[2][64] = {{0}, {0}};
    int dev = 0;
    GLQ_CUDA(cudaGetDevice(&dev));
    for (int b0 = 0; b0 < B; b0 += per) {
        const int nb = std::min(per, B - b0);
        const int wide = nb > 4 ? 1 : 0;
        const dim3 grid(cdiv(N, kWarpsPerCta));
        const size_t need = smem * nb;
        if (need > 48 * 1024 && (dev < 0 || dev >= 64 || configured[wide][dev] < need)) {
            if (wide)
                GLQ_CUDA(cudaFuncSetAttribute(gptq_i8_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(smem * per)));
            else
                GLQ_CUDA(cudaFuncSetAttribute(gptq_i8_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              (int)(smem * std::min(per, 4))));
            if (dev >= 0 && dev < 64) configured[wide][dev] = wide ? smem * per : smem * std::min(per, 4);
        }
        const float* xb = x + (size_t)b0 * K;
        const float* lb = lora_out ? lora_out + (size_t)b0 * N : nullptr;
        float* yb = y + (size_t)b0 * N;
        if (wide)
            gptq_i8_kernel<8><<<grid, kThreads, need, st>>>(xb, q, reinterpret_cast<const __half*>(scales),
                                                            reinterpret_cast<const __half*>(zeros), lb, yb, nb, N, K,
                                                            groupsize, n_groups, sym);
        else
            gptq_i8_kernel<4><<<grid, kThreads, need, st>>>(xb, q, reinterpret_cast<const __half*>(scales),
                                                            reinterpret_cast<const __half*>(zeros), lb, yb, nb, N, K,
                                                            groupsize, n_groups, sym);
        GLQ_CUDA(cudaGetLastError());
    }
    return GLQ_OK;
}

// ---------------------------------------------------------------------------------------------
// glq_turbo_dequant_matmul_static: the same product as glq_turbo_dequant_matmul, with k split over
// CTAs so that a single small matmul fills the machine, for callers that cannot hand over (or
// allocate) a workspace.  The partial sums and the arrival counters of the split live in a fixed
// array that is part of the library image.
// ---------------------------------------------------------------------------------------------
#define GLQ_STATIC_SCRATCH_BYTES (4u << 20)  /* partial sums */
#define GLQ_STATIC_COUNTERS 4096             /* arrival counters (ints), in front of the partial sums */
static __device__ __align__(256) unsigned char g_static_scratch[GLQ_STATIC_COUNTERS * 4 + GLQ_STATIC_SCRATCH_BYTES];

extern "C" size_t glq_static_scratch_bytes(void) { return GLQ_STATIC_SCRATCH_BYTES; }

extern "C" size_t glq_static_scratch_needed(int B, int N, int K) {
    Geometry g;
    if (B <= 0 || N <= 0 || K <= 0 || K % 4 != 0) return 0;
    if (plan_geometry(GLQ_FMT_T2, GLQ_EPI_LINEAR, N, K, 0, 1, B, true, &g) != GLQ_OK) return 0;
    return g.scratch_bytes;
}

extern "C" int glq_turbo_dequant_matmul_static(const void* x_rot, const uint8_t* packed, const float* norms,
                                               const float* centroids, void* y, int B, int N, int K, void* stream) {
    if (B < 0 || N < 0) return GLQ_ERR_ARG;
    if (B == 0 || N == 0) return GLQ_OK;
    if (!x_rot || !packed || !norms || !centroids || !y) return GLQ_ERR_ARG;
    if (K <= 0 || K % 4 != 0) return GLQ_ERR_UNSUPPORTED;
    if (!aligned_to(x_rot, 2) || !aligned_to(y, 2) || !aligned_to(norms, 4) || !aligned_to(centroids, 4)) return GLQ_ERR_ALIGN;
    // The array's name is only a host-side handle: its device address is looked up once per device,
    // with that device current, and it is that address the kernel gets.
    static unsigned char* dev_ptr[64] = {nullptr};
    int dev = 0;
    GLQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return GLQ_ERR_UNSUPPORTED;
    if (dev_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        GLQ_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (ptr == nullptr) return GLQ_ERR_CUDA;
        dev_ptr[dev] = reinterpret_cast<unsigned char*>(ptr);
    }
    Geometry g;
    int rc = plan_geometry(GLQ_FMT_T2, GLQ_EPI_LINEAR, N, K, 0, 1, B, true, &g);
    if (rc != GLQ_OK) return rc;
    // sizes the fixed array cannot hold are rejected, not truncated
    if (g.scratch_bytes > GLQ_STATIC_SCRATCH_BYTES || g.n_counters > GLQ_STATIC_COUNTERS) return GLQ_ERR_WORKSPACE;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // every call shares the array and it keeps the previous call's contents: the counters must start at zero
    if (g.n_counters > 0) GLQ_CUDA(cudaMemsetAsync(dev_ptr[dev], 0, g.n_counters * sizeof(int), st));
    SkinnyParams p{};
    p.w.codes = packed;
    p.w.reserved = aligned_to(packed, 8) ? 1 : 0;
    p.w.norms = norms;
    p.w.centroids = centroids;
    p.w.N = N;
    p.w.K = K;
    p.sv_slices = 1;
    p.x = reinterpret_cast<const __half*>(x_rot);
    p.ldx = K;
    p.y = reinterpret_cast<__half*>(y);
    p.ldy = N;
    p.max_rows = B;
    p.rows_stride = B;
    p.x_vec = (aligned16(x_rot) && K % 8 == 0) ? 1 : 0;
    p.x_extent = (long long)B * K;
    p.y_extent = (long long)B * N;
    p.counters = reinterpret_cast<int*>(dev_ptr[dev]);
    p.scratch = reinterpret_cast<float4*>(dev_ptr[dev] + GLQ_STATIC_COUNTERS * 4);
    fill_geometry(p, g);
    return launch_skinny(GLQ_FMT_T2, true, p, g, 1, st);
}

// ---------------------------------------------------------------------------------------------
// Load-time re-tiling and the dequantised-tile check
// ---------------------------------------------------------------------------------------------
static inline bool slot_ok(int slot, int count) { return count >= 1 && count <= 2 && slot >= 0 && slot < count; }

extern "C" int glq_pack_gptq(const int32_t* q, const void* scales, const void* zeros, int bits, int N, int K,
                             int group_size, void* tiled, int slot, int count, void* stream) {
    if (!q || !scales || !tiled || N <= 0 || K <= 0 || !slot_ok(slot, count)) return GLQ_ERR_ARG;
    if (bits != 2 && bits != 4) return GLQ_ERR_UNSUPPORTED;
    const int kb = bits == 2 ? 128 : 64;
    if (group_size <= 0 || group_size % kb != 0) return GLQ_ERR_UNSUPPORTED;
    const size_t words = (size_t)cdiv(N, 16) * cdiv(K, kb) * 144;
    pack_gptq_kernel<<<(unsigned)((words + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        q, reinterpret_cast<const __half*>(scales), reinterpret_cast<const __half*>(zeros), bits, N, K, group_size,
        reinterpret_cast<unsigned char*>(tiled), slot, count);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

extern "C" int glq_pack_turbo(const uint8_t* packed, int N, int K, void* tiled, int slot, int count, void* stream) {
    if (!packed || !tiled || N <= 0 || K <= 0 || !slot_ok(slot, count)) return GLQ_ERR_ARG;
    if (K % 4 != 0) return GLQ_ERR_UNSUPPORTED;
    const size_t words = (size_t)cdiv(N, 16) * cdiv(K, 128) * 128;
    pack_turbo_kernel<<<(unsigned)((words + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        packed, N, K, reinterpret_cast<unsigned char*>(tiled), slot, count);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

extern "C" int glq_pack_rows_f32(const float* v, int N, float* out, int slot, int count, void* stream) {
    if (!v || !out || N <= 0 || !slot_ok(slot, count)) return GLQ_ERR_ARG;
    const int n = cdiv(N, 16) * 16;
    pack_rows_f32_kernel<<<(n + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(v, N, out, slot, count);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

extern "C" int glq_pack_sv(const void* sv, int N, int rank, void* out, int slot, int count, void* stream) {
    if (!sv || !out || N <= 0 || rank <= 0 || !slot_ok(slot, count)) return GLQ_ERR_ARG;
    if (rank % 16 != 0) return GLQ_ERR_UNSUPPORTED;
    const size_t total = (size_t)cdiv(N, 16) * cdiv(rank, 64) * 1024;
    pack_sv_kernel<<<(unsigned)((total + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const __half*>(sv), N, rank, reinterpret_cast<__half*>(out), slot, count);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

extern "C" int glq_pack_f16(const void* W, long stride_n, long stride_k, int N, int K, void* tiled, void* stream) {
    if (!W || !tiled || N <= 0 || K <= 0) return GLQ_ERR_ARG;
    const size_t elems = glq_tiled_f16_bytes(N, K) / 2;
    pack_f16_kernel<<<(unsigned)((elems + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const __half*>(W), stride_n, stride_k, N, K, reinterpret_cast<__half*>(tiled), elems);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

extern "C" int glq_dequant_tiled(int fmt, const void* tiled, const float* norms_tiled, const float* centroids, int N,
                                 int K, int slot, int count, void* out, void* stream) {
    if (!tiled || !out || N <= 0 || K <= 0 || !slot_ok(slot, count)) return GLQ_ERR_ARG;
    const size_t elems = (size_t)N * K;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (fmt == GLQ_FMT_Q2 || fmt == GLQ_FMT_Q4) {
        dequant_tiled_q_kernel<<<(unsigned)((elems + 255) / 256), 256, 0, st>>>(
            fmt, reinterpret_cast<const unsigned char*>(tiled), N, K, slot, count, reinterpret_cast<__half*>(out));
    } else if (fmt == GLQ_FMT_T2) {
        if (!norms_tiled || !centroids) return GLQ_ERR_ARG;
        dequant_tiled_t2_kernel<<<(unsigned)((elems + 255) / 256), 256, 0, st>>>(
            reinterpret_cast<const unsigned char*>(tiled), norms_tiled, centroids, N, K, slot, count,
            reinterpret_cast<float*>(out));
    } else {
        return GLQ_ERR_UNSUPPORTED;
    }
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

// ---------------------------------------------------------------------------------------------
// First bounds violation recorded by a self-checking kernel: {code, index, limit, block<<32|thread};
// all zero when there was none.  Synchronises the device.
// ---------------------------------------------------------------------------------------------
// ---------------------------------------------------------------------------------------------
// randomized Hadamard rotation
// ---------------------------------------------------------------------------------------------
template <typename TI, typename TO>
static int launch_rht(const void* x, int64_t ldx, const float* signs, int rows, int d, int n, float scale, void* y,
                      int64_t ldy, cudaStream_t st) {
    const size_t smem = (size_t)n * sizeof(float);
    auto kern = rht_kernel<TI, TO>;
    if (smem > 48 * 1024) GLQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<rows, 256, smem, st>>>(reinterpret_cast<const TI*>(x), ldx, signs, d, n, scale, reinterpret_cast<TO*>(y), ldy);
    GLQ_CUDA(cudaGetLastError());
    return GLQ_OK;
}

extern "C" int glq_rht_forward(const void* x, int x_is_f32, int64_t ldx, const float* signs, int rows, int d, float scale,
                               void* y, int y_is_f32, int64_t ldy, void* stream) {
    if (!x || !y || !signs || rows < 0 || d <= 0) return GLQ_ERR_ARG;
    if (rows == 0) return GLQ_OK;
    int n = 1;
    while (n < d) n <<= 1;
    if (n > 32768) return GLQ_ERR_UNSUPPORTED;       // n floats of shared memory per row
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (x_is_f32 && y_is_f32) return launch_rht<float, float>(x, ldx, signs, rows, d, n, scale, y, ldy, st);
    if (!x_is_f32 && !y_is_f32) return launch_rht<__half, __half>(x, ldx, signs, rows, d, n, scale, y, ldy, st);
    if (x_is_f32) return launch_rht<float, __half>(x, ldx, signs, rows, d, n, scale, y, ldy, st);
    return launch_rht<__half, float>(x, ldx, signs, rows, d, n, scale, y, ldy, st);
}

int glq_moe_error_words(unsigned long long* out4, int clear);   // moe.cu: the error word of that translation unit

extern "C" int glq_debug_error(unsigned long long* out4, int clear) {
    if (!out4) return GLQ_ERR_ARG;
    GLQ_CUDA(cudaMemcpyFromSymbol(out4, g_glq_err, 4 * sizeof(unsigned long long)));
    if (clear) {
        unsigned long long z[4] = {0, 0, 0, 0};
        GLQ_CUDA(cudaMemcpyToSymbol(g_glq_err, z, sizeof(z)));
    }
    unsigned long long m[4] = {0, 0, 0, 0};
    const int rc = glq_moe_error_words(m, clear);
    if (rc != GLQ_OK) return rc;
    if (out4[0] == 0 && m[0] != 0)
        for (int i = 0; i < 4; ++i) out4[i] = m[i];
    return GLQ_OK;
}
