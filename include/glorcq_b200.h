/*
 * glorcq_b200 -- C ABI of the B200 (sm_100a) kernels for the GLoRCQ real-quant inference path:
 *     y = x . dequant(Wq)^T + (x . U) . SV^T      (U shared by clustered experts)
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless said otherwise, every
 * function enqueues on the given stream (a cudaStream_t passed as void*) and never synchronises,
 * so all of them can be captured into a CUDA graph.  Return value: GLQ_OK or a negative GLQ_ERR_*;
 * argument errors are decided on the host before anything is launched.
 *
 * The entry points named glq_turbo_* / glq_gptq_* take exactly the tensors that the reference's
 * two native modules take (inference/kernels/turbo_matmul.cu:255-318, 417-464 and
 * inference/kernels/gptq_matmul.cu:223-315), except that the caller owns the output buffer.
 * The other entry points work on weights re-tiled once at load time (glq_pack_*), which is what
 * the Python classes in glorcq_b200 use.
 */
#ifndef GLORCQ_B200_H
#define GLORCQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GLQ_OK 0
#define GLQ_ERR_ARG (-1)         /* null pointer, negative or inconsistent size */
#define GLQ_ERR_ALIGN (-2)       /* pointer or leading dimension not aligned as required */
#define GLQ_ERR_UNSUPPORTED (-3) /* shape / group size / rank outside what the kernels cover */
#define GLQ_ERR_CUDA (-4)        /* a CUDA call failed; see glq_last_cuda_error() */
#define GLQ_ERR_WORKSPACE (-5)   /* workspace too small */

/* weight formats of the tiled (load-time) layout */
#define GLQ_FMT_Q2 0  /* 2-bit integer codes, fp16 scale and zero per (row, group)       */
#define GLQ_FMT_Q4 1  /* 4-bit integer codes, fp16 scale and zero per (row, group)       */
#define GLQ_FMT_T2 2  /* 2-bit codebook indices, fp32 norm per row, 4-entry fp32 codebook */
#define GLQ_FMT_F16 3 /* dense fp16                                                        */

/* epilogues of glq_grouped_matmul */
#define GLQ_EPI_LINEAR 0 /* y = fp16(fp16(q-part) + fp16(low-rank part)) [* entry scale] [+ bias] */
#define GLQ_EPI_SWIGLU 1 /* fused gate|up weight: y = silu(gate(x)) * up(x)                            */

/* One weight matrix in the tiled layout (all device pointers; unused ones NULL). */
typedef struct glq_weight {
    const void* codes;      /* tiled codes with their scales (Q2/Q4/T2) or tiled fp16 values (F16) */
    const void* reserved0;
    const float* norms;     /* T2: per-row norms in tile order                                   */
    const float* centroids; /* T2: (4,) fp32; (8,) for a fused gate|up weight: gate's, then up's  */
    const void* sv;         /* packed output-side low-rank factor, or NULL                       */
    const void* bias;       /* (N,) fp16 or NULL (GLQ_EPI_LINEAR only)                           */
    int32_t N;              /* output features                                                   */
    int32_t K;              /* input features                                                    */
    int32_t rank;           /* low-rank width (multiple of 16), 0 = none                         */
    int32_t reserved;
} glq_weight_t;

/* ---------------------------------------------------------------------------------------------
 * Library information
 * ------------------------------------------------------------------------------------------ */
int glq_version(void);
const char* glq_status_string(int status);
int glq_last_cuda_error(void); /* cudaError_t of the last failed CUDA call on this thread */

/* ---------------------------------------------------------------------------------------------
 * Drop-ins for the reference's native modules (row-major, un-tiled operands).
 * ------------------------------------------------------------------------------------------ */

/* turbo_dequant_matmul (inference/kernels/turbo_matmul.cu:255-318):
 *   y[b,n] = norms[n] * sum_k centroids[idx(n,k)] * x_rot[b,k]
 * x_rot (B,K) fp16, packed (N,K/4) uint8 (code j of a byte in bits [2j,2j+1]), norms (N,) fp32,
 * centroids (4,) fp32, y (B,N) fp16.  K % 4 == 0.  B == 0 or N == 0 returns GLQ_OK, no launch. */
int glq_turbo_dequant_matmul(const void* x_rot, const uint8_t* packed, const float* norms, const float* centroids,
                             void* y, int B, int N, int K, void* stream);

/* turbo_dequant_grouped_gemv (inference/kernels/turbo_matmul.cu:417-464): E independent GEMVs,
 * expert e uses x_grouped[e,:] and rows [e*N_out, (e+1)*N_out).  y (E*N_out,) fp16. */
int glq_turbo_dequant_grouped_gemv(const void* x_grouped, const uint8_t* packed_cat, const float* norms_cat,
                                   const float* centroids, void* y, int E, int N_out, int K, void* stream);

/* gptq_dequant_matmul (inference/kernels/gptq_matmul.cu:223-315):
 *   y[b,n] = sum_k (q[n,k] - zeros[n,k/g]) * scales[n,k/g] * x[b,k]  (+ lora_out[b,n])
 * x (B,K) fp32, q (N,K) int8 (any int8 value), scales/zeros (N,n_groups) fp16, lora_out (B,N) fp32
 * or NULL, y (B,N) fp32; sym != 0 ignores zeros. */
int glq_gptq_dequant_matmul(const float* x, const int8_t* q, const void* scales, const void* zeros,
                            const float* lora_out, float* y, int B, int N, int K, int groupsize, int n_groups,
                            int sym, void* stream);

/* glq_turbo_dequant_matmul_static -- no counterpart in the reference.
 * Same operands and result as glq_turbo_dequant_matmul, for hosts that cannot allocate device
 * memory on this path and have no workspace to lend: for example a serving process that hands all
 * device memory to one arena at start-up and forbids cudaMalloc afterwards (it synchronises the
 * device and fragments the arena), or a plugin called from a thread that does not own an allocator.
 * The k dimension is split over CTAs so that one small matmul still occupies every SM; the partial
 * sums and arrival counters of that split live in a fixed array inside the library image
 * (glq_static_scratch_bytes() = 4 MiB plus 16 KiB of counters; every GPU that loads the library
 * holds it until the process exits).  Nothing is allocated or freed by this call.
 *   - Problems whose split needs more than that are refused with GLQ_ERR_WORKSPACE.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress with
 *     that device current); make that first call before any stream capture begins.
 *   - All calls share the one array, which keeps the previous call's contents; the counters are
 *     cleared on the stream before each launch, but two calls that overlap on the GPU (different
 *     streams, or different host threads) race on it: serialise them. */
size_t glq_static_scratch_bytes(void);
/* bytes of the fixed array a call with these sizes would use: 0 when the planned launch does not split k
 * (it then never touches the array), more than glq_static_scratch_bytes() when the call would be refused */
size_t glq_static_scratch_needed(int B, int N, int K);
int glq_turbo_dequant_matmul_static(const void* x_rot, const uint8_t* packed, const float* norms,
                                    const float* centroids, void* y, int B, int N, int K, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Load-time re-tiling (device to device).  Rows are grouped in tiles of 16, tiles in pairs.
 *   Q2  : [pair][k block of 128][tile in pair][576 B]; a block is 32 lanes x 16 B of codes -- lane
 *         4g+t holds codes k = 128*kb + 32*t + 0..31 of row 16*i+g (words 0,1) and of row 16*i+g+8
 *         (words 2,3) -- followed by 8 x (scale g, zero g, scale g+8, zero g+8) fp16 of the block's group
 *   Q4  : the same with k blocks of 64 (16 codes per lane and row)
 *   T2  : [pair][k block of 128][tile in pair][512 B] of codebook indices; norms in tile order
 *   F16 : [row tile][k block of 64][k step 0..3][lane][4 x half2] = the m16n8k16 A fragment
 *   SV  : [pair][64-column slice][32 rows of the pair][64 columns] fp16
 * Source tile i of a matrix lands in destination tile i*count + slot: count = 1 is a plain matrix,
 * count = 2 interleaves two matrices of one shape tile by tile (slot 0 = gate, slot 1 = up), so that
 * a pair is (gate tile p, up tile p) and one launch computes silu(gate x) * (up x).  The
 * destination buffers must be zero-filled before packing (padding tiles are not written).
 * These replace the (N,K) int32 / (N,K/4) uint8 / (N,G) fp16 tensors stored by the reference's
 * quantizer (joint_optim.py:319-327; turbo_weight_quantizer.py:149-156).
 * ------------------------------------------------------------------------------------------ */
size_t glq_tiled_bytes(int fmt, int n_rows, int K, int count);       /* codes (+ scales) buffer */
size_t glq_sv_bytes(int n_rows, int rank, int count);                /* packed SV buffer         */
size_t glq_rows_f32_count(int n_rows, int count);                    /* floats of a tile-ordered row vector */

/* codes (N,K) int32 in [0, 2^bits), scales/zeros (N,G) fp16 (zeros NULL: symmetric) -> Q2 / Q4 */
int glq_pack_gptq(const int32_t* q, const void* scales, const void* zeros, int bits, int N, int K, int group_size,
                  void* tiled, int slot, int count, void* stream);
/* packed (N,K/4) uint8 2-bit indices -> T2 */
int glq_pack_turbo(const uint8_t* packed, int N, int K, void* tiled, int slot, int count, void* stream);
/* (N,) fp32 row values (norms) -> tile order */
int glq_pack_rows_f32(const float* v, int N, float* out, int slot, int count, void* stream);
/* SV (N, rank) fp16 row-major -> packed SV */
int glq_pack_sv(const void* sv, int N, int rank, void* out, int slot, int count, void* stream);
/* W fp16 -> tiled F16.  element (n,k) is read from W[n*stride_n + k*stride_k] */
size_t glq_tiled_f16_bytes(int N, int K);
int glq_pack_f16(const void* W, long stride_n, long stride_k, int N, int K, void* tiled, void* stream);

/* Dequantised weights of the matrix in (slot, count) of a tiled buffer, for bit-exact checks against
 * the reference's tiles: Q2/Q4 -> out (N,K) fp16 = fp16((q - z) * s) (inference/quantized_linear.py:271-284);
 * T2 -> out (N,K) fp32 = centroids[idx] * norm (inference/kernels/__init__.py:142-143). */
int glq_dequant_tiled(int fmt, const void* tiled, const float* norms_tiled, const float* centroids, int N, int K,
                      int slot, int count, void* out, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Grouped skinny matmul: the decode GEMV / batched-decode kernel.
 *
 * For every live problem slot s (s < *n_slots, or all n_problems):
 *     rows   = slot_count[s] activation rows ("entries" slot_offset[s] .. +rows)
 *     weight = table[slot_index[s]]
 *     x row of entry e   = x + entry_row[e] * ldx      (entry_row NULL: e)
 *     y row of entry e   = y + e * ldy
 *     a row of entry e   = a + e * lda                 (precomputed x.U, fp16, width rank)
 * and y = epilogue(x . dequant(W)^T, a . SV^T).  All slots share format, shape and group size.
 * With table == NULL the inline descriptor is used for every slot.  GLQ_EPI_SWIGLU takes a fused
 * gate|up weight (count = 2 above), N is then the width of each of the two, a0 / a1 are x.U of the
 * gate / up cluster.
 * ------------------------------------------------------------------------------------------ */
typedef struct glq_mm_args {
    int32_t fmt;         /* GLQ_FMT_* */
    int32_t group_size;  /* Q2: multiple of 128; Q4: multiple of 64; others ignored */
    int32_t epilogue;    /* GLQ_EPI_* */
    int32_t n_problems;  /* slots covered by the grid */
    int32_t max_rows;    /* upper bound of rows per slot (sizes shared memory and passes) */
    int32_t rows_stride; /* entries reserved per slot when slot_offset is NULL */
    int32_t N, K, rank;  /* shape shared by all slots */
    int32_t total_rows;  /* upper bound of the entries of all slots together (sizes the workspace of the
                            many-row path); 0: n_problems * max_rows */
    glq_weight_t w;              /* inline descriptor */
    const glq_weight_t* w_table; /* device array indexed by slot_index[], or NULL */
    const int32_t* slot_index;  /* device, NULL: identity */
    const int32_t* n_slots;     /* device scalar, NULL: n_problems */
    const int32_t* slot_count;  /* device, NULL: max_rows for every slot */
    const int32_t* slot_offset; /* device, NULL: slot * rows_stride */
    const int32_t* entry_row;   /* device, NULL: identity */
    const void* entry_scale;    /* device fp16 per entry, NULL: none (GLQ_EPI_LINEAR only) */
    const void* x;  int64_t ldx;   /* fp16 */
    const void* a0; const void* a1; int64_t lda; /* fp16 x.U per entry, NULL: no low-rank term */
    void* y;        int64_t ldy;   /* fp16 */
    void* workspace; size_t workspace_bytes; /* scratch: split-k partial sums, or the re-tiled activations
                                                of the many-row path (contents irrelevant)               */
    int32_t* counters; size_t n_counters;    /* arrival counters: zero before the first use, left zero   */
    int32_t flags;    /* GLQ_MM_* */
    int32_t reserved;
} glq_mm_args_t;
/* a0 / a1 are written by the launch issued on this stream immediately before this call, and nothing
 * else this call reads is: the kernel may then be launched programmatically dependent (it starts while
 * that launch still runs and waits for it only before the low-rank term). */
#define GLQ_MM_A_FROM_PREVIOUS_LAUNCH 1
/* The operation issued on this stream immediately before this call is a kernel launch of this library
 * (no event wait or foreign work in between): the launch may be programmatically dependent on it; the
 * kernel waits for that launch before its first load. */
#define GLQ_MM_AFTER_KERNEL 2
/* Another stream runs grouped products at the same time: use two thirds of the CTA slots, so that both find room. */
#define GLQ_MM_SHARE_SM 4

/* Scratch bytes / arrival counters a call with these args needs (both 0 when no CTA-level k split is
 * used).  The counters must be zero when a call starts and are zero again when it ends, so one
 * zero-initialised array can serve any sequence of calls on one stream; the scratch needs no
 * initialisation. */
size_t glq_mm_workspace_bytes(const glq_mm_args_t* args);
size_t glq_mm_counters(const glq_mm_args_t* args);
int glq_grouped_matmul(const glq_mm_args_t* args, void* stream);

/* Randomized Hadamard rotation of activation rows (rht_forward, hadamard_rotation.py:50-65, which
 * multiplies by the signs and calls the third-party fast-hadamard-transform):
 *   y[row] = scale * H_n * (signs . x[row]),  H_n in natural (Sylvester) order, n = next power of two >= d;
 * x is zero-padded to n and the first d outputs are kept.  x / y are fp16 or fp32 ((rows, d), leading
 * dimensions in elements), signs (d,) fp32; the butterflies run in fp32.  n <= 32768. */
int glq_rht_forward(const void* x, int x_is_f32, int64_t ldx, const float* signs, int rows, int d, float scale, void* y,
                    int y_is_f32, int64_t ldy, void* stream);

/* First bounds violation or timed-out wait recorded by a kernel: {code, index, limit,
 * block<<32|thread}, all zero when there was none.  Synchronises the device; clear != 0 resets it. */
int glq_debug_error(unsigned long long* out4, int clear);

/* One quantized linear layer on B activation rows (GLoRCQLinear.forward,
 * inference/quantized_linear.py:286-355): y = Q(x) + a . SV^T + bias with a = x . U given by the
 * caller (`a`, (B,rank) fp16), or computed here from `ut` (U^T in the tiled F16 layout) into the
 * workspace, or absent (a == NULL and ut == NULL). */
int glq_linear_forward(int fmt, int group_size, const glq_weight_t* w, const void* ut, const void* x, int64_t ldx,
                       const void* a, void* y, int64_t ldy, int B, void* workspace, size_t workspace_bytes,
                       int32_t* counters, size_t n_counters, void* stream);
size_t glq_linear_workspace_bytes(int fmt, int group_size, const glq_weight_t* w, int B);
size_t glq_linear_counters(int fmt, int group_size, const glq_weight_t* w, int B);

/* ---------------------------------------------------------------------------------------------
 * MoE block forward (GraphCompatibleMoeBlock.forward, inference/moe_block.py:381-436), entirely on
 * the device: router matmul, softmax in fp32, top-k, optional renormalisation, per-expert token
 * lists, x.U per routed expert, fused gate|up with SwiGLU, down projection scaled by the routing
 * weight, shared expert with its sigmoid gate, combine.  No host synchronisation and fixed launch
 * shapes, so the whole call can be captured into a CUDA graph; only the routed experts' weights are
 * read.  The weighted sum over a token's experts is done in fp16 in top-k slot order for up to
 * `slot_order_max_tokens` tokens (the reference's decode loop, inference/moe_block.py:474-476) and
 * in expert order above (index_add over experts, inference/moe_block.py:716-739).
 * ------------------------------------------------------------------------------------------ */
typedef struct glq_moe_desc {
    int32_t H, I, E, top_k;
    int32_t I_shared;        /* 0: no shared expert */
    int32_t rank;            /* low-rank width of every projection (0: none) */
    int32_t fmt, group_size; /* format of the expert projections */
    int32_t norm_topk_prob;
    int32_t router_rows;     /* E, or E+1 when row E is the shared expert's gate */
    int32_t slot_order_max_tokens;
    int32_t reserved;
    const void* router_t;          /* tiled F16 (dense0_rows x H): the router rows, optionally followed (from row
                                      sh_a_row, a multiple of 16) by the shared expert's U_gate^T and U_up^T so
                                      that one dense product yields logits, shared gate logit and both x.U */
    const glq_weight_t* gate_up;   /* device table [E]: fused gate|up, N = I */
    const glq_weight_t* down;      /* device table [E]: N = H, K = I */
    const glq_weight_t* ut_gate_up; /* device table [2E] of dense U^T (rank x H): gate of expert e at e, up at E+e */
    const glq_weight_t* ut_down;    /* device table [E] of dense U^T (rank x I); both NULL when rank == 0 */
    int32_t dense0_rows;            /* rows of router_t (== router_rows when nothing is appended) */
    int32_t sh_a_row;               /* first appended row, 0 when nothing is appended */
    glq_weight_t sh_gate_up, sh_down;            /* shared expert (ignored when I_shared == 0) */
    const void* sh_ut_gate; const void* sh_ut_up; const void* sh_ut_down; /* tiled U^T or NULL */
    /* codebook format only: rotations applied to the input of the quantized product (the low-rank
     * term sees the unrotated input), as tiled F16 matrices Pi (y = x . Pi^T), or NULL for identity:
     * H x H before gate/up, I x I before down, I_shared x I_shared before the shared down */
    const void* rot_in; const void* rot_mid; const void* sh_rot_mid;
    /* the same three rotations as randomized Hadamard transforms: (dim,) fp32 sign vectors, or NULL; a sign
     * vector takes precedence over the dense matrix of the same position (scale 1/sqrt(dim)) */
    const float* rht_in; const float* rht_mid; const float* sh_rht_mid;
    /* Optional plain row-major fp16 copies of the dense operands.  With them (and 2/4-bit integer codes, up to 4
     * tokens, the block's own router) the whole block up to the per-entry down outputs runs as ONE persistent
     * cooperative kernel instead of nine launches; all NULL: the launches above.  router_rm: the rows of router_t
     * (dense0_rows x H).  ut_rm_gate_up / ut_rm_down: device arrays of 2E / E pointers to U^T (rank x H / rank x I)
     * in the order of ut_gate_up / ut_down.  sh_ut_rm_down: U^T (rank x I_shared) of the shared down projection
     * (needed only when the shared expert has a low-rank term). */
    const void* router_rm;
    const void* const* ut_rm_gate_up;
    const void* const* ut_rm_down;
    const void* sh_ut_rm_down;
} glq_moe_desc_t;

/* 1 when a call with this descriptor and token count (and the block's own router) runs the persistent kernel */
int glq_moe_uses_fused_kernel(const glq_moe_desc_t* d, int n_tokens);
/* Diagnostic: with GLQ_FUSED_TRACE set in the environment, thread 0 of every CTA of the persistent kernel stamps
 * the GPU's global timer (ns) after each of its steps; this copies the stamps of the last launch ([CTA][16]
 * words, followed by the final values of the kernel's arrival counters; n_words <= 4352) to the host.  Synchronise first. */
int glq_moe_fused_trace(unsigned long long* out, int n_words);
size_t glq_moe_workspace_bytes(const glq_moe_desc_t* d, int n_tokens);
size_t glq_moe_counters(const glq_moe_desc_t* d, int n_tokens);
/* x (n_tokens, H) fp16 -> out (n_tokens, H) fp16; router_logits (n_tokens, E) fp16 may be NULL.
 * sel_out (n_tokens, top_k) int32 and weight_out (n_tokens, top_k) fp16 may be NULL. */
/* aux_stream (cudaStream_t), ev_fork, ev_join (cudaEvent_t): when all three are given, the shared
 * expert's launches go to aux_stream, forked from `stream` after the router product and joined before
 * the combine, so that they overlap the routed experts (captured as a parallel branch of a graph);
 * NULL runs everything on `stream`. */
int glq_moe_forward(const glq_moe_desc_t* d, const void* x, int n_tokens, void* out, void* router_logits,
                    int32_t* sel_out, void* weight_out, void* workspace, size_t workspace_bytes, int32_t* counters,
                    size_t n_counters, void* stream, void* aux_stream, void* ev_fork, void* ev_join);

/* Expert-parallel form of the same block.  The reference runs every expert on one device; its call
 * site is still GraphCompatibleMoeBlock.forward (inference/moe_block.py:381-436).  Rank r of `world`
 * holds the experts e with e mod world == r (the other entries of the gate_up / down / ut tables are
 * never read); router and shared expert are replicated.  Every rank numbers the (token, expert)
 * entries alike, writes the weighted down-projection rows of its own experts into `entry_out`
 * ((n_tokens*top_k, H) fp16, caller-owned) and leaves the others zero, so that a sum all-reduce of
 * the ranks' buffers is exact (one non-zero term per row) and the combine that follows gives
 * bit-identical results for every world size.  The exchange itself is the caller's:
 *   phase EXPERTS  -> all-reduce(entry_out) on `stream` -> phase COMBINE.
 * ep == NULL, or world == 1 with phase ALL, is glq_moe_forward. */
enum { GLQ_MOE_PHASE_ALL = 0, GLQ_MOE_PHASE_EXPERTS = 1, GLQ_MOE_PHASE_COMBINE = 2, GLQ_MOE_PHASE_EXCHANGE = 3 };
/* The exchange as one kernel of this library over peer-mapped memory (NVLink / NVSwitch), instead of the
 * caller's all-reduce:  phase EXPERTS (entry_out = a rank-local staging buffer) -> phase EXCHANGE -> phase
 * COMBINE.  Phase EXCHANGE stores the rows of this rank's experts into every rank's exchange buffer
 * (plain peer stores, 16 B each), publishes the step number in every rank's flag words and waits, for at
 * most a second, until every rank has published the same step; a wait that runs out sets *error and the
 * kernel returns.  The buffers have two halves used by alternate steps, so that a rank one step ahead
 * never writes rows another rank still reads; phase COMBINE reads the half of the last exchanged step.
 * entry_bufs and flags are device arrays of `world` pointers valid on this device (each rank's buffer of
 * 2*half_elems fp16 and its `world` int32 flag words, zeroed once before the first step); epoch and
 * error are this rank's own device words, zeroed once.  All ranks must run the same sequence of steps. */
typedef struct glq_ep_peers {
    void* const* entry_bufs; int32_t* const* flags;
    int32_t* epoch; int32_t* error;
    size_t half_elems;
    uint64_t wait_limit_ns; /* longest wait for the other ranks' flags, in nanoseconds of the GPU's global timer; 0: one
                               second.  *error keeps the step number of the FIRST wait that ran out (0: none); the
                               host reads it at its own synchronisation points and must not use results of later steps */
} glq_ep_peers_t;
/* flags of glq_moe_ep_t: phase EXPERTS leaves the rows of other ranks' entries unwritten instead of zeroing
 * them (the peer-memory exchange copies only this rank's rows; an all-reduce needs the zeros) */
#define GLQ_MOE_EP_NO_ZERO_FILL 1
typedef struct glq_moe_ep {
    int32_t rank, world, phase, flags; /* GLQ_MOE_EP_* */
    void* entry_out; /* NULL: use the workspace (world == 1 only) */
    /* Routing decided by the caller instead of the block's router (the fused-experts adapter
     * GLoRCQExperts.forward, inference/quantized_linear.py:395-428): sel_in (n_tokens, top_k) int32 expert
     * indices (an index outside [0, E) drops the slot), weight_in (n_tokens, top_k) fp16; both NULL for
     * the block's own router.  Needs I_shared == 0 and router_logits == NULL; router_t is not read. */
    const int32_t* sel_in; const void* weight_in;
    /* The decoder's steps after the block (the transformers layer adds the residual and the next layer norm
     * follows; the reference leaves both to that host model), folded into the combine: when normed_out is set,
     * out = residual + block output (residual (n_tokens, H) fp16 or NULL) and normed_out (n_tokens, H) fp16 =
     * rms_norm(out, norm_eps) * norm_weight ((H,) fp16, NULL = ones).  H <= 8192. */
    const void* residual; const void* norm_weight; void* normed_out;
    float norm_eps; int32_t reserved2;
    const glq_ep_peers_t* peers; /* phases EXCHANGE and COMBINE: the peer-memory exchange; NULL otherwise */
} glq_moe_ep_t;
int glq_moe_forward_ep(const glq_moe_desc_t* d, const void* x, int n_tokens, void* out, void* router_logits,
                       int32_t* sel_out, void* weight_out, void* workspace, size_t workspace_bytes, int32_t* counters,
                       size_t n_counters, void* stream, void* aux_stream, void* ev_fork, void* ev_join,
                       const glq_moe_ep_t* ep);

/* ---------------------------------------------------------------------------------------------
 * One decode step of grouped-query attention over a static key/value cache, in one launch.  The
 * reference leaves attention to the transformers modules it wraps (inference/graph_wrapper.py:84-127
 * calls the model with a StaticCache); this entry point serves the host model of this package.
 * q (B, n_heads*head_dim), k_new / v_new (B, n_kv*head_dim) fp16 as the projections produce them;
 * optional per-head RMS-norm weights (head_dim,) fp16 for q and k; rotary embedding in the rotate-half
 * convention from cos / sin tables (max positions, head_dim) fp16 at position *pos (device int64, so a
 * captured launch follows the replayed position); the new key / value are stored into the caches
 * (B, n_kv, max_len, head_dim) fp16 at that position; out (B, n_heads*head_dim) fp16 =
 * softmax(q k^T / sqrt(head_dim)) v over positions 0..*pos.  head_dim in {32, 64, 128, 256}.
 * The cached positions of a head are split over several CTAs when the cache is long; their partial
 * results go through `workspace` (glq_attn_decode_workspace_bytes; contents irrelevant) and are merged
 * by the CTA that arrives last; `counters` (B * n_heads ints) must be zero before the first call and are
 * left zero. */
size_t glq_attn_decode_workspace_bytes(int B, int n_heads, int head_dim, int max_len);
int glq_attn_decode(const void* q, const void* k_new, const void* v_new, const void* cos_t, const void* sin_t,
                    const int64_t* pos, void* k_cache, void* v_cache, void* out, int B, int n_heads, int n_kv,
                    int head_dim, int max_len, const void* q_norm_w, const void* k_norm_w, float eps, void* workspace,
                    size_t workspace_bytes, int32_t* counters, size_t n_counters, void* stream);

/* The prompt's form of the first half of glq_attn_decode: q (B, T, n_heads, head_dim) and k (B, T, n_kv, head_dim) get
 * the optional per-head RMS norm and the rotary embedding of positions[t] in place; the new keys and v (B, T, n_kv,
 * head_dim) are written into the static cache at positions[t] (host-model glue; the reference lets the transformers
 * attention modules do this, inference/graph_wrapper.py:84-127).  head_dim 32, 64, 128 or 256. */
int glq_rope_prefill(void* q, void* k, const void* v, const void* cos_t, const void* sin_t, const int64_t* positions,
                     void* k_cache, void* v_cache, int B, int T, int n_heads, int n_kv, int head_dim, int max_len,
                     const void* q_norm_w, const void* k_norm_w, float eps, void* stream);

/* Causal attention of a prompt written at positions 0..T-1, after glq_rope_prefill: y[b, t, h] =
 * softmax(q[b, t, h] . k[b, 0..t, h / group]^T / sqrt(head_dim)) v[b, 0..t, h / group], fp16 with fp32 accumulation;
 * q and y (B, T, n_heads, head_dim), k and v (B, T, n_kv, head_dim), contiguous and 16-byte aligned; only the keys up
 * to each query are read.  head_dim 64 or 128 (GLQ_ERR_UNSUPPORTED otherwise).  Host-model glue: the reference lets
 * the transformers attention modules do this (inference/graph_wrapper.py:84-127). */
int glq_attn_prefill(const void* q, const void* k, const void* v, void* y, int B, int T, int n_heads, int n_kv,
                     int head_dim, void* stream);

/* x_out = x + delta and h_out = rms_norm(x_out, eps) * weight on (rows, H) fp16 rows (weight (H,) fp16 or NULL):
 * the residual add and layer norm between the attention output projection and the MoE block of a decoder layer
 * (host-model glue, as glq_attn_decode).  H a multiple of 8, at most 8192. */
int glq_add_rmsnorm(const void* x, const void* delta, const void* weight, float eps, int rows, int H, void* x_out,
                    void* h_out, void* stream);

/* Output projection of the decoder with the greedy arg-max folded in: logits (B, V) fp16 = x (B, H) . W^T for
 * a dense fp16 W (V, H) in the checkpoint's row-major layout (the `lm_head` of the transformers model the
 * reference wraps; its decode loop takes the arg-max of the last position after every replay,
 * inference/graph_wrapper.py:186-208).  B <= 8 rows, H a multiple of 32 (<= 8192), x and W 16-byte aligned.
 * logits may be NULL (arg-max only) and argmax_out ((B,) int64: lowest index of the largest fp16-rounded
 * logit per row) may be NULL (logits only).  With argmax_out: workspace of glq_lm_head_workspace_bytes()
 * (contents irrelevant) and one int32 counter that is zero before the first call and left zero. */
size_t glq_lm_head_workspace_bytes(void);
int glq_lm_head(const void* x, int64_t ldx, const void* W, int B, int V, int H, void* logits, int64_t ldl,
                int64_t* argmax_out, void* workspace, size_t workspace_bytes, int32_t* counter, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GLORCQ_B200_H */
