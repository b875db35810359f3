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
#define GLQ_EPI_SWIGLU 1 /* two weights w0 (gate), w1 (up): y = silu(lin0(x)) * lin1(x)           */

/* One weight matrix in the tiled layout (all device pointers; unused ones NULL). */
typedef struct glq_weight {
    const void* codes;      /* tiled codes (Q2/Q4/T2) or tiled fp16 values (F16)                 */
    const void* sz;         /* Q2/Q4: tiled (scale, zero) fp16 pairs                             */
    const float* norms;     /* T2: (N,) fp32                                                     */
    const float* centroids; /* T2: (4,) fp32                                                     */
    const void* sv;         /* (N, rank) fp16 row-major output-side low-rank factor, or NULL     */
    const void* bias;       /* (N,) fp16 or NULL                                                 */
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

/* ---------------------------------------------------------------------------------------------
 * Load-time re-tiling (device to device).  Tiled layouts, rows in tiles of 16:
 *   Q2/T2: [row tile][k block of 128][lane 0..31][4 x u32]; lane = 4*g + t holds codes
 *          k = 128*kb + 32*t + 0..31 of row 16*rt+g (words 0,1) and of row 16*rt+g+8 (words 2,3)
 *   Q4   : same with k blocks of 64, 16 codes per lane and row
 *   F16  : [row tile][k block of 64][k step 0..3][lane][4 x half2] = the m16n8k16 A fragment
 *   sz   : [row tile][group][g 0..7][scale g, zero g, scale g+8, zero g+8] fp16
 * replacing the (N,K) int32 / (N,K/4) uint8 / (N,G) fp16 tensors stored by the reference's
 * quantizer (joint_optim.py:319-327; turbo_weight_quantizer.py:149-156).
 * ------------------------------------------------------------------------------------------ */
size_t glq_tiled_codes_bytes(int fmt, int N, int K);
size_t glq_tiled_sz_bytes(int N, int n_groups);

/* codes (N,K) int32 with values in [0, 2^bits) -> tiled Q2 (bits 2) or Q4 (bits 4) */
int glq_pack_codes_i32(const int32_t* q, int bits, int N, int K, void* tiled, void* stream);
/* packed (N,K/4) uint8 2-bit codes -> tiled T2 (or Q2) */
int glq_pack_codes_u8(const uint8_t* packed, int N, int K, void* tiled, void* stream);
/* scales, zeros (N,G) fp16 (zeros may be NULL: symmetric) -> tiled sz */
int glq_pack_sz(const void* scales, const void* zeros, int N, int n_groups, void* tiled, void* stream);
/* W fp16 -> tiled F16.  element (n,k) is read from W[n*stride_n + k*stride_k] */
int glq_pack_f16(const void* W, long stride_n, long stride_k, int N, int K, void* tiled, void* stream);

/* Dequantised weights from the tiled layout, for bit-exact checks against the reference's tiles:
 * Q2/Q4 -> out (N,K) fp16 = fp16((q - z) * s)  (inference/quantized_linear.py:271-284);
 * T2    -> out (N,K) fp32 = centroids[idx] * norm (inference/kernels/__init__.py:142-143). */
int glq_dequant_tiled(int fmt, const glq_weight_t* w, int group_size, void* out, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Grouped skinny matmul: the decode GEMV / batched-decode kernel.
 *
 * For every live problem slot s (s < *n_slots, or all n_problems):
 *     rows   = slot_count[s] activation rows ("entries" slot_offset[s] .. +rows)
 *     weight = table[slot_index[s]]
 *     x row of entry e   = x + entry_row[e] * ldx      (entry_row NULL: e)
 *     y row of entry e   = y + e * ldy
 *     a row of entry e   = a + e * lda                 (precomputed x.U, fp16, width rank)
 * and y = epilogue(x . dequant(W)^T, a . SV^T).  All slots share format, shape class and group
 * size.  With table == NULL the inline descriptor is used for every slot.
 * ------------------------------------------------------------------------------------------ */
typedef struct glq_mm_args {
    int32_t fmt;         /* GLQ_FMT_* */
    int32_t group_size;  /* Q2: multiple of 128; Q4: multiple of 64; others ignored */
    int32_t epilogue;    /* GLQ_EPI_* */
    int32_t n_problems;  /* slots covered by the grid */
    int32_t max_rows;    /* upper bound of rows per slot (sizes shared memory and passes) */
    int32_t rows_stride; /* entries reserved per slot when slot_offset is NULL */
    int32_t N, K, rank;  /* shape shared by all slots */
    int32_t reserved;
    glq_weight_t w0, w1;           /* inline descriptors (w1 only for GLQ_EPI_SWIGLU) */
    const glq_weight_t* w0_table;  /* device arrays indexed by slot_index[], or NULL */
    const glq_weight_t* w1_table;
    const int32_t* slot_index;  /* device, NULL: identity */
    const int32_t* n_slots;     /* device scalar, NULL: n_problems */
    const int32_t* slot_count;  /* device, NULL: max_rows for every slot */
    const int32_t* slot_offset; /* device, NULL: slot * rows_stride */
    const int32_t* entry_row;   /* device, NULL: identity */
    const void* entry_scale;    /* device fp16 per entry, NULL: none (GLQ_EPI_LINEAR only) */
    const void* x;  int64_t ldx;   /* fp16 */
    const void* a0; const void* a1; int64_t lda; /* fp16 x.U per entry for w0 / w1, NULL: no low-rank term */
    void* y;        int64_t ldy;   /* fp16 */
    void* workspace; size_t workspace_bytes; /* scratch for split-k partial sums (contents irrelevant)   */
    int32_t* counters; size_t n_counters;    /* arrival counters: zero before the first use, left zero   */
} glq_mm_args_t;

/* Scratch bytes / arrival counters a call with these args needs (both 0 when k is not split).  The
 * counters must be zero when a call starts and are zero again when it ends, so one zero-initialised
 * array can serve any sequence of calls on one stream; the scratch needs no initialisation. */
size_t glq_mm_workspace_bytes(const glq_mm_args_t* args);
size_t glq_mm_counters(const glq_mm_args_t* args);
int glq_grouped_matmul(const glq_mm_args_t* args, void* stream);

/* One quantized linear layer on B activation rows (GLoRCQLinear.forward,
 * inference/quantized_linear.py:286-355): y = Q(x) + a . SV^T + bias with a = x . U given by the
 * caller (`a`, (B,rank) fp16), or computed here from `ut` (U^T in the tiled F16 layout) into the
 * workspace, or absent (a == NULL and ut == NULL). */
int glq_linear_forward(int fmt, int group_size, const glq_weight_t* w, const void* ut, const void* x, int64_t ldx,
                       const void* a, void* y, int64_t ldy, int B, void* workspace, size_t workspace_bytes,
                       int32_t* counters, size_t n_counters, void* stream);
size_t glq_linear_workspace_bytes(int fmt, int group_size, const glq_weight_t* w, int B);
size_t glq_linear_counters(int fmt, int group_size, const glq_weight_t* w, int B);

#ifdef __cplusplus
}
#endif
#endif /* GLORCQ_B200_H */
