/*
 * reinstinct_cuda.h — C ABI of libreinstinct_cuda.so, the sm_100a (B200) backend for
 * the quantized-weight hot path of the reinstinct engine.
 *
 * This is the surface a `src/cuda` module binds in place of `src/hip`: one entry point
 * per launch wrapper of the reference's runtime, so launch geometry lives behind the
 * ABI instead of in the caller.  Plain pointers and sizes only.  Every pointer named
 * `*_dev` / w / xq / y / x is a DEVICE pointer unless the comment says host.
 *
 * Conventions (src/hip/mod.rs:19-22, src/runtime/qwen35.rs:4282-4292):
 *   - every call returns an int: 0 on success, a positive cudaError_t value, or a
 *     negative RC_ERR_* code; nothing aborts and nothing throws across the boundary;
 *   - launches are asynchronous on `stream` (a cudaStream_t / CUstream passed as
 *     void*, NULL = the default stream); no entry point allocates, frees,
 *     synchronises or reads back, so all of them are legal under stream capture;
 *   - the caller owns every buffer; inputs and outputs never alias;
 *   - weights are in the repacked-v2 layout of src/quant/<fmt>.rs::repack_for_matvec,
 *     read unchanged; activations cross the boundary as 40-byte BlockQ8 blocks
 *     (kernels/quantize_q8.cpp:16-21) that need only 8-byte alignment;
 *   - `ggml_type` is the GGUF discriminant (src/gguf/types.rs:16-35).
 */
#ifndef REINSTINCT_CUDA_H
#define REINSTINCT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RC_ABI_VERSION 1

/* src/gguf/types.rs:16-35 */
enum rc_ggml_type {
    RC_TYPE_Q4_0 = 2,
    RC_TYPE_Q5_1 = 7,   /* MoE expert tensors (src/runtime/qwen35.rs:421): Q5_K nibble and 5th-bit planes, then d | m << 16
                         * per sub-block (src/quant/q5_1.rs:62-100); the Q5_K kernel bodies with dsc = d, deff = -m */
    RC_TYPE_Q8_0 = 8,
    RC_TYPE_Q4_K = 12,
    RC_TYPE_Q5_K = 13,
    RC_TYPE_Q6_K = 14,
    RC_TYPE_IQ4_XS = 23,
    /* KERNEL type of an IQ3_S tensor (src/runtime/qwen35.rs:281-286): the repacked IQ4_XS planes
     * (16 nibble bytes and one fp16 scale per 32 weights) read through the codebook v = 2n - 15
     * (src/quant/iq3_s.rs:193-214).  Every matvec / GEMM entry point takes it; rc_repack_for_matvec
     * does not (RC_ERR_BAD_TYPE): the planes come from the caller's own iq3_s::repack_for_matvec
     * (src/quant/iq3_s.rs:216-260), which needs ggml's 512-entry grid table. */
    RC_TYPE_IQ3_S = 21,
    /* accepted by rc_repack_for_matvec / rc_ondisk_len as SOURCE types only: the loaders relabel
     * them onto one of the six above (src/runtime/qwen35.rs:274-307) */
    RC_SRC_Q3_K = 11,   /* exact: Q6_K blocks with q6 = q3 + 28, sc6 = sc3 - 32 (src/quant/q3_k.rs:92-121) */
    RC_SRC_IQ4_NL = 20, /* exact: the repacked IQ4_XS planes with d as the sub-block scale (src/quant/iq4_nl.rs:51-73) */
    RC_SRC_BF16 = 30    /* requantized to Q8_0 (src/quant/q8_0.rs:45-61) */
};

enum rc_error {
    RC_OK = 0,
    RC_ERR_BAD_TYPE = -1,      /* ggml_type not one of the six above                  */
    RC_ERR_BAD_SHAPE = -2,     /* in_dim not a multiple of the block size, zero dims  */
    RC_ERR_NULL_POINTER = -3,
    RC_ERR_MISALIGNED = -4,    /* weight base not 16-byte, BlockQ8 base not 8-byte    */
    RC_ERR_TOO_MANY_ROWS = -5, /* n_rows beyond what the entry point accepts          */
    RC_ERR_SCRATCH_TOO_SMALL = -6,
    RC_ERR_NO_DEVICE = -7,     /* no sm_100 device / kernels not loadable             */
    RC_ERR_BAD_ARGUMENT = -8,
    RC_ERR_STATIC_LIMIT = -9   /* size beyond the fixed scratch of rc_matvec_f32_noalloc     */
};

#define RC_BLOCKQ8_BYTES 40          /* kernels/quantize_q8.cpp:16-21 */
#define RC_MATVEC_MAX_ROWS 16        /* src/runtime/prefill.rs:42 MAX_BATCHED_ROWS */

/* ---- library ---------------------------------------------------------------- */

/* Selects `device`, checks it is compute capability 10.x and sets the kernels'
 * shared-memory attributes.  Call once per device before stream capture; the
 * launch entry points call it lazily for the current device otherwise.
 * Replaces KernelCache::compile + Module::load (src/runtime/mod.rs:195-245). */
int rc_init(int device);
int rc_abi_version(void);
/* Static string for any code returned by this library
 * (hip::Hip::err_str, src/hip/sys.rs:107-119). */
const char *rc_error_string(int code);

/* ---- layout helpers (host arithmetic only) ------------------------------------ */

/* src/quant/q4_k.rs:92-95 (same rule in q4_0.rs:60-63, q8_0.rs:68-71, iq4_xs.rs:79-82) */
size_t rc_repacked_n_sub_padded(size_t in_dim);
/* src/quant/<fmt>.rs::repacked_len; 0 for an unsupported type or shape */
size_t rc_repacked_len(int ggml_type, size_t in_dim, size_t out_dim);
/* bytes of the on-disk GGUF rows for the same shape; 0 if unsupported */
size_t rc_ondisk_len(int ggml_type, size_t in_dim, size_t out_dim);

/* The type whose kernels run tensors of `src_type` (itself for the six native types, Q6_K / IQ4_XS /
 * Q8_0 for RC_SRC_Q3_K / RC_SRC_IQ4_NL / RC_SRC_BF16); -1 if the type is not supported. */
int rc_kernel_type(int src_type);

/* On-disk GGUF rows (device) -> repacked-v2 planes (device), done on the GPU.
 * Produces byte-for-byte what src/quant/<fmt>.rs::repack_for_matvec produces on the
 * host (q4_0.rs:86-104, q4_k.rs:126-176, q5_k.rs:97-151, q6_k.rs:86-148,
 * q8_0.rs:93-119, iq4_xs.rs:106-136); the step GpuMatvecTensor::from_bytes_matvec
 * (src/runtime/qwen35.rs:251-331) performs at load.  A source-only type (RC_SRC_*) comes out as
 * the planes of rc_kernel_type(type), which is the type to pass to every other entry point; its
 * output size is rc_repacked_len(rc_kernel_type(type), ...).  `blocks_dev` needs 2-byte
 * alignment, `out_dev` 16-byte. */
int rc_repack_for_matvec(void *stream, int ggml_type, const void *blocks_dev,
                         size_t in_dim, size_t out_dim, void *out_dev);

/* ---- activation quantizer --------------------------------------------------------- */

/* launch_quantize_q8 (src/runtime/gemma4.rs:1495-1506),
 * launch_quantize_q8_into (src/runtime/qwen35.rs:3202-3211);
 * kernel quantize_q8_f32 (kernels/quantize_q8.cpp:23-54).
 * x f32 [n_vec][in_dim] -> xq BlockQ8 [n_vec][in_dim/32]; in_dim % 32 == 0. */
int rc_quantize_q8(void *stream, const float *x, void *xq, uint32_t in_dim, uint32_t n_vec);

/* ---- decode matvec ------------------------------------------------------------------- */

/* launch_matvec_xq8 (src/runtime/gemma4.rs:1526-1564),
 * launch_matvec_repacked_xq8 (src/runtime/qwen35.rs:2232-2280); kernels
 * matvec_{q4_0,q4k,q5k,q6k,q8_0,iq4xs}_repacked_f32.
 * y f32 [out_dim] = W[out_dim][in_dim] . xq[in_dim/32]. */
int rc_matvec(void *stream, int ggml_type, const void *w, const void *xq, float *y,
              uint32_t in_dim, uint32_t out_dim);

/* matmul_kquant_batched_into's kernel launch (src/runtime/prefill.rs:448-508),
 * bmm_batched_kquant (src/runtime/qwen35.rs:4085-4111); kernels
 * matvec_<fmt>_repacked_batched{,16}_f32.  1 <= n_rows <= RC_MATVEC_MAX_ROWS; Q8_0 is
 * accepted too (the reference has no batched Q8_0 kernel, prefill.rs:350-354).
 * xq [n_rows][in_dim/32], y f32 [n_rows][out_dim]. */
int rc_matvec_batched(void *stream, int ggml_type, const void *w, const void *xq, float *y,
                      uint32_t in_dim, uint32_t out_dim, uint32_t n_rows);

/* launch_matvec (src/runtime/gemma4.rs:1508-1520), launch_matvec_dispatch
 * (src/runtime/qwen35.rs:2179-2229): quantize x into the caller's xq scratch
 * ((in_dim/32)*40 bytes), then rc_matvec. */
int rc_matvec_f32(void *stream, int ggml_type, const void *w, const float *x, float *y,
                  uint32_t in_dim, uint32_t out_dim, void *xq_scratch, size_t scratch_bytes);

/* Same result as rc_matvec_f32, for callers that cannot hand in a scratch buffer and must not
 * allocate one: a decode thread for which cudaMalloc's device-wide synchronisation would stall
 * every stream, or a plug-in living inside a host runtime that has already reserved all of HBM
 * for its own pool, so that cudaMalloc would simply fail.  It has no counterpart in the
 * reference, whose wrappers always own an xq8 buffer (src/runtime/gemma4.rs:1508-1520).
 * The quantized activations go to a fixed array inside the library instead
 * (RC_NOALLOC_SCRATCH_BYTES of device memory, held by every GPU that loads the library until
 * the process exits); x, w and y are still the caller's.  in_dim above RC_NOALLOC_MAX_IN_DIM
 * returns RC_ERR_STATIC_LIMIT.  The call allocates and frees nothing.
 * The first call on each device looks the array's address up once (with that device current);
 * make that first call before any stream capture.  All calls on a device share the one array
 * and each overwrites the part it uses, so nothing needs clearing between calls, but two calls
 * whose kernels overlap on the GPU (different streams) race on it: keep them on one stream. */
#define RC_NOALLOC_SCRATCH_BYTES (64 * 1024)
#define RC_NOALLOC_MAX_IN_DIM ((RC_NOALLOC_SCRATCH_BYTES / RC_BLOCKQ8_BYTES) * 32)
int rc_matvec_f32_noalloc(void *stream, int ggml_type, const void *w, const float *x, float *y,
                          uint32_t in_dim, uint32_t out_dim);

/* Test and debug aid: the per-(activation row, weight row, sub-block) integers the
 * matvec forms before scaling.  idots int32 [n_rows][out_dim][in_dim/32][2]; slot 1 is
 * used by Q6_K only (the second 16-weight half, kernels/matvec_q6k_repacked.cpp:83-109). */
int rc_matvec_block_dots(void *stream, int ggml_type, const void *w, const void *xq,
                         int32_t *idots, uint32_t in_dim, uint32_t out_dim, uint32_t n_rows);

/* Measurement aid: overrides the matvec launch heuristics for the calling process (ks =
 * warps that split one weight row, grid_mult = CTAs launched per resident CTA slot; 0 restores
 * the heuristic; no_pdl != 0 launches the matvec and quantize kernels without programmatic
 * stream serialization).  No counterpart in the reference, whose geometry is fixed in its wrappers
 * (src/runtime/gemma4.rs:1530-1551). */
void rc_tune_matvec(int ks, int grid_mult, int no_pdl);
/* Measurement aid: force_dp4a != 0 sends the MMQ entry points through the dp4a kernel instead of
 * the tensor-core kernels.  The low byte of kind picks the kernel: 0 the default (rc_matmul: the
 * integer-operand f16 GEMM with a drain per sub-block; rc_mmq_gemm and the grouped GEMM: int8 operands,
 * Q6_K on the integer-operand f16 kernel of that family), 8 the int8-operand kernel and 16 the
 * integer-operand f16 kernel of the BlockQ8-input family everywhere (rc_matmul then quantizes to BlockQ8
 * / its planar form), 32 sends rc_matmul through the f16-DEQUANTIZED GEMM of rc_matmul_f16 (an
 * approximation) with (kind >> 8) & 0xFFF forcing its token-tile width (128, 256, 512) and kind >> 20 a
 * mask of pipeline parts it skips or traces (results then invalid).  With kind 16 the upper bits are the
 * skip mask of that kernel.  For A/B timing and cross-checking only. */
void rc_tune_mmq(int force_dp4a, int kind);
/* Reads (synchronously) the device-side status word: 0, or the codes of the bounded waits that
 * gave up: bits 0-7 the int8 GEMM, 8-11 the BlockQ8-input f16 GEMM, 12-15 the dense exact GEMM of
 * rc_matmul, 16-19 the peer gather / barrier, 20-23 the fused decode FFN (1 its grid barrier, 2 the wait for
 * the peers' intermediate records, 3 the wait for the peers' output rows), 24-31 the f16-dequantized GEMM.  A nonzero value means the
 * affected outputs are invalid; the context stays usable.  The words are sticky: they keep the
 * last code until rc_device_status_clear.  hipDeviceSynchronize + error check in the
 * reference's tests (src/runtime/kernels.rs) is the nearest counterpart. */
int rc_device_status(unsigned int *status);
/* The same read, then the words are reset to 0 (status may be NULL).  Call it with no kernel of
 * this library in flight. */
int rc_device_status_clear(unsigned int *status);
/* Measurement aid: copies out (synchronously) the phase timestamps the f16-operand GEMM records
 * per CTA when bit 7 of its rc_tune_mmq mask is set: 160 x 8 uint64 (globaltimer ns: start,
 * set-up done, predecessor done, first stage full, last commit, accumulator full, drain done,
 * tensor memory freed).  No counterpart in the reference. */
int rc_debug_read_trace(void *out, size_t bytes);
/* Measurement aid: copies out (synchronously) the per-role cycle counters that the dense exact GEMM
 * of rc_matmul accumulates per CTA when rc_tune_mmq's kind is 64 (Q4_K and Q8_0 only): 160 x 32
 * uint64, six counters for each of: token producer, MMA issuer, the two expander groups, the first
 * and the last epilogue warp.  No counterpart in the reference. */
int rc_debug_read_prof(void *out, size_t bytes);
/* Measurement aid: phase timestamps (globaltimer ns) of rc_ffn_decode launches.  The first call switches the
 * recording on; every call copies out and then clears the maxima.  Layout, uint64: [0, 16) the marks of CTA 0
 * of the latest launch (0 start, 1 x quantized, 2 first warp past its gate/up rows, 3 every CTA of the GPU
 * past them, 4 intermediate staged, 5 down rows done, 6 output complete), [16, 32) for each mark the latest
 * time any CTA passed it since the previous call, then, if `bytes` has room, [32, 32 + 8 * 160) marks 0..7
 * of every CTA (CTA index fastest).  No counterpart in the reference. */
int rc_debug_read_ffn_trace(void *out, size_t bytes);

/* ---- int8 MMQ GEMM --------------------------------------------------------------------- */

/* matmul_mmq_into's kernel launch (src/runtime/prefill.rs:512-567), bmm_mmq
 * (src/runtime/qwen35.rs:4116-4148); kernels mmq_gemm_<fmt>_repacked{,_narrow}_f32.
 * Y f32 [p_rows][out_dim] = Xq[p_rows][in_dim/32] . W^T, any p_rows >= 1. */
int rc_mmq_gemm(void *stream, int ggml_type, const void *w, const void *xq, float *y,
                uint32_t in_dim, uint32_t out_dim, uint32_t p_rows);

/* PrefillGemm::matmul_into_raw (src/runtime/prefill.rs:343-437).  x f32 [n_rows][in_dim].
 * n_rows <= RC_MATVEC_MAX_ROWS: quantize X to BlockQ8 in the caller's scratch, then the batched
 * matvec.  More rows: the same quantizer writes its int8 values as an integer-valued f16 operand
 * image (plus the d and xsum planes) into the scratch, then the tensor-core GEMM whose accumulator
 * tile of every 32-wide sub-block is the exact integer block dot (mmq_gemm_q4k_repacked.cpp:98-166),
 * scaled in f32 per sub-block; small matrices with few rows take 16-row passes of the batched matvec
 * instead, and Q5_1 always does.  On every route the per-block integer dots are exact and the f32
 * result is within 1e-3 relative L2 of the reference formulation (seen: 1e-6); which route runs
 * depends on the shape only, never on the scratch.  xq_scratch: 16-byte aligned and
 * rc_matmul_scratch_bytes large, else RC_ERR_MISALIGNED / RC_ERR_SCRATCH_TOO_SMALL (the reference
 * sizes its xq8 buffer as (in_dim / 32) * 40 bytes per row, src/runtime/prefill.rs:283: a binding
 * sizes it with rc_matmul_scratch_bytes instead). */
int rc_matmul(void *stream, int ggml_type, const void *w, const float *x, float *y,
              uint32_t in_dim, uint32_t out_dim, uint32_t n_rows, void *xq_scratch,
              size_t scratch_bytes);
/* An APPROXIMATION of rc_matmul for more than 16 rows, faster on wide batches: both operands
 * dequantized and rounded once to f16 (weights d * sc * q, activations d * q times a power of two per
 * token), whole-K f32 accumulation in tensor memory, no per-block integer dots.  About 3e-4 relative
 * L2 from rc_matmul's result (inside the reference's own 1e-3 GPU-vs-CPU bound, but not bit-exact at
 * the block level), and with few tiles it splits K and adds partial sums atomically, so two runs may
 * differ in the last bits and y is zeroed first.  Same arguments and scratch size as rc_matmul.
 * No counterpart in the reference. */
int rc_matmul_f16(void *stream, int ggml_type, const void *w, const float *x, float *y,
                  uint32_t in_dim, uint32_t out_dim, uint32_t n_rows, void *scratch,
                  size_t scratch_bytes);
/* Debug variant of rc_matmul's tensor-core route (any n_rows >= 1): besides y it writes the tile the
 * kernel drains for every (activation row, weight row, sub-block), before any f32 scaling, as
 * int32 idots[n_rows][out_dim][in_dim / 32]: the integer block dot, times the integer sub-scale
 * for the K-quants (Q4_K / Q5_K: sc * idot; Q6_K: sc_lo * I0 + sc_hi * I1).  Not Q5_1.  The
 * reference has no such dump; its kernels hold these integers in registers
 * (kernels/mmq_gemm_q4k_repacked.cpp:150-161). */
int rc_matmul_block_dots(void *stream, int ggml_type, const void *w, const float *x, float *y,
                         int32_t *idots, uint32_t in_dim, uint32_t out_dim, uint32_t n_rows,
                         void *scratch, size_t scratch_bytes);
/* bytes rc_matmul / rc_matvec_f32 need in xq_scratch */
size_t rc_matmul_scratch_bytes(uint32_t in_dim, uint32_t n_rows);

/* ---- MoE: expert sort, gather, scatter, grouped GEMM --------------------------------------- */

/* launch_moe_sort (src/runtime/qwen35.rs:2892-2938, src/runtime/gemma4.rs:1825-1870);
 * kernels moe_sort_{zero,histogram,scan,scatter} (kernels/moe_expert_sort.cpp:27-76).
 * ids int32 [n_entries] (entry = tok*n_used + slot); outputs count[n_expert],
 * cursor[n_expert] (scratch), expert_off[n_expert+1], tile_off[n_expert+1] (prefix of
 * ceil(count/bn)), perm[n_entries].  Ids outside [0,n_expert) are dropped.  Order
 * inside one expert is ascending entry index (the reference leaves it unspecified). */
int rc_moe_sort(void *stream, const int32_t *ids, uint32_t n_entries, uint32_t n_expert,
                uint32_t bn, int32_t *count, int32_t *cursor, int32_t *expert_off,
                int32_t *tile_off, int32_t *perm);
/* tile width the grouped GEMM assumes for tile_off (MOE_GEMM_BN, qwen35.rs:127) */
uint32_t rc_moe_tile_bn(void);

/* launch_moe_gather_xq (src/runtime/qwen35.rs:2999-3013); kernel moe_gather_xq
 * (kernels/moe_expert_sort.cpp:82-96): xq_dst[p] = xq_src[perm[p] / n_used]. */
int rc_moe_gather_xq(void *stream, const void *xq_src, const int32_t *perm, void *xq_dst,
                     uint32_t n_sub, uint32_t n_used, uint32_t n_entries);

/* launch_moe_scatter_rows (src/runtime/qwen35.rs:3016-3030); kernel moe_scatter_rows
 * (kernels/moe_expert_sort.cpp:100-110): dst[perm[p]] = src[p], `dim` floats a row. */
int rc_moe_scatter_rows(void *stream, const float *src, const int32_t *perm, float *dst,
                        uint32_t dim, uint32_t n_entries);

/* launch_moe_grouped_gemm (src/runtime/qwen35.rs:3036-3064,
 * src/runtime/gemma4.rs:1909-1936); kernels mmq_gemm_{q4k,q5k,q6k,q8_0}_grouped_f32
 * (kernels/mmq_gemm_q4k_grouped.cpp:38-165).  All six types are accepted.  xq and y
 * are in expert-sorted order; expert e uses slab + e*bytes_per_expert. */
int rc_mmq_gemm_grouped(void *stream, int ggml_type, const void *slab,
                        size_t bytes_per_expert, const int32_t *expert_off,
                        const int32_t *tile_off, uint32_t n_expert, const void *xq, float *y,
                        uint32_t in_dim, uint32_t out_dim, uint32_t n_entries);

/* ---- fused BlockQ8 producers ------------------------------------------------------------------- */

/* launch_rmsnorm_q8; kernel rmsnorm_q8_f32 (kernels/rmsnorm_q8.cpp:38-103): per vector
 * v = x * rsqrt(mean(x^2) + eps) * w, quantized to BlockQ8 (out [n_vec][n/32]).  n % 32 == 0. */
int rc_rmsnorm_q8(void *stream, const float *x, const float *w, void *out, uint32_t n, uint32_t n_vec, float eps);

/* launch_add_rmsnorm_q8; kernel add_rmsnorm_q8_f32 (kernels/qwen35_fused.cpp:66-118): hidden += add
 * (add may be NULL: hidden is then only read), y = rmsnorm(hidden) * w as f32 (y may be NULL) and as
 * BlockQ8.  One vector per row of n_vec; any n % 32 == 0 (the reference's kernel stops at 8192). */
int rc_add_rmsnorm_q8(void *stream, float *hidden, const float *add, const float *w, float *y, void *out,
                      uint32_t n, uint32_t n_vec, float eps);

/* launch_swiglu_q8; kernel swiglu_q8_f32 (kernels/qwen35_fused.cpp:123-138): out = silu(gate) * up as
 * f32 (out may be NULL) and as BlockQ8 (q8 [n/32]); n % 32 == 0 (several vectors: pass their total). */
int rc_swiglu_q8(void *stream, const float *gate, const float *up, float *out, void *q8, size_t n);

/* The grouped GEMM taking f32 activations: what the sequence quantize_q8 -> moe_gather_xq ->
 * rc_mmq_gemm_grouped (gate / up) and moe_geglu_q8 -> rc_mmq_gemm_grouped (down) computes, through the
 * f16-operand tensor-core kernel of rc_matmul (same quantizer, operands rounded once to f16, whole-K
 * accumulation: within 1e-3 relative L2 of the exact-integer route, about 3e-4).  Sorted entry j takes
 * its activation row from x[(index ? index[j] / div : j) * row_stride ...]: for gate / up pass the
 * sort's perm and div = n_used (token rows, row_stride = in_dim); for down pass the gate_up output in
 * sorted order (index NULL, row_stride = 2 * in_dim) and act = RC_ACT_GEGLU / RC_ACT_SWIGLU, which
 * applies act(gate) * up on the fly; act = -1 takes x as is.  y f32 [n_entries][out_dim] in sorted
 * order.  scratch: 16-byte aligned, rc_mmq_gemm_grouped_scratch_bytes large.  No reference counterpart
 * as one call (launch_moe_grouped_gemm takes BlockQ8: src/runtime/qwen35.rs:3036-3064). */
size_t rc_mmq_gemm_grouped_scratch_bytes(uint32_t in_dim, uint32_t n_entries);
int rc_mmq_gemm_grouped_f32(void *stream, int ggml_type, const void *slab, size_t bytes_per_expert,
                            const int32_t *expert_off, const int32_t *tile_off, uint32_t n_expert,
                            const float *x, const int32_t *index, uint32_t div, size_t row_stride, int act,
                            float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_entries, void *scratch,
                            size_t scratch_bytes);

/* kernel sigmoid_mul_q8_f32 (kernels/qwen35_fused.cpp:139-152): x[i] = x[i] * sigmoid(gate[i]) in place
 * and as BlockQ8; n % 32 == 0. */
int rc_sigmoid_mul_q8(void *stream, float *x, const float *gate, void *q8, size_t n);

/* kernel rmsnorm_gated_q8_f32 (kernels/qwen35_fused.cpp:204-224): per head h of head_dim values
 * y = rmsnorm(x_h) * w * silu(z_h) as f32 (y may be NULL) and as BlockQ8; w has head_dim entries shared
 * by the heads.  head_dim % 32 == 0, head_dim <= 1024. */
int rc_rmsnorm_gated_q8(void *stream, const float *x, const float *z, const float *w, float *y, void *q8,
                        uint32_t n_heads, uint32_t head_dim, float eps);

/* launch_moe_expert_matvec and launch_moe_down (src/runtime/qwen35.rs:3066-3139); kernels
 * moe_matvec_{q4k,q5k,q6k,q8_0}_repacked_f32 and moe_matvec_{q5k,q6k}_down_f32: the decode-side
 * routed-expert matvec.  For token t and routing slot j:
 *   y[t][j][:] = W[ids[t][j]] . xq[t * xq_tok_stride + j * xq_slot_stride]
 * with W[e] = slab + e * bytes_per_expert and the strides in BlockQ8 blocks, as the reference passes
 * them (gate and up share the token's row: tok stride in_dim/32, slot stride 0; down has one row per
 * slot: tok stride n_used * in_dim/32, slot stride in_dim/32).  ids int32 [n_tok][n_used] on the device; an id outside [0, n_expert) yields zeros.
 * All six types; one geometry for both reference wrappers (rows are split across warps by shape). */
int rc_moe_expert_matvec(void *stream, int ggml_type, const void *slab, size_t bytes_per_expert,
                         const int32_t *ids, uint32_t n_expert, const void *xq, float *y, uint32_t in_dim,
                         uint32_t out_dim, uint32_t n_used, uint32_t n_tok, uint32_t xq_tok_stride,
                         uint32_t xq_slot_stride);

/* launch_moe_gate_up_swiglu (src/runtime/qwen35.rs:3141-3167); kernel moe_gate_up_swiglu_q4k_repacked_f32:
 * y[t][j][i] = silu(Wgate[ids[t][j]][i] . x) * (Wup[ids[t][j]][i] . x), one launch in place of two expert
 * matvecs and the activation.  gate_slab and up_slab have the same type, shape and bytes_per_expert;
 * x is addressed as in rc_moe_expert_matvec.  All six types (the reference: Q4_K); in_dim % 1024 == 0. */
int rc_moe_gate_up_swiglu(void *stream, int ggml_type, const void *gate_slab, const void *up_slab,
                          size_t bytes_per_expert, const int32_t *ids, uint32_t n_expert, const void *xq, float *y,
                          uint32_t in_dim, uint32_t out_dim, uint32_t n_used, uint32_t n_tok, uint32_t xq_tok_stride,
                          uint32_t xq_slot_stride);

/* ---- MoE glue around the grouped GEMMs ------------------------------------------------------- */

/* launch_moe_topk (src/runtime/gemma4.rs:1649-1670); kernel moe_topk_f32 (kernels/moe_topk.cpp:17-107):
 * softmax over n_expert logits per token (NaN logits count as -inf), the n_used largest
 * probabilities (ties: lowest expert index) renormalised over their sum with the floor
 * 6.103515625e-5.  logits f32 [n_tok][n_expert]; ids int32, weights f32 [n_tok][n_used].
 * n_expert <= 1024, n_used <= 32. */
int rc_moe_topk(void *stream, const float *logits, uint32_t n_tok, uint32_t n_expert, uint32_t n_used,
                int32_t *ids, float *weights);

/* launch_moe_geglu_q8 (src/runtime/gemma4.rs:1784-1800); kernel moe_geglu_q8_f32
 * (kernels/moe_geglu_q8.cpp:34-66): act(gate) * up of the fused gate_up GEMM output, quantized
 * straight to BlockQ8 for the down GEMM.  gu f32 [n_slot][2*ff] (gate half, then up half),
 * out BlockQ8 [n_slot][ff/32]; ff % 32 == 0.  act: RC_ACT_GEGLU (tanh GELU) or RC_ACT_SWIGLU
 * (x / (1 + exp(-x)), kernels/swiglu.cpp:11-21). */
enum rc_gated_act { RC_ACT_GEGLU = 0, RC_ACT_SWIGLU = 1 };
int rc_moe_act_q8(void *stream, const float *gu, void *out, uint32_t ff, uint32_t n_slot, int act);

/* launch_moe_combine (src/runtime/gemma4.rs:1804-1823); kernel moe_combine_f32
 * (kernels/moe_combine.cpp:16-37): out[t][i] = sum_j weights[t][j] * expert_scale[ids[t][j]] *
 * experts[t][j][i], accumulated in slot order.  expert_scale may be NULL (all ones).  A slot whose id is
 * negative (a dropped entry) adds nothing. */
int rc_moe_combine(void *stream, const float *experts, const int32_t *ids, const float *weights,
                   const float *expert_scale, float *out, uint32_t hidden, uint32_t n_used, uint32_t n_tok);

/* ---- row-shard gather over NVLink peer memory ---------------------------------------------- */

/* The reference has no collectives (its multi-GPU mode is layer pipelining over
 * hipMemcpyPeerAsync, src/runtime/pipeline.rs:1-19).  Row-sharded matvec outputs of a decode
 * step are tens of kilobytes, far below the size at which a library collective's launch latency
 * is amortised, so the gather is one small kernel: every rank stores its shard straight into
 * every peer's gathered buffer (peer-mapped memory), publishes a step counter in each peer's flag
 * array and waits, with a time limit, until all peers' counters have arrived.  No host
 * involvement, so a whole sharded layer can be replayed from one CUDA graph.
 *
 * rc_ipc_*: export / import a cudaMalloc'ed buffer between the processes of one box (one process
 * per GPU); `handle` is 64 bytes.  peer_dst[r] is rank r's gathered buffer (world * bytes, own
 * entry included), peer_flags[r] rank r's array of `world` 64-bit counters (zeroed once),
 * epoch a 64-bit counter in this rank's memory (zeroed once); both arrays are HOST arrays of
 * `world` <= RC_MAX_PEERS device pointers.  bytes % 16 == 0.  A wait that runs out sets the device status word
 * (rc_device_status, bit 16) and lets the kernel end. */
#define RC_MAX_PEERS 8
#define RC_IPC_HANDLE_BYTES 64
int rc_ipc_get_handle(const void *dev_ptr, void *handle);
int rc_ipc_open_handle(const void *handle, void **dev_ptr);
int rc_ipc_close_handle(void *dev_ptr);
int rc_allgather_push(void *stream, const void *src, size_t bytes, void *const *peer_dst,
                      void *const *peer_flags, void *epoch, uint32_t rank, uint32_t world);
/* Two calls that gather into the SAME buffers need one more handshake between them: a rank's wait only
 * proves that its peers have pushed this call's shards, not that their consumers of the previous call have
 * finished reading.  Alternating between two gathered buffers closes that window (a rank pushes call e + 2
 * after it saw its peers' call e + 1, which they start only after their consumer of call e: the handshake
 * kernel waits for its stream predecessor); reinstinct_b200/runtime.py's PeerAllGather does so.
 *
 * rc_peer_barrier: the handshake alone (epoch publication + bounded wait), for producers that store into
 * their peers' memory themselves (rc_matmul_gather).  A peer's stores are complete on this device when the
 * peer's barrier kernel, launched behind them on the same stream, has published its epoch. */
int rc_peer_barrier(void *stream, void *const *peer_flags, void *epoch, uint32_t rank, uint32_t world);
/* The work of `world` ranks done by ONE cooperative launch on one device (one CTA per rank, co-resident):
 * the way to exercise the gather on a box with fewer GPUs than ranks, since separate launches that wait on
 * one another are not guaranteed to run at the same time.  srcs, dsts, flags, epochs: host arrays of `world`
 * device pointers (rank r's shard, gathered buffer, flag array, epoch counter).  The reference tests its
 * two-stage pipeline on one device the same way (tests/qwen35_pipeline.rs:8-10). */
int rc_allgather_push_logical(void *stream, const void *const *srcs, size_t bytes, void *const *dsts,
                              void *const *flags, void *const *epochs, uint32_t world);
/* The decode FFN of one GPU as ONE cooperative launch: step_swiglu_ffn (src/runtime/qwen35.rs:2694-2707:
 * quantize x, gate and up matvecs, silu(gate) * up, quantize, down matvec), row-sharded over `world` GPUs.
 * This rank holds rows [ffn_begin, ffn_begin + ffn_local) of gate_w and up_w ([ffn_total, in_dim], both of
 * gate_type) and rows [out_begin, out_begin + out_local) of down_w ([out_total, ffn_total], down_type).  It
 * stores its ffn_local values of the intermediate silu(gate) * up, as f32, into every rank's intermediate
 * vector (every rank then quantizes the whole vector itself, block by block as rc_quantize_q8 does) and its
 * out_local output rows into every rank's arrival vector; the launch ends when all out_total rows of this call
 * have arrived at this rank and have been copied to y (f32 [out_total]; may be pinned host memory, as may x,
 * 16-byte aligned).  h_peers, y_peers: host arrays of `world` device pointers (own buffers included, peers'
 * mapped with rc_ipc_open_handle): h_peers[r] = rank r's f32 [3][ffn_total] (16-byte aligned), y_peers[r] =
 * rank r's f32 [3][out_total]; work: rc_ffn_decode_work_bytes(ffn_local) bytes of this rank's memory.  Before
 * the first call, once, every byte of the h and y buffers is set to 0xFF ("not arrived": arrival is read off
 * the values themselves, no flags or fences; the three copies take turns call by call and a launch refills
 * the one that the call after the next uses) and work to zero; they then belong to this shape, and every rank makes the same
 * sequence of calls.  Same per-block arithmetic as rc_quantize_q8 / rc_matvec / rc_swiglu_q8; a row's partial
 * sums are added in a fixed order that depends on the shapes only, so results repeat bit for bit, and differ
 * from the launch chain's in the last bits where the two split a row differently.  in_dim and ffn_total
 * multiples of 1024; format pairs (gate, down): (Q4_K, Q6_K), (Q4_K, Q4_K), (Q5_K, Q6_K), (Q6_K, Q6_K),
 * (Q8_0, Q8_0), (Q4_0, Q4_0), else RC_ERR_BAD_TYPE.  A cooperative launch of one CTA per SM; may be captured
 * in a CUDA graph.  A wait that runs out (a peer that never launched) sets bits 20-23 of rc_device_status (2:
 * the intermediate, 3: the output rows) and the launch ends; the buffers and counters of the shape are then
 * out of step with the peers' and must be set up again (fill, zero) on every rank before the next call. */
size_t rc_ffn_decode_work_bytes(uint32_t ffn_local);
int rc_ffn_decode(void *stream, int gate_type, int down_type, const void *gate_w, const void *up_w,
                  const void *down_w, const float *x, float *y, uint32_t in_dim, uint32_t ffn_local,
                  uint32_t ffn_total, uint32_t ffn_begin, uint32_t out_local, uint32_t out_total,
                  uint32_t out_begin, uint32_t world, uint32_t rank, void *const *h_peers,
                  void *const *y_peers, void *work);
/* The same step (step_swiglu_ffn, src/runtime/qwen35.rs:2694-2707) as one cooperative launch per GPU with the
 * down projection sharded along its CONTRACTION: this rank holds rows [b, b + ffn_local) of gate_w and up_w
 * ([ffn_total, in_dim]) and the matching columns of down_w as a tensor of its own, [out_total][ffn_local]
 * (ffn_local a whole number of the down format's blocks, so a row's blocks [b / 256, ...) are taken as they
 * are).  A rank's slice of the intermediate never leaves it; every rank stores its out_total partial sums into
 * slot `rank` of every rank's partial buffer and adds the `world` slots in rank order into y (f32 [out_total],
 * may be pinned host memory, as may x, 16-byte aligned).  part_peers: host array of `world` device pointers,
 * part_peers[r] = rank r's f32 [3][world][out_total], every byte 0xFF before the first call; work:
 * rc_ffn_decode_tp_work_bytes(ffn_local) bytes of this rank's memory, zeroed once.  One exchange per step
 * instead of rc_ffn_decode's two, and ffn_local / 32 instead of ffn_total / 32 blocks to quantize per CTA; the
 * sum over ranks replaces part of a row sum, so results differ from the one-GPU step in the last bits (and
 * repeat bit for bit).  in_dim a multiple of 1024; format pairs as rc_ffn_decode.  Every rank makes the same
 * sequence of calls; a wait that runs out sets bits 20-23 of rc_device_status (1: this GPU's own CTAs, 3: the
 * peers' partial sums) and the launch ends; buffers and work must then be set up again on every rank. */
size_t rc_ffn_decode_tp_work_bytes(uint32_t ffn_local);
int rc_ffn_decode_tp(void *stream, int gate_type, int down_type, const void *gate_w, const void *up_w,
                     const void *down_w, const float *x, float *y, uint32_t in_dim, uint32_t ffn_local,
                     uint32_t out_total, uint32_t world, uint32_t rank, void *const *part_peers, void *work);
/* Expert parallelism without the host (no counterpart in the reference, which pipelines layers): the routed rows
 * of this rank's tokens travel to the rank that owns their expert and the results travel back by plain stores
 * into peer memory; between the two exchanges the owner runs the reference's own sequence on what it received
 * (rc_moe_sort, rc_moe_gather_xq with n_used = 1, rc_mmq_gemm_grouped, rc_moe_scatter_rows; launch wrappers at
 * src/runtime/qwen35.rs:2892-3064).  Shapes are static: every (source, owner) pair has `cap` slots (cap >= the
 * entries one rank can route, n_tok * n_used), unused slots carry expert id -1, which those kernels skip; so a
 * step is a fixed launch sequence and can be captured in a CUDA graph.  Expert e belongs to rank e /
 * experts_per_rank.  Buffers per rank (mapped into every rank with rc_ipc_open_handle; *_peers are host arrays
 * of `world` device pointers, own buffers included):
 *   rows  BlockQ8 [2][world * cap][in_dim / 32]   ids  int32 [2][world * cap], every entry -1 before the first step
 *   ret   f32 [world * cap][dim]
 * One step on every rank, `buf` alternating 0, 1 from step to step:
 *   rc_ep_plan      back[e] = owner * cap + (count of earlier entries with that owner), -1 for a dropped id
 *   rc_ep_dispatch  stores each entry's row and local expert index into slot (this rank, slot) of its owner's
 *                   buffers `buf`, and marks this rank's OTHER ids buffer unused for the next step
 *   rc_peer_barrier
 *   the owner's sort / gather / grouped GEMM / scatter over its world * cap slots of buffer `buf`
 *   rc_ep_return    stores the result row of every used slot into slot (this rank, slot) of its source's ret
 *   rc_peer_barrier
 *   rc_ep_collect   out[e] = ret[back[e]] (zeros for a dropped entry)
 * The placement depends on the ids only; an entry's result does not depend on where it was placed. */
int rc_ep_plan(void *stream, const int32_t *ids, uint32_t n_entries, uint32_t experts_per_rank, uint32_t cap,
               uint32_t world, int32_t *back);
int rc_ep_dispatch(void *stream, const int32_t *ids, const int32_t *back, const void *xq, uint32_t n_entries,
                   uint32_t n_used, uint32_t in_dim, uint32_t experts_per_rank, uint32_t cap, uint32_t rank,
                   uint32_t world, uint32_t buf, void *const *rows_peers, void *const *ids_peers);
int rc_ep_return(void *stream, const int32_t *ids_in, const float *y_in, uint32_t dim, uint32_t cap,
                 uint32_t rank, uint32_t world, void *const *ret_peers);
int rc_ep_collect(void *stream, const int32_t *back, const float *ret, float *out, uint32_t dim,
                  uint32_t n_entries);
/* Row-sharded PrefillGemm::matmul_into_raw that gathers its own output: this rank holds weight rows
 * [row_begin, row_begin + out_dim) of an [out_total, in_dim] matrix; the kernel's finished tiles are stored
 * into columns row_begin.. of EVERY rank's [n_rows][out_total] f32 output (y_peers: host array of `world`
 * device pointers, this rank's own buffer included, the others peer-mapped with rc_ipc_open_handle), while
 * other tiles still compute.  Always the tensor-core kernel of rc_matmul (any n_rows >= 1, not Q5_1), so
 * every rank's rows are bit-identical to the unsharded call.  Follow it with rc_peer_barrier; alternate two
 * output buffers between consecutive calls (see above).  No counterpart in the reference, whose only
 * multi-device transfer is a peer copy of the hidden state (src/runtime/pipeline.rs:333-349). */
int rc_matmul_gather(void *stream, int ggml_type, const void *w, const float *x, float *const *y_peers,
                     uint32_t world, uint32_t out_total, uint32_t row_begin, uint32_t in_dim,
                     uint32_t out_dim, uint32_t n_rows, void *scratch, size_t scratch_bytes);

/* ---- device API mirror (src/hip/sys.rs:57-101, src/hip/mod.rs) --------------------------- */

enum rc_memcpy_kind { /* src/hip/sys.rs:45-53 */
    RC_MEMCPY_H2H = 0, RC_MEMCPY_H2D = 1, RC_MEMCPY_D2H = 2, RC_MEMCPY_D2D = 3,
    RC_MEMCPY_DEFAULT = 4
};
enum rc_capture_mode { RC_CAPTURE_GLOBAL = 0, RC_CAPTURE_THREAD_LOCAL = 1, RC_CAPTURE_RELAXED = 2 };

int rc_get_device_count(int *count);
int rc_set_device(int device);
int rc_get_device(int *device);
int rc_device_get_name(char *name, int len, int device);
int rc_device_total_mem(size_t *bytes, int device);
int rc_mem_get_info(size_t *free_bytes, size_t *total_bytes);
int rc_device_can_access_peer(int *can, int device, int peer);
/* "already enabled" is reported as success (src/hip/mod.rs:125-131) */
int rc_device_enable_peer_access(int peer);
int rc_device_synchronize(void);

int rc_malloc(void **ptr, size_t bytes);
int rc_free(void *ptr);
int rc_memcpy(void *dst, const void *src, size_t bytes, int kind);
int rc_memcpy_async(void *dst, const void *src, size_t bytes, int kind, void *stream);
/* A small copy (up to 16 MiB, 16-byte aligned, a multiple of 16 bytes) done by a kernel instead of the copy
 * engine: either side may be pinned host memory.  For steps replayed from a CUDA graph whose few-KB input or
 * output sits in host memory: a memcpy node costs 8-10 us of such a step here, this launch 3.  No counterpart
 * in the reference (its uploads are hipMemcpyAsync, src/hip/sys.rs:64). */
int rc_copy_small(void *stream, void *dst, const void *src, size_t bytes);
int rc_memcpy_peer_async(void *dst, int dst_device, const void *src, int src_device,
                         size_t bytes, void *stream);
int rc_memset_async(void *dst, int value, size_t bytes, void *stream);

int rc_stream_create(void **stream);
int rc_stream_destroy(void *stream);
int rc_stream_synchronize(void *stream);
int rc_stream_wait_event(void *stream, void *event);

int rc_event_create(void **event);
int rc_event_record(void *event, void *stream);
int rc_event_synchronize(void *event);
int rc_event_elapsed_time(float *ms, void *start, void *stop);
int rc_event_destroy(void *event);

int rc_stream_begin_capture(void *stream, int mode);
int rc_stream_end_capture(void *stream, void **graph);
int rc_graph_instantiate(void **graph_exec, void *graph);
int rc_graph_launch(void *graph_exec, void *stream);
int rc_graph_destroy(void *graph);
int rc_graph_exec_destroy(void *graph_exec);

#ifdef __cplusplus
}
#endif
#endif /* REINSTINCT_CUDA_H */
