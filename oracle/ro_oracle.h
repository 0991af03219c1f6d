/*
 * TEST INFRASTRUCTURE — CPU oracle for the quantized-weight hot path.
 *
 * A plain-C restatement of the arithmetic the reference engine
 * (sixvolts/reinstinct) defines for this path.  Only tests, the smoke check and
 * the benchmark's CPU-baseline leg may link or call it; the shipped library never
 * does.  Each function names the reference file:line it follows.
 *
 * Pinning: the f16 conversions, the six on-disk block decoders and the six
 * repacked-v2 builders are checked against every known-answer unit test the
 * reference keeps in src/quant/{half,q4_0,q4_k,q5_k,q6_k,q8_0,iq4_xs}.rs (ported
 * as vectors under tests/golden/).  The reference has no CPU implementation and
 * no test of the int8 activation quantizer, of the per-block integer dots or of
 * the expert sort; for those this oracle follows the kernel sources and is
 * cross-checked by exact identities (integer dots times scales equals the f64 dot
 * of dequantized weights with dequantized activations) — "parity unpinned" by a
 * reference vector for exactly those three pieces.
 */
#ifndef RO_ORACLE_H
#define RO_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGUF type discriminants (src/gguf/types.rs:16-35). */
enum {
    RO_Q4_0 = 2,
    RO_Q8_0 = 8,
    RO_Q4_K = 12,
    RO_Q5_K = 13,
    RO_Q6_K = 14,
    RO_Q5_1 = 7,   /* runs on the Q5_K kernel bodies with dsc = d, deff = -m (src/quant/q5_1.rs:11-20) */
    RO_IQ3_S = 21, /* kernel type only: IQ4_XS planes read through the codebook 2n - 15; no on-disk decode here */
    RO_IQ4_XS = 23,
    /* accepted as sources only: relabelled onto one of the six above */
    RO_Q3_K = 11,
    RO_IQ4_NL = 20,
    RO_BF16 = 30
};

/* Activation block, packed 40 bytes: f32 d, f32 xsum, i8 qs[32]
 * (kernels/quantize_q8.cpp:16-21). */
#define RO_BLOCKQ8_BYTES 40

/* src/quant/half.rs:9-84 */
float    ro_f16_to_f32(uint16_t bits);
uint16_t ro_f32_to_f16(float v);
float    ro_bf16_to_f32(uint16_t bits);

/* Per-format constants; 0 for an unknown type. */
size_t ro_block_bytes(int type);   /* bytes of one on-disk block    */
size_t ro_block_weights(int type); /* weights in one on-disk block  */

/* Padded sub-block count per repacked row (src/quant/q4_k.rs:92-95 and the same
 * rule in q4_0.rs:60-63, q8_0.rs:68-71, iq4_xs.rs:79-82). */
size_t ro_nsp(size_t in_dim);
/* Bytes of a repacked tensor; 0 when the shape is not allowed for the type. */
size_t ro_repacked_len(int type, size_t in_dim, size_t out_dim);

/* On-disk blocks -> f32, n_weights a multiple of the block size. 0 on success. */
int ro_dequantize(int type, const uint8_t *blocks, float *out, size_t n_weights);
/* On-disk rows [out_dim][in_dim/blk] -> repacked-v2 planes. 0 on success. */
int ro_repack(int type, const uint8_t *blocks, size_t in_dim, size_t out_dim, uint8_t *out);

/* kernels/quantize_q8.cpp:23-54 with the reciprocal pinned to an IEEE divide. */
void ro_quantize_q8(const float *x, uint8_t *out, size_t in_dim, size_t n_vec);
/* BlockQ8 rows back to f32 (d * qs), for the exact-identity cross-check. */
void ro_dequantize_q8(const uint8_t *xq, float *out, size_t in_dim, size_t n_vec);

/*
 * int8-path matvec / batched matvec / GEMM (one definition: per activation row,
 * per weight row, per 32-wide sub-block).  w is repacked-v2, xq is
 * BlockQ8[n_rows][in_dim/32].  Any of the three outputs may be NULL:
 *   y32   [n_rows][out_dim]  f32 terms summed in f32 in sub-block order
 *   y64   [n_rows][out_dim]  the same f32 terms summed in f64
 *   idots [n_rows][out_dim][in_dim/32][2]  the per-block integers; Q6_K fills
 *         both slots (I0, I1), the other formats slot 0 with slot 1 = 0.
 * rows [row_begin,row_end) of the weight only (for threaded callers).
 */
int ro_matvec_q8(int type, const uint8_t *w, const uint8_t *xq, size_t in_dim,
                 size_t out_dim, size_t n_rows, size_t row_begin, size_t row_end,
                 float *y32, double *y64, int32_t *idots);

/* src/cpu/ops.rs:108-140: y[j] = sum_i x[i]*w[j*in+i], sequential f32. */
void ro_matvec_f32(const float *x, const float *w, size_t in_dim, size_t out_dim,
                   float *y, int n_threads);

/* Timed CPU baseline: dequantize rows then ro_matvec_f32 semantics for n_rows
 * activation rows, row-parallel over n_threads.  w_f32 scratch is
 * [out_dim][in_dim] and is filled by the call when dequant != 0. */
int ro_cpu_path(int type, const uint8_t *blocks, const float *x, size_t in_dim,
                size_t out_dim, size_t n_rows, float *w_f32, float *y, int n_threads,
                int dequant);

/* kernels/moe_expert_sort.cpp:27-76 as a stable counting sort.  ids
 * [n_entries]; out-of-range ids are dropped as the kernels drop them. */
void ro_moe_sort(const int32_t *ids, size_t n_entries, size_t n_expert, size_t bn,
                 int32_t *count, int32_t *expert_off, int32_t *tile_off, int32_t *perm);

/* kernels/moe_topk.cpp:43-107 / src/cpu/gemma4.rs:365-372: softmax over
 * n_expert logits, the n_used largest (lowest index first on ties),
 * renormalised with the floor 6.103515625e-5 on the sum. */
void ro_router_topk(const float *logits, size_t n_tok, size_t n_expert, size_t n_used,
                    int32_t *ids, float *weights);

/* Fused BlockQ8 producers: rmsnorm (+ residual add) and SwiGLU followed by the quantizer
 * (kernels/rmsnorm_q8.cpp:38-103, kernels/qwen35_fused.cpp:66-138). */
void ro_rmsnorm_q8(const float *x, const float *add, const float *w, float *hidden_out, float *y_out,
                   uint8_t *out, size_t n, size_t n_vec, float eps);
void ro_swiglu_q8(const float *gate, const float *up, float *out_f32, uint8_t *q8, size_t n);
/* kernels/qwen35_fused.cpp:139-152 and :204-224 */
void ro_sigmoid_mul_q8(float *x, const float *gate, uint8_t *q8, size_t n);
void ro_rmsnorm_gated_q8(const float *x, const float *z, const float *w, float *y, uint8_t *q8,
                         size_t n_heads, size_t head_dim, float eps);

/* Relabelled source formats (src/runtime/qwen35.rs:274-307): decoders of the source blocks
 * (src/quant/q3_k.rs:123-162, iq4_nl.rs:32-46), the exact Q3_K -> Q6_K block transcode
 * (q3_k.rs:92-121), the Q8_0 quantizer BF16 tensors go through (q8_0.rs:45-61), the kernel type
 * of a source type, and the source rows -> repacked planes of that kernel type. */
void ro_dequantize_q3_k(const uint8_t *blocks, float *out, size_t n_weights);
void ro_q3k_to_q6k(const uint8_t *blocks, uint8_t *out, size_t n_weights);
void ro_dequantize_iq4_nl(const uint8_t *blocks, float *out, size_t n_weights);
void ro_quantize_q8_0(const float *vals, uint8_t *out, size_t n);
int ro_kernel_type(int src_type);
int ro_repack_any(int src_type, const uint8_t *src, size_t in_dim, size_t out_dim, uint8_t *out);

/* kernels/moe_geglu_q8.cpp:34-66: BlockQ8(act(gate) * up) of gu [n_slot][2*ff]; act 0 = tanh GELU,
 * 1 = SiLU (kernels/swiglu.cpp:11-21).  act_out (may be NULL) gets the f32 values. */
void ro_moe_act_q8(const float *gu, uint8_t *out, size_t ff, size_t n_slot, int act, float *act_out);

/* kernels/moe_combine.cpp:16-37: out[t][i] = sum_j (weights[t][j] * expert_scale[ids[t][j]]) *
 * experts[t][j][i]; expert_scale may be NULL. */
void ro_moe_combine(const float *experts, const int32_t *ids, const float *weights, const float *expert_scale,
                    float *out, size_t hidden, size_t n_used, size_t n_tok);

/* Grouped GEMM over expert-sorted rows (kernels/mmq_gemm_q4k_grouped.cpp:38-165):
 * rows expert_off[e]..expert_off[e+1] of xq use slab + e*bytes_per_expert. */
int ro_grouped_q8(int type, const uint8_t *slab, size_t bytes_per_expert,
                  const int32_t *expert_off, size_t n_expert, const uint8_t *xq,
                  size_t in_dim, size_t out_dim, float *y32, double *y64);

#ifdef __cplusplus
}
#endif
#endif
