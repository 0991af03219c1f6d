// Internal launch functions behind the C ABI (one per kernel family).  All return RC_OK,
// a negative rc_error or a positive cudaError_t; arguments are validated by the callers in
// rc_api.cu.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace rc {

int launch_quantize_q8(cudaStream_t s, const float *x, void *xq, uint32_t in_dim, uint32_t n_vec);

// planar form for the tensor-core GEMM (see rc_quantize.cu)
size_t quantize_planar_bytes(uint32_t in_dim, uint32_t n_vec);
int launch_quantize_q8_planar(cudaStream_t s, const float *x, void *out, uint32_t in_dim, uint32_t n_vec);

int launch_repack(cudaStream_t s, int type, const void *blocks, size_t in_dim, size_t out_dim,
                  void *out);

// Decode and small-batch matvec (1 <= n_rows <= 16).  idots != nullptr selects the debug
// variant that also writes the per-block integers.
int launch_matvec(cudaStream_t s, int type, const void *w, const void *xq, float *y,
                  uint32_t in_dim, uint32_t out_dim, uint32_t n_rows, int32_t *idots);
int matvec_set_attributes();
bool matvec_pdl_enabled();
int launch_matvec_grouped(cudaStream_t s, int type, const void *slab, size_t bytes_per_expert,
                          const int32_t *expert_off, const int32_t *tile_off, uint32_t n_expert,
                          const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
                          uint32_t n_entries);
int moe_set_attributes();
// the decode FFN of one GPU in one cooperative launch (rc_matvec.cu)
size_t ffn_decode_work_bytes(uint32_t ffn_local);
int ffn_device_error(unsigned int *out, bool clear);
int ffn_read_trace(void *out, size_t bytes);
int launch_ffn_decode_tp(cudaStream_t s, int gate_type, int down_type, const void *gate, const void *up, const void *down, const float *x,
                         float *y, uint32_t in_dim, uint32_t ffn_local, uint32_t out_total, uint32_t world, uint32_t rank,
                         void *const *part_peers, void *work);
size_t ffn_decode_tp_work_bytes(uint32_t ffn_local);
int launch_ep_plan(cudaStream_t s, const int32_t *ids, uint32_t n_entries, uint32_t experts_per_rank, uint32_t cap, uint32_t world,
                   int32_t *back);
int launch_ep_dispatch(cudaStream_t s, const int32_t *ids, const int32_t *back, const void *xq, uint32_t n_entries, uint32_t n_used,
                       uint32_t n_sub, uint32_t experts_per_rank, uint32_t cap, uint32_t rank, uint32_t world, uint32_t buf,
                       void *const *rows_peers, void *const *ids_peers);
int launch_ep_return(cudaStream_t s, const int32_t *ids_in, const float *y_in, uint32_t dim, uint32_t cap, uint32_t rank, uint32_t world,
                     void *const *ret_peers);
int launch_ep_collect(cudaStream_t s, const int32_t *back, const float *ret, float *out, uint32_t dim, uint32_t n_entries);
int launch_ffn_decode(cudaStream_t s, int gate_type, int down_type, const void *gate, const void *up, const void *down, const float *x,
                      uint32_t in_dim, uint32_t ffn_local, uint32_t ffn_total, uint32_t ffn_begin, uint32_t out_local,
                      uint32_t out_total, uint32_t out_begin, uint32_t world, uint32_t rank, void *const *h_peers,
                      void *const *y_peers, float *y, void *work);

int launch_mmq_gemm(cudaStream_t s, int type, const void *w, const void *xq, float *y,
                    uint32_t in_dim, uint32_t out_dim, uint32_t p_rows);
// quantize + GEMM from f32 activations; uses the planar form when the scratch allows it
int launch_mmq_gemm_f32(cudaStream_t s, int type, const void *w, const float *x, float *y, uint32_t in_dim,
                        uint32_t out_dim, uint32_t p_rows, void *scratch, size_t scratch_bytes);
int launch_mmq_grouped(cudaStream_t s, int type, const void *slab, size_t bytes_per_expert,
                       const int32_t *expert_off, const int32_t *tile_off, uint32_t n_expert,
                       const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
                       uint32_t n_entries);
int mmq_set_attributes();
// rc_mmq_deq.cu: the f16-operand dense GEMM (activations as f32 in, scratch holds their f16 image)
int mmq_deq_set_attributes();
void mmq_deq_set_bn(int bn);
int mmq_deq_device_error(unsigned int *out, bool clear);
size_t mmq_deq_scratch_bytes(uint32_t in_dim, uint32_t n_tok);
size_t mmq_deq_grouped_scratch_bytes(uint32_t in_dim, uint32_t n_entries);
int launch_mmq_deq_grouped_f32(cudaStream_t s, int type, const void *slab, size_t bytes_per_expert, const int32_t *expert_off,
                               const int32_t *tile_off, uint32_t n_expert, const float *x, const int32_t *index, uint32_t div,
                               size_t row_stride, int act, float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_entries,
                               void *scratch);
int launch_mmq_deq_f32(cudaStream_t s, int type, const void *w, const float *x, float *y, uint32_t in_dim, uint32_t out_dim,
                       uint32_t n_tok, void *scratch);
// rc_mmq_x.cu: the dense GEMM with exact integer block dots (integer-valued f16 operands, per-sub-block drain)
int mmq_x_set_attributes();
bool mmq_x_supports(int type);
void mmq_x_set_prof(int on);
void mmq_x_set_debug(int mask);
int mmq_x_read_prof(void *out, size_t bytes);
int mmq_x_device_error(unsigned int *out, bool clear);
size_t mmq_x_scratch_bytes(uint32_t in_dim, uint32_t n_tok);
// y_peers != nullptr: the result is rows [col_off, col_off + out_dim) of a [n_tok][ld_out] matrix and is stored
// into each of the n_peers copies of it (this rank's own and its peers' mapped ones); y is then unused
int launch_mmq_x_f32(cudaStream_t s, int type, const void *w, const float *x, float *y, uint32_t in_dim, uint32_t out_dim,
                     uint32_t n_tok, void *scratch, int32_t *dump, float *const *y_peers = nullptr, uint32_t n_peers = 0,
                     uint32_t ld_out = 0, uint32_t col_off = 0);
uint32_t mmq_grouped_bn();
uint32_t matvec_grouped_bn();
void mmq_force_dp4a(int on);
void mmq_set_kind(int kind);
int mmq_device_error(unsigned int *out, bool clear);

int launch_moe_sort(cudaStream_t s, const int32_t *ids, uint32_t n_entries, uint32_t n_expert,
                    uint32_t bn, int32_t *count, int32_t *cursor, int32_t *expert_off,
                    int32_t *tile_off, int32_t *perm);
int launch_moe_gather_xq(cudaStream_t s, const void *xq_src, const int32_t *perm, void *xq_dst,
                         uint32_t n_sub, uint32_t n_used, uint32_t n_entries);
int launch_moe_scatter_rows(cudaStream_t s, const float *src, const int32_t *perm, float *dst,
                            uint32_t dim, uint32_t n_entries);

int launch_allgather_push(cudaStream_t s, const void *src, size_t bytes, void *const *peer_dst,
                          void *const *peer_flags, void *epoch, uint32_t rank, uint32_t world);
int gather_device_error(unsigned int *out, bool clear);
int launch_allgather_push_logical(cudaStream_t s, const void *const *srcs, size_t bytes, void *const *dsts, void *const *flags,
                                  void *const *epochs, uint32_t world);

int launch_rmsnorm_q8(cudaStream_t s, const float *x, const float *add, const float *w, float *hidden_io, float *y, void *out,
                      uint32_t n, uint32_t n_vec, float eps);
int launch_sigmoid_mul_q8(cudaStream_t s, float *x, const float *gate, void *q8, size_t n);
int launch_rmsnorm_gated_q8(cudaStream_t s, const float *x, const float *z, const float *w, float *y, void *q8, uint32_t n_heads,
                            uint32_t head_dim, float eps);
int launch_swiglu_q8(cudaStream_t s, const float *gate, const float *up, float *out, void *q8, size_t n);
int launch_moe_expert_matvec(cudaStream_t s, int type, const void *slab, size_t bpe, const int32_t *ids, uint32_t n_expert,
                             const void *xq, float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_used, uint32_t n_tok,
                             uint32_t tok_stride, uint32_t slot_stride);
int launch_moe_gate_up_swiglu(cudaStream_t s, int type, const void *gate_slab, const void *up_slab, size_t bpe, const int32_t *ids,
                              uint32_t n_expert, const void *xq, float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_used,
                              uint32_t n_tok, uint32_t tok_stride, uint32_t slot_stride);
int launch_moe_topk(cudaStream_t s, const float *logits, uint32_t n_tok, uint32_t n_expert, uint32_t n_used,
                    int32_t *ids, float *weights);
int launch_moe_act_q8(cudaStream_t s, const float *gu, void *out, uint32_t ff, uint32_t n_slot, int act);
int launch_moe_combine(cudaStream_t s, const float *experts, const int32_t *ids, const float *weights,
                       const float *expert_scale, float *out, uint32_t hidden, uint32_t n_used, uint32_t n_tok);

// Per-device one-time setup (kernel attributes); returns RC_OK or an error.
int ensure_device_ready();
int sm_count();

} // namespace rc
