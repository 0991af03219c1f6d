// C ABI of libreinstinct_cuda.so: argument checks, dispatch and the device-API mirror.
// The declarations and the reference interfaces they stand in for are in
// include/reinstinct_cuda.h.
#include <cstdio>
#include <cstring>

#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {

namespace {
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices];
bool g_ready[kMaxDevices];
} // namespace



int sm_count()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    return g_sm_count[dev] > 0 ? g_sm_count[dev] : 148;
}

int ensure_device_ready()
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return RC_ERR_NO_DEVICE;
    if (g_ready[dev]) return RC_OK;
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return (int)e;
    // The kernels are sm_100a only; there is no other code path to fall back to.
    if (prop.major != 10) return RC_ERR_NO_DEVICE;
    g_sm_count[dev] = prop.multiProcessorCount;
    int rc = matvec_set_attributes();
    if (rc) return rc;
    rc = mmq_set_attributes();
    if (rc) return rc;
    rc = mmq_deq_set_attributes();
    if (rc) return rc;
    rc = mmq_x_set_attributes();
    if (rc) return rc;
    rc = moe_set_attributes();
    if (rc) return rc;
    g_ready[dev] = true;
    return RC_OK;
}

namespace {

inline cudaStream_t S(void *s) { return reinterpret_cast<cudaStream_t>(s); }

int check_weight_args(int type, const void *w, const void *xq, const void *y, uint32_t in_dim,
                      uint32_t out_dim)
{
    if (!fmt_known(type)) return RC_ERR_BAD_TYPE;
    if (in_dim == 0 || out_dim == 0 || in_dim % fmt_block_weights(type)) return RC_ERR_BAD_SHAPE;
    if (!w || !xq || !y) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)w & 15u) || ((uintptr_t)xq & 7u) || ((uintptr_t)y & 3u)) return RC_ERR_MISALIGNED;
    return RC_OK;
}

} // namespace
} // namespace rc

using namespace rc;

extern "C" {

int rc_abi_version(void) { return RC_ABI_VERSION; }

int rc_init(int device)
{
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return (int)e;
    return ensure_device_ready();
}

const char *rc_error_string(int code)
{
    switch (code) {
    case RC_OK: return "success";
    case RC_ERR_BAD_TYPE: return "unsupported ggml type (expected Q4_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS or IQ3_S planes)";
    case RC_ERR_BAD_SHAPE: return "bad shape (zero dimension, or in_dim not a multiple of the format's block size)";
    case RC_ERR_NULL_POINTER: return "null pointer argument";
    case RC_ERR_MISALIGNED: return "misaligned pointer (weights need 16 bytes, BlockQ8 8 bytes, f32 4 bytes)";
    case RC_ERR_TOO_MANY_ROWS: return "too many activation rows for this entry point";
    case RC_ERR_SCRATCH_TOO_SMALL: return "scratch buffer too small";
    case RC_ERR_NO_DEVICE: return "no usable sm_100 device";
    case RC_ERR_BAD_ARGUMENT: return "bad argument";
    case RC_ERR_STATIC_LIMIT: return "in_dim exceeds RC_NOALLOC_MAX_IN_DIM, the fixed scratch of rc_matvec_f32_noalloc";
    }
    if (code > 0) return cudaGetErrorString((cudaError_t)code);
    return "unknown reinstinct_cuda error";
}

size_t rc_repacked_n_sub_padded(size_t in_dim) { return nsp_of((uint32_t)(in_dim / 32)); }

size_t rc_repacked_len(int type, size_t in_dim, size_t out_dim)
{
    return repacked_len_of(type, in_dim, out_dim);
}

size_t rc_ondisk_len(int type, size_t in_dim, size_t out_dim)
{
    if (type == SRC_Q3_K || type == SRC_IQ4_NL || type == SRC_BF16) {
        // the relabelled tensor must be a legal tensor of its kernel type
        if (in_dim == 0 || in_dim % fmt_block_weights(fmt_kernel_type(type))) return 0;
        return out_dim * (in_dim / src_block_weights(type)) * src_block_bytes(type);
    }
    if (!fmt_known(type) || in_dim == 0 || in_dim % fmt_block_weights(type)) return 0;
    return out_dim * (in_dim / fmt_block_weights(type)) * fmt_block_bytes(type);
}

int rc_kernel_type(int src_type) { return fmt_kernel_type(src_type); }

int rc_repack_for_matvec(void *stream, int type, const void *blocks_dev, size_t in_dim,
                         size_t out_dim, void *out_dev)
{
    const int ktype = fmt_kernel_type(type); // a source-only type is repacked as the type it relabels onto
    if (ktype < 0) return RC_ERR_BAD_TYPE;
    if (in_dim == 0 || in_dim % fmt_block_weights(ktype) || in_dim > 0xFFFFFFE0ull ||
        out_dim > 0xFFFFFFFFull)
        return RC_ERR_BAD_SHAPE;
    if (out_dim == 0) return RC_OK;
    if (!blocks_dev || !out_dev) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)out_dev & 15u) || ((uintptr_t)blocks_dev & 1u)) return RC_ERR_MISALIGNED;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_repack(S(stream), type, blocks_dev, in_dim, out_dim, out_dev);
}

int rc_quantize_q8(void *stream, const float *x, void *xq, uint32_t in_dim, uint32_t n_vec)
{
    if (in_dim == 0 || in_dim % 32) return RC_ERR_BAD_SHAPE;
    if (n_vec == 0) return RC_OK;
    if (!x || !xq) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)x & 3u) || ((uintptr_t)xq & 7u)) return RC_ERR_MISALIGNED;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_quantize_q8(S(stream), x, xq, in_dim, n_vec);
}

int rc_matvec(void *stream, int type, const void *w, const void *xq, float *y, uint32_t in_dim,
              uint32_t out_dim)
{
    int rc = check_weight_args(type, w, xq, y, in_dim, out_dim);
    if (rc) return rc;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_matvec(S(stream), type, w, xq, y, in_dim, out_dim, 1, nullptr);
}

int rc_matvec_batched(void *stream, int type, const void *w, const void *xq, float *y,
                      uint32_t in_dim, uint32_t out_dim, uint32_t n_rows)
{
    if (n_rows == 0) return RC_OK;
    if (n_rows > RC_MATVEC_MAX_ROWS) return RC_ERR_TOO_MANY_ROWS;
    int rc = check_weight_args(type, w, xq, y, in_dim, out_dim);
    if (rc) return rc;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_matvec(S(stream), type, w, xq, y, in_dim, out_dim, n_rows, nullptr);
}

int rc_matvec_block_dots(void *stream, int type, const void *w, const void *xq, int32_t *idots,
                         uint32_t in_dim, uint32_t out_dim, uint32_t n_rows)
{
    if (n_rows == 0) return RC_OK;
    if (n_rows > RC_MATVEC_MAX_ROWS) return RC_ERR_TOO_MANY_ROWS;
    int rc = check_weight_args(type, w, xq, idots, in_dim, out_dim);
    if (rc) return rc;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_matvec(S(stream), type, w, xq, nullptr, in_dim, out_dim, n_rows, idots);
}

size_t rc_matmul_scratch_bytes(uint32_t in_dim, uint32_t n_rows)
{
    // BlockQ8 records, or the planar form of the same values (a few bytes of row padding more)
    const size_t records = (size_t)n_rows * (in_dim / 32) * RC_BLOCKQ8_BYTES;
    const size_t planar = quantize_planar_bytes(in_dim, n_rows);
    // beyond the matvec's row limit: the operand image of the activations the dense GEMM reads (the
    // integer-valued one of the default route, or the dequantized one of rc_matmul_f16)
    const size_t image = n_rows > RC_MATVEC_MAX_ROWS ? mmq_x_scratch_bytes(in_dim, n_rows) : 0;
    const size_t image_deq = n_rows > RC_MATVEC_MAX_ROWS ? mmq_deq_scratch_bytes(in_dim, n_rows) : 0;
    size_t m = records > planar ? records : planar;
    m = m > image ? m : image;
    return m > image_deq ? m : image_deq;
}

int rc_matvec_f32(void *stream, int type, const void *w, const float *x, float *y, uint32_t in_dim,
                  uint32_t out_dim, void *xq_scratch, size_t scratch_bytes)
{
    return rc_matmul(stream, type, w, x, y, in_dim, out_dim, 1, xq_scratch, scratch_bytes);
}

int rc_mmq_gemm(void *stream, int type, const void *w, const void *xq, float *y, uint32_t in_dim,
                uint32_t out_dim, uint32_t p_rows)
{
    if (p_rows == 0) return RC_OK;
    int rc = check_weight_args(type, w, xq, y, in_dim, out_dim);
    if (rc) return rc;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_mmq_gemm(S(stream), type, w, xq, y, in_dim, out_dim, p_rows);
}

int rc_matmul(void *stream, int type, const void *w, const float *x, float *y, uint32_t in_dim,
              uint32_t out_dim, uint32_t n_rows, void *xq_scratch, size_t scratch_bytes)
{
    if (n_rows == 0) return RC_OK;
    if (!x) return RC_ERR_NULL_POINTER;
    int rc = check_weight_args(type, w, xq_scratch, y, in_dim, out_dim);
    if (rc) return rc;
    if (scratch_bytes < (size_t)n_rows * (in_dim / 32) * RC_BLOCKQ8_BYTES) return RC_ERR_SCRATCH_TOO_SMALL;
    rc = ensure_device_ready();
    if (rc) return rc;
    // Row-count dispatch of PrefillGemm::matmul_into_raw (src/runtime/prefill.rs:343-437):
    // few rows stream the weights once through the matvec, more rows go to the tensor cores.
    if (n_rows <= RC_MATVEC_MAX_ROWS) {
        rc = launch_quantize_q8(S(stream), x, xq_scratch, in_dim, n_rows);
        if (rc) return rc;
        return launch_matvec(S(stream), type, w, xq_scratch, y, in_dim, out_dim, n_rows, nullptr);
    }
    return launch_mmq_gemm_f32(S(stream), type, w, x, y, in_dim, out_dim, n_rows, xq_scratch, scratch_bytes);
}

int rc_matmul_f16(void *stream, int type, const void *w, const float *x, float *y, uint32_t in_dim,
                  uint32_t out_dim, uint32_t n_rows, void *scratch, size_t scratch_bytes)
{
    if (n_rows == 0) return RC_OK;
    if (!x) return RC_ERR_NULL_POINTER;
    int rc = check_weight_args(type, w, scratch, y, in_dim, out_dim);
    if (rc) return rc;
    if (((uintptr_t)scratch & 15u)) return RC_ERR_MISALIGNED;
    if (scratch_bytes < mmq_deq_scratch_bytes(in_dim, n_rows)) return RC_ERR_SCRATCH_TOO_SMALL;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_mmq_deq_f32(S(stream), type, w, x, y, in_dim, out_dim, n_rows, scratch);
}

int rc_matmul_block_dots(void *stream, int type, const void *w, const float *x, float *y, int32_t *idots,
                         uint32_t in_dim, uint32_t out_dim, uint32_t n_rows, void *scratch, size_t scratch_bytes)
{
    if (n_rows == 0) return RC_OK;
    if (!x || !idots) return RC_ERR_NULL_POINTER;
    int rc = check_weight_args(type, w, scratch, y, in_dim, out_dim);
    if (rc) return rc;
    if (!mmq_x_supports(type)) return RC_ERR_BAD_TYPE;
    if (((uintptr_t)scratch & 15u) || ((uintptr_t)idots & 3u)) return RC_ERR_MISALIGNED;
    if (scratch_bytes < mmq_x_scratch_bytes(in_dim, n_rows)) return RC_ERR_SCRATCH_TOO_SMALL;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_mmq_x_f32(S(stream), type, w, x, y, in_dim, out_dim, n_rows, scratch, idots);
}

/* ---- allocation-free matvec ---------------------------------------------------------------- */

} // extern "C"

namespace {
// Quantized-activation scratch of rc_matvec_f32_noalloc.  In host code this name is only a
// handle for cudaGetSymbolAddress; kernels must be given the address that call returns.
static __device__ __align__(256) unsigned char g_noalloc_xq[RC_NOALLOC_SCRATCH_BYTES];
void *g_noalloc_ptr[kMaxDevices];

// Device address of g_noalloc_xq on the current device, looked up once per device.
int noalloc_scratch(void **out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return RC_ERR_NO_DEVICE;
    if (!g_noalloc_ptr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_xq);
        if (e != cudaSuccess) return (int)e;
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return RC_OK;
}
} // namespace

extern "C" {

int rc_matvec_f32_noalloc(void *stream, int type, const void *w, const float *x, float *y,
                          uint32_t in_dim, uint32_t out_dim)
{
    if (!x) return RC_ERR_NULL_POINTER;
    if (in_dim > RC_NOALLOC_MAX_IN_DIM) return RC_ERR_STATIC_LIMIT;
    int rc = ensure_device_ready();
    if (rc) return rc;
    void *xq = nullptr;
    rc = noalloc_scratch(&xq);
    if (rc) return rc;
    rc = check_weight_args(type, w, xq, y, in_dim, out_dim);
    if (rc) return rc;
    if (((uintptr_t)x & 3u)) return RC_ERR_MISALIGNED;
    // the quantizer rewrites every block the matvec reads, so stale contents never matter
    rc = launch_quantize_q8(S(stream), x, xq, in_dim, 1);
    if (rc) return rc;
    return launch_matvec(S(stream), type, w, xq, y, in_dim, out_dim, 1, nullptr);
}

uint32_t rc_moe_tile_bn(void) { return matvec_grouped_bn(); }

int rc_moe_sort(void *stream, const int32_t *ids, uint32_t n_entries, uint32_t n_expert,
                uint32_t bn, int32_t *count, int32_t *cursor, int32_t *expert_off,
                int32_t *tile_off, int32_t *perm)
{
    if (n_expert == 0 || bn == 0) return RC_ERR_BAD_ARGUMENT;
    if (!count || !cursor || !expert_off || !tile_off) return RC_ERR_NULL_POINTER;
    if (n_entries && (!ids || !perm)) return RC_ERR_NULL_POINTER;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_moe_sort(S(stream), ids, n_entries, n_expert, bn, count, cursor, expert_off,
                           tile_off, perm);
}

int rc_moe_gather_xq(void *stream, const void *xq_src, const int32_t *perm, void *xq_dst,
                     uint32_t n_sub, uint32_t n_used, uint32_t n_entries)
{
    if (n_entries == 0 || n_sub == 0) return RC_OK;
    if (n_used == 0) return RC_ERR_BAD_ARGUMENT;
    if (!xq_src || !perm || !xq_dst) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)xq_src & 7u) || ((uintptr_t)xq_dst & 7u)) return RC_ERR_MISALIGNED;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_moe_gather_xq(S(stream), xq_src, perm, xq_dst, n_sub, n_used, n_entries);
}

int rc_moe_scatter_rows(void *stream, const float *src, const int32_t *perm, float *dst,
                        uint32_t dim, uint32_t n_entries)
{
    if (n_entries == 0 || dim == 0) return RC_OK;
    if (!src || !perm || !dst) return RC_ERR_NULL_POINTER;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_moe_scatter_rows(S(stream), src, perm, dst, dim, n_entries);
}

int rc_mmq_gemm_grouped(void *stream, int type, const void *slab, size_t bytes_per_expert,
                        const int32_t *expert_off, const int32_t *tile_off, uint32_t n_expert,
                        const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
                        uint32_t n_entries)
{
    if (n_entries == 0) return RC_OK;
    if (n_expert == 0) return RC_ERR_BAD_ARGUMENT;
    int rc = check_weight_args(type, slab, xq, y, in_dim, out_dim);
    if (rc) return rc;
    if (!expert_off || !tile_off) return RC_ERR_NULL_POINTER;
    if (bytes_per_expert < repacked_len_of(type, in_dim, out_dim)) return RC_ERR_BAD_ARGUMENT;
    // every expert's planes are read with 16-byte loads
    if (n_expert > 1 && (bytes_per_expert & 15u)) return RC_ERR_MISALIGNED;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_mmq_grouped(S(stream), type, slab, bytes_per_expert, expert_off, tile_off,
                              n_expert, xq, y, in_dim, out_dim, n_entries);
}

/* ---- fused BlockQ8 producers ------------------------------------------------------------------- */

int rc_add_rmsnorm_q8(void *stream, float *hidden, const float *add, const float *w, float *y, void *out, uint32_t n,
                      uint32_t n_vec, float eps)
{
    if (n == 0 || n % 32) return RC_ERR_BAD_SHAPE;
    if (n_vec == 0) return RC_OK;
    if (!hidden || !w || !out) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)hidden & 3u) || ((uintptr_t)add & 3u) || ((uintptr_t)w & 3u) || ((uintptr_t)y & 3u) || ((uintptr_t)out & 7u))
        return RC_ERR_MISALIGNED;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_rmsnorm_q8(S(stream), hidden, add, w, hidden, y, out, n, n_vec, eps);
}

int rc_rmsnorm_q8(void *stream, const float *x, const float *w, void *out, uint32_t n, uint32_t n_vec, float eps)
{
    if (n == 0 || n % 32) return RC_ERR_BAD_SHAPE;
    if (n_vec == 0) return RC_OK;
    if (!x || !w || !out) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)x & 3u) || ((uintptr_t)w & 3u) || ((uintptr_t)out & 7u)) return RC_ERR_MISALIGNED;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_rmsnorm_q8(S(stream), x, nullptr, w, nullptr, nullptr, out, n, n_vec, eps);
}

int rc_sigmoid_mul_q8(void *stream, float *x, const float *gate, void *q8, size_t n)
{
    if (n % 32) return RC_ERR_BAD_SHAPE;
    if (n == 0) return RC_OK;
    if (!x || !gate || !q8) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)x & 3u) || ((uintptr_t)gate & 3u) || ((uintptr_t)q8 & 7u)) return RC_ERR_MISALIGNED;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_sigmoid_mul_q8(S(stream), x, gate, q8, n);
}

int rc_rmsnorm_gated_q8(void *stream, const float *x, const float *z, const float *w, float *y, void *q8, uint32_t n_heads,
                        uint32_t head_dim, float eps)
{
    if (head_dim == 0 || head_dim % 32 || head_dim > 1024) return RC_ERR_BAD_SHAPE;
    if (n_heads == 0) return RC_OK;
    if (!x || !z || !w || !q8) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)x & 3u) || ((uintptr_t)z & 3u) || ((uintptr_t)w & 3u) || ((uintptr_t)y & 3u) || ((uintptr_t)q8 & 7u))
        return RC_ERR_MISALIGNED;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_rmsnorm_gated_q8(S(stream), x, z, w, y, q8, n_heads, head_dim, eps);
}

int rc_swiglu_q8(void *stream, const float *gate, const float *up, float *out, void *q8, size_t n)
{
    if (n % 32) return RC_ERR_BAD_SHAPE;
    if (n == 0) return RC_OK;
    if (!gate || !up || !q8) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)gate & 3u) || ((uintptr_t)up & 3u) || ((uintptr_t)out & 3u) || ((uintptr_t)q8 & 7u)) return RC_ERR_MISALIGNED;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_swiglu_q8(S(stream), gate, up, out, q8, n);
}

size_t rc_mmq_gemm_grouped_scratch_bytes(uint32_t in_dim, uint32_t n_entries)
{
    return mmq_deq_grouped_scratch_bytes(in_dim, n_entries);
}

int rc_mmq_gemm_grouped_f32(void *stream, int type, const void *slab, size_t bytes_per_expert, const int32_t *expert_off,
                            const int32_t *tile_off, uint32_t n_expert, const float *x, const int32_t *index, uint32_t div,
                            size_t row_stride, int act, float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_entries,
                            void *scratch, size_t scratch_bytes)
{
    if (n_entries == 0) return RC_OK;
    int rc = check_weight_args(type, slab, scratch, y, in_dim, out_dim);
    if (rc) return rc;
    if (!x || !expert_off || !tile_off) return RC_ERR_NULL_POINTER;
    if (n_expert == 0 || act < -1 || act > 1 || (index && div == 0) || row_stride < (size_t)in_dim * (act >= 0 ? 2u : 1u))
        return RC_ERR_BAD_ARGUMENT;
    if (((uintptr_t)scratch & 15u) || ((uintptr_t)x & 3u) || (n_expert > 1 && (bytes_per_expert & 15u))) return RC_ERR_MISALIGNED;
    if (scratch_bytes < mmq_deq_grouped_scratch_bytes(in_dim, n_entries)) return RC_ERR_SCRATCH_TOO_SMALL;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_mmq_deq_grouped_f32(S(stream), type, slab, bytes_per_expert, expert_off, tile_off, n_expert, x, index, div,
                                      row_stride, act, y, in_dim, out_dim, n_entries, scratch);
}

int rc_moe_expert_matvec(void *stream, int type, const void *slab, size_t bytes_per_expert, const int32_t *ids,
                         uint32_t n_expert, const void *xq, float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_used,
                         uint32_t n_tok, uint32_t xq_tok_stride, uint32_t xq_slot_stride)
{
    if (n_tok == 0 || n_used == 0) return RC_OK;
    int rc = check_weight_args(type, slab, xq, y, in_dim, out_dim);
    if (rc) return rc;
    if (!ids) return RC_ERR_NULL_POINTER;
    if (n_expert == 0 || n_used > 65535u) return RC_ERR_BAD_ARGUMENT;
    if (n_expert > 1 && (bytes_per_expert & 15u)) return RC_ERR_MISALIGNED;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_moe_expert_matvec(S(stream), type, slab, bytes_per_expert, ids, n_expert, xq, y, in_dim, out_dim, n_used,
                                    n_tok, xq_tok_stride, xq_slot_stride);
}

int rc_moe_gate_up_swiglu(void *stream, int type, const void *gate_slab, const void *up_slab, size_t bytes_per_expert,
                          const int32_t *ids, uint32_t n_expert, const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
                          uint32_t n_used, uint32_t n_tok, uint32_t xq_tok_stride, uint32_t xq_slot_stride)
{
    if (n_tok == 0 || n_used == 0) return RC_OK;
    int rc = check_weight_args(type, gate_slab, xq, y, in_dim, out_dim);
    if (rc) return rc;
    if (!up_slab || !ids) return RC_ERR_NULL_POINTER;
    if ((uintptr_t)up_slab & 15u) return RC_ERR_MISALIGNED;
    if (in_dim % 1024u) return RC_ERR_BAD_SHAPE;
    if (n_expert == 0 || n_used > 65535u) return RC_ERR_BAD_ARGUMENT;
    if (n_expert > 1 && (bytes_per_expert & 15u)) return RC_ERR_MISALIGNED;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_moe_gate_up_swiglu(S(stream), type, gate_slab, up_slab, bytes_per_expert, ids, n_expert, xq, y, in_dim, out_dim,
                                     n_used, n_tok, xq_tok_stride, xq_slot_stride);
}

/* ---- MoE glue ------------------------------------------------------------------------------------ */

int rc_moe_topk(void *stream, const float *logits, uint32_t n_tok, uint32_t n_expert, uint32_t n_used,
                int32_t *ids, float *weights)
{
    if (n_tok == 0) return RC_OK;
    if (n_expert == 0 || n_expert > 1024 || n_used == 0 || n_used > 32 || n_used > n_expert) return RC_ERR_BAD_ARGUMENT;
    if (!logits || !ids || !weights) return RC_ERR_NULL_POINTER;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_moe_topk(S(stream), logits, n_tok, n_expert, n_used, ids, weights);
}

int rc_moe_act_q8(void *stream, const float *gu, void *out, uint32_t ff, uint32_t n_slot, int act)
{
    if (ff == 0 || ff % 32) return RC_ERR_BAD_SHAPE;
    if (act != RC_ACT_GEGLU && act != RC_ACT_SWIGLU) return RC_ERR_BAD_ARGUMENT;
    if (n_slot == 0) return RC_OK;
    if (!gu || !out) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)gu & 3u) || ((uintptr_t)out & 7u)) return RC_ERR_MISALIGNED;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_moe_act_q8(S(stream), gu, out, ff, n_slot, act);
}

int rc_moe_combine(void *stream, const float *experts, const int32_t *ids, const float *weights,
                   const float *expert_scale, float *out, uint32_t hidden, uint32_t n_used, uint32_t n_tok)
{
    if (n_tok == 0 || hidden == 0) return RC_OK;
    if (n_used == 0) return RC_ERR_BAD_ARGUMENT;
    if (!experts || !ids || !weights || !out) return RC_ERR_NULL_POINTER;
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_moe_combine(S(stream), experts, ids, weights, expert_scale, out, hidden, n_used, n_tok);
}

/* ---- peer gather -------------------------------------------------------------------------------- */

int rc_ipc_get_handle(const void *dev_ptr, void *handle)
{
    if (!dev_ptr || !handle) return RC_ERR_NULL_POINTER;
    static_assert(sizeof(cudaIpcMemHandle_t) == RC_IPC_HANDLE_BYTES, "IPC handle size");
    return (int)cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(handle), const_cast<void *>(dev_ptr));
}
int rc_ipc_open_handle(const void *handle, void **dev_ptr)
{
    if (!dev_ptr || !handle) return RC_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    return (int)cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
int rc_ipc_close_handle(void *dev_ptr) { return (int)cudaIpcCloseMemHandle(dev_ptr); }

int rc_peer_barrier(void *stream, void *const *peer_flags, void *epoch, uint32_t rank, uint32_t world)
{
    if (world == 0 || world > RC_MAX_PEERS || rank >= world) return RC_ERR_BAD_ARGUMENT;
    if (!peer_flags || !epoch) return RC_ERR_NULL_POINTER;
    for (uint32_t r = 0; r < world; r++) {
        if (!peer_flags[r]) return RC_ERR_NULL_POINTER;
        if ((uintptr_t)peer_flags[r] & 7u) return RC_ERR_MISALIGNED;
    }
    // the gather kernel with an empty shard: epoch publication and the bounded wait only
    return launch_allgather_push(S(stream), nullptr, 0, peer_flags, peer_flags, epoch, rank, world);
}

int rc_allgather_push_logical(void *stream, const void *const *srcs, size_t bytes, void *const *dsts, void *const *flags,
                              void *const *epochs, uint32_t world)
{
    if (world == 0 || world > RC_MAX_PEERS) return RC_ERR_BAD_ARGUMENT;
    if (bytes % 16 || bytes / 16 > 0xFFFFFFFFull) return RC_ERR_BAD_SHAPE;
    if (!srcs || !dsts || !flags || !epochs) return RC_ERR_NULL_POINTER;
    for (uint32_t r = 0; r < world; r++) {
        if (!srcs[r] || !dsts[r] || !flags[r] || !epochs[r]) return RC_ERR_NULL_POINTER;
        if (((uintptr_t)srcs[r] & 15u) || ((uintptr_t)dsts[r] & 15u) || ((uintptr_t)flags[r] & 7u) || ((uintptr_t)epochs[r] & 7u))
            return RC_ERR_MISALIGNED;
    }
    return launch_allgather_push_logical(S(stream), srcs, bytes, dsts, flags, epochs, world);
}

int rc_matmul_gather(void *stream, int type, const void *w, const float *x, float *const *y_peers, uint32_t world,
                     uint32_t out_total, uint32_t row_begin, uint32_t in_dim, uint32_t out_dim, uint32_t n_rows, void *scratch,
                     size_t scratch_bytes)
{
    if (n_rows == 0) return RC_OK;
    if (world == 0 || world > RC_MAX_PEERS) return RC_ERR_BAD_ARGUMENT;
    if (!x || !y_peers) return RC_ERR_NULL_POINTER;
    for (uint32_t g = 0; g < world; g++)
        if (!y_peers[g]) return RC_ERR_NULL_POINTER;
    int rc = check_weight_args(type, w, scratch, y_peers[0], in_dim, out_dim);
    if (rc) return rc;
    if (!mmq_x_supports(type)) return RC_ERR_BAD_TYPE;
    if ((uint64_t)row_begin + out_dim > out_total) return RC_ERR_BAD_SHAPE;
    if (((uintptr_t)scratch & 15u)) return RC_ERR_MISALIGNED;
    if (scratch_bytes < mmq_x_scratch_bytes(in_dim, n_rows)) return RC_ERR_SCRATCH_TOO_SMALL;
    rc = ensure_device_ready();
    if (rc) return rc;
    return launch_mmq_x_f32(S(stream), type, w, x, nullptr, in_dim, out_dim, n_rows, scratch, nullptr, y_peers, world, out_total,
                            row_begin);
}

size_t rc_ffn_decode_work_bytes(uint32_t ffn_local) { return ffn_decode_work_bytes(ffn_local); }

int rc_ffn_decode(void *stream, int gate_type, int down_type, const void *gate_w, const void *up_w, const void *down_w,
                  const float *x, float *y, uint32_t in_dim, uint32_t ffn_local, uint32_t ffn_total, uint32_t ffn_begin,
                  uint32_t out_local, uint32_t out_total, uint32_t out_begin, uint32_t world, uint32_t rank,
                  void *const *h_peers, void *const *y_peers, void *work)
{
    if (world == 0 || world > RC_MAX_PEERS || rank >= world) return RC_ERR_BAD_ARGUMENT;
    if (!fmt_known(gate_type) || !fmt_known(down_type)) return RC_ERR_BAD_TYPE;
    // whole 1024-wide iterations on both contractions
    if (in_dim == 0 || in_dim % 1024u || ffn_total == 0 || ffn_total % 1024u || ffn_local == 0 || out_local == 0 ||
        (uint64_t)ffn_begin + ffn_local > ffn_total || (uint64_t)out_begin + out_local > out_total)
        return RC_ERR_BAD_SHAPE;
    if (!gate_w || !up_w || !down_w || !x || !y || !h_peers || !y_peers || !work) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)gate_w & 15u) || ((uintptr_t)up_w & 15u) || ((uintptr_t)down_w & 15u) || ((uintptr_t)x & 15u) || ((uintptr_t)y & 3u) ||
        ((uintptr_t)work & 15u))
        return RC_ERR_MISALIGNED;
    for (uint32_t r = 0; r < world; r++) {
        if (!h_peers[r] || !y_peers[r]) return RC_ERR_NULL_POINTER;
        if (((uintptr_t)h_peers[r] & 15u) || ((uintptr_t)y_peers[r] & 3u)) return RC_ERR_MISALIGNED;
    }
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_ffn_decode(S(stream), gate_type, down_type, gate_w, up_w, down_w, x, in_dim, ffn_local, ffn_total, ffn_begin,
                             out_local, out_total, out_begin, world, rank, h_peers, y_peers, y, work);
}

size_t rc_ffn_decode_tp_work_bytes(uint32_t ffn_local) { return ffn_decode_tp_work_bytes(ffn_local); }

int rc_ffn_decode_tp(void *stream, int gate_type, int down_type, const void *gate_w, const void *up_w, const void *down_w,
                     const float *x, float *y, uint32_t in_dim, uint32_t ffn_local, uint32_t out_total, uint32_t world,
                     uint32_t rank, void *const *part_peers, void *work)
{
    if (world == 0 || world > RC_MAX_PEERS || rank >= world) return RC_ERR_BAD_ARGUMENT;
    if (!fmt_known(gate_type) || !fmt_known(down_type)) return RC_ERR_BAD_TYPE;
    // whole 1024-wide iterations on the first contraction; the slice of the second one in whole blocks of the down format
    if (in_dim == 0 || in_dim % 1024u || ffn_local == 0 || ffn_local % fmt_block_weights(down_type) || ffn_local % 32u || out_total == 0)
        return RC_ERR_BAD_SHAPE;
    if (!gate_w || !up_w || !down_w || !x || !y || !part_peers || !work) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)gate_w & 15u) || ((uintptr_t)up_w & 15u) || ((uintptr_t)down_w & 15u) || ((uintptr_t)x & 15u) || ((uintptr_t)y & 3u) ||
        ((uintptr_t)work & 15u))
        return RC_ERR_MISALIGNED;
    for (uint32_t r = 0; r < world; r++) {
        if (!part_peers[r]) return RC_ERR_NULL_POINTER;
        if ((uintptr_t)part_peers[r] & 3u) return RC_ERR_MISALIGNED;
    }
    int rc = ensure_device_ready();
    if (rc) return rc;
    return launch_ffn_decode_tp(S(stream), gate_type, down_type, gate_w, up_w, down_w, x, y, in_dim, ffn_local, out_total, world, rank,
                                part_peers, work);
}

int rc_ep_plan(void *stream, const int32_t *ids, uint32_t n_entries, uint32_t experts_per_rank, uint32_t cap, uint32_t world,
               int32_t *back)
{
    if (world == 0 || world > RC_MAX_PEERS || experts_per_rank == 0 || cap == 0) return RC_ERR_BAD_ARGUMENT;
    if (n_entries == 0) return RC_OK;
    if (!ids || !back) return RC_ERR_NULL_POINTER;
    return launch_ep_plan(S(stream), ids, n_entries, experts_per_rank, cap, world, back);
}

int rc_ep_dispatch(void *stream, const int32_t *ids, const int32_t *back, const void *xq, uint32_t n_entries, uint32_t n_used,
                   uint32_t in_dim, uint32_t experts_per_rank, uint32_t cap, uint32_t rank, uint32_t world, uint32_t buf,
                   void *const *rows_peers, void *const *ids_peers)
{
    if (world == 0 || world > RC_MAX_PEERS || rank >= world || experts_per_rank == 0 || cap == 0 || n_used == 0) return RC_ERR_BAD_ARGUMENT;
    if (in_dim == 0 || in_dim % 32u) return RC_ERR_BAD_SHAPE;
    if (!rows_peers || !ids_peers || (n_entries && (!ids || !back || !xq))) return RC_ERR_NULL_POINTER;
    if ((uintptr_t)xq & 7u) return RC_ERR_MISALIGNED;
    for (uint32_t r = 0; r < world; r++) {
        if (!rows_peers[r] || !ids_peers[r]) return RC_ERR_NULL_POINTER;
        if (((uintptr_t)rows_peers[r] & 7u) || ((uintptr_t)ids_peers[r] & 3u)) return RC_ERR_MISALIGNED;
    }
    return launch_ep_dispatch(S(stream), ids, back, xq, n_entries, n_used, in_dim / 32u, experts_per_rank, cap, rank, world, buf, rows_peers,
                              ids_peers);
}

int rc_ep_return(void *stream, const int32_t *ids_in, const float *y_in, uint32_t dim, uint32_t cap, uint32_t rank, uint32_t world,
                 void *const *ret_peers)
{
    if (world == 0 || world > RC_MAX_PEERS || rank >= world || cap == 0) return RC_ERR_BAD_ARGUMENT;
    if (dim == 0 || dim % 4u) return RC_ERR_BAD_SHAPE;
    if (!ids_in || !y_in || !ret_peers) return RC_ERR_NULL_POINTER;
    if ((uintptr_t)y_in & 15u) return RC_ERR_MISALIGNED;
    for (uint32_t r = 0; r < world; r++) {
        if (!ret_peers[r]) return RC_ERR_NULL_POINTER;
        if ((uintptr_t)ret_peers[r] & 15u) return RC_ERR_MISALIGNED;
    }
    return launch_ep_return(S(stream), ids_in, y_in, dim, cap, rank, world, ret_peers);
}

int rc_ep_collect(void *stream, const int32_t *back, const float *ret, float *out, uint32_t dim, uint32_t n_entries)
{
    if (dim == 0 || dim % 4u) return RC_ERR_BAD_SHAPE;
    if (n_entries == 0) return RC_OK;
    if (!back || !ret || !out) return RC_ERR_NULL_POINTER;
    if (((uintptr_t)ret & 15u) || ((uintptr_t)out & 15u)) return RC_ERR_MISALIGNED;
    return launch_ep_collect(S(stream), back, ret, out, dim, n_entries);
}

int rc_allgather_push(void *stream, const void *src, size_t bytes, void *const *peer_dst,
                      void *const *peer_flags, void *epoch, uint32_t rank, uint32_t world)
{
    if (world == 0 || world > RC_MAX_PEERS || rank >= world) return RC_ERR_BAD_ARGUMENT;
    if (bytes == 0) return RC_OK;
    if (bytes % 16 || bytes / 16 > 0xFFFFFFFFull) return RC_ERR_BAD_SHAPE;
    if (!src || !peer_dst || !peer_flags || !epoch) return RC_ERR_NULL_POINTER;
    if ((uintptr_t)src & 15u) return RC_ERR_MISALIGNED;
    for (uint32_t r = 0; r < world; r++) {
        if (!peer_dst[r] || !peer_flags[r]) return RC_ERR_NULL_POINTER;
        if (((uintptr_t)peer_dst[r] & 15u) || ((uintptr_t)peer_flags[r] & 7u)) return RC_ERR_MISALIGNED;
    }
    return launch_allgather_push(S(stream), src, bytes, peer_dst, peer_flags, epoch, rank, world);
}

/* ---- device API mirror ------------------------------------------------------------------- */

int rc_get_device_count(int *count) { return count ? (int)cudaGetDeviceCount(count) : RC_ERR_NULL_POINTER; }
int rc_set_device(int device) { return (int)cudaSetDevice(device); }
int rc_get_device(int *device) { return device ? (int)cudaGetDevice(device) : RC_ERR_NULL_POINTER; }

int rc_device_get_name(char *name, int len, int device)
{
    if (!name || len <= 0) return RC_ERR_NULL_POINTER;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return (int)e;
    std::snprintf(name, (size_t)len, "%s", prop.name);
    return RC_OK;
}

int rc_device_total_mem(size_t *bytes, int device)
{
    if (!bytes) return RC_ERR_NULL_POINTER;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return (int)e;
    *bytes = prop.totalGlobalMem;
    return RC_OK;
}

int rc_mem_get_info(size_t *free_bytes, size_t *total_bytes)
{
    if (!free_bytes || !total_bytes) return RC_ERR_NULL_POINTER;
    return (int)cudaMemGetInfo(free_bytes, total_bytes);
}

int rc_device_can_access_peer(int *can, int device, int peer)
{
    return can ? (int)cudaDeviceCanAccessPeer(can, device, peer) : RC_ERR_NULL_POINTER;
}

int rc_device_enable_peer_access(int peer)
{
    cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError(); // clear the sticky-less error state
        return RC_OK;
    }
    return (int)e;
}

int rc_device_synchronize(void) { return (int)cudaDeviceSynchronize(); }

int rc_malloc(void **ptr, size_t bytes) { return ptr ? (int)cudaMalloc(ptr, bytes) : RC_ERR_NULL_POINTER; }
int rc_free(void *ptr) { return (int)cudaFree(ptr); }

int rc_memcpy(void *dst, const void *src, size_t bytes, int kind)
{
    return (int)cudaMemcpy(dst, src, bytes, (cudaMemcpyKind)kind);
}
int rc_memcpy_async(void *dst, const void *src, size_t bytes, int kind, void *stream)
{
    return (int)cudaMemcpyAsync(dst, src, bytes, (cudaMemcpyKind)kind, S(stream));
}
// A small copy done by the SMs: 16-byte words, one CTA per 16 KB.
static __global__ void __launch_bounds__(1024) rc_copy_small_kernel(uint4 *__restrict__ dst, const uint4 *__restrict__ src, uint32_t n16)
{
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

int rc_copy_small(void *stream, void *dst, const void *src, size_t bytes)
{
    if (bytes == 0) return RC_OK;
    if (!dst || !src) return RC_ERR_NULL_POINTER;
    if (bytes % 16 || bytes > (1u << 24)) return RC_ERR_BAD_SHAPE;
    if (((uintptr_t)dst & 15u) || ((uintptr_t)src & 15u)) return RC_ERR_MISALIGNED;
    const uint32_t n16 = (uint32_t)(bytes / 16);
    rc_copy_small_kernel<<<std::min<uint32_t>((n16 + 1023u) / 1024u, 64u), 1024, 0, S(stream)>>>((uint4 *)dst, (const uint4 *)src, n16);
    return (int)cudaGetLastError();
}

int rc_memcpy_peer_async(void *dst, int dst_device, const void *src, int src_device, size_t bytes,
                         void *stream)
{
    return (int)cudaMemcpyPeerAsync(dst, dst_device, src, src_device, bytes, S(stream));
}
int rc_memset_async(void *dst, int value, size_t bytes, void *stream)
{
    return (int)cudaMemsetAsync(dst, value, bytes, S(stream));
}

int rc_stream_create(void **stream)
{
    if (!stream) return RC_ERR_NULL_POINTER;
    cudaStream_t s;
    cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    *stream = (void *)s;
    return (int)e;
}
int rc_stream_destroy(void *stream) { return (int)cudaStreamDestroy(S(stream)); }
int rc_stream_synchronize(void *stream) { return (int)cudaStreamSynchronize(S(stream)); }
int rc_stream_wait_event(void *stream, void *event)
{
    return (int)cudaStreamWaitEvent(S(stream), (cudaEvent_t)event, 0);
}

int rc_event_create(void **event)
{
    if (!event) return RC_ERR_NULL_POINTER;
    cudaEvent_t ev;
    cudaError_t e = cudaEventCreate(&ev);
    *event = (void *)ev;
    return (int)e;
}
int rc_event_record(void *event, void *stream) { return (int)cudaEventRecord((cudaEvent_t)event, S(stream)); }
int rc_event_synchronize(void *event) { return (int)cudaEventSynchronize((cudaEvent_t)event); }
int rc_event_elapsed_time(float *ms, void *start, void *stop)
{
    return ms ? (int)cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop) : RC_ERR_NULL_POINTER;
}
int rc_event_destroy(void *event) { return (int)cudaEventDestroy((cudaEvent_t)event); }

int rc_stream_begin_capture(void *stream, int mode)
{
    return (int)cudaStreamBeginCapture(S(stream), (cudaStreamCaptureMode)mode);
}
int rc_stream_end_capture(void *stream, void **graph)
{
    if (!graph) return RC_ERR_NULL_POINTER;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(S(stream), &g);
    *graph = (void *)g;
    return (int)e;
}
int rc_graph_instantiate(void **graph_exec, void *graph)
{
    if (!graph_exec) return RC_ERR_NULL_POINTER;
    cudaGraphExec_t ge = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ge, (cudaGraph_t)graph, 0);
    *graph_exec = (void *)ge;
    return (int)e;
}
int rc_graph_launch(void *graph_exec, void *stream)
{
    return (int)cudaGraphLaunch((cudaGraphExec_t)graph_exec, S(stream));
}
int rc_graph_destroy(void *graph) { return (int)cudaGraphDestroy((cudaGraph_t)graph); }
int rc_graph_exec_destroy(void *graph_exec) { return (int)cudaGraphExecDestroy((cudaGraphExec_t)graph_exec); }


} // extern "C"

namespace rc {
void matvec_set_tuning(int ks, int grid_mult, int no_pdl);
} // namespace rc
extern "C" void rc_tune_matvec(int ks, int grid_mult, int no_pdl) { rc::matvec_set_tuning(ks, grid_mult, no_pdl); }
extern "C" void rc_tune_mmq(int force_dp4a, int kind)
{
    rc::mmq_force_dp4a(force_dp4a);
    rc::mmq_set_kind(kind);
}
namespace rc { int mmq_deq_read_trace(void *out, size_t bytes); }
extern "C" int rc_debug_read_trace(void *out, size_t bytes) { return rc::mmq_deq_read_trace(out, bytes); }
extern "C" int rc_debug_read_prof(void *out, size_t bytes) { return rc::mmq_x_read_prof(out, bytes); }
extern "C" int rc_debug_read_ffn_trace(void *out, size_t bytes) { return rc::ffn_read_trace(out, bytes); }
namespace {
int device_status(unsigned int *status, bool clear)
{
    unsigned int g = 0;
    int rc = rc::mmq_device_error(status, clear);
    if (rc) return rc;
    rc = rc::mmq_x_device_error(&g, clear);
    *status |= (g & 0xFu) << 12;
    if (rc) return rc;
    rc = rc::gather_device_error(&g, clear);
    *status |= (g & 0xFu) << 16;
    if (rc) return rc;
    rc = rc::ffn_device_error(&g, clear);
    *status |= (g & 0xFu) << 20;
    if (rc) return rc;
    rc = rc::mmq_deq_device_error(&g, clear);
    *status |= (g & 0xFFu) << 24;
    return rc;
}
} // namespace
extern "C" int rc_device_status(unsigned int *status)
{
    if (!status) return RC_ERR_NULL_POINTER;
    return device_status(status, false);
}
extern "C" int rc_device_status_clear(unsigned int *status)
{
    unsigned int s = 0;
    const int rc = device_status(&s, true);
    if (status) *status = s;
    return rc;
}
