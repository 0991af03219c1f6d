// Fused producers of BlockQ8 activations: the decode path quantizes each activation once, in the
// kernel that makes it, instead of writing f32 and launching quantize_q8 behind it.
//   rmsnorm_q8       kernels/rmsnorm_q8.cpp:38-103        y = x * rsqrt(mean(x^2) + eps) * w -> BlockQ8
//   add_rmsnorm_q8   kernels/qwen35_fused.cpp:66-118      hidden += add, then the same (also writes y)
//   swiglu_q8        kernels/qwen35_fused.cpp:123-138     silu(gate) * up -> f32 and BlockQ8
//   sigmoid_mul_q8   kernels/qwen35_fused.cpp:139-152     x *= sigmoid(gate) -> f32 (in place) and BlockQ8
//   rmsnorm_gated_q8 kernels/qwen35_fused.cpp:204-224     per head: rmsnorm(x) * w * silu(z) -> f32 and BlockQ8
// The quantizer is quantize_q8_kernel's (same butterfly order, IEEE divides).  The sum of squares is
// reduced in one fixed order, restated by the oracle: thread t of 1024 adds the squares of elements
// t, t + 1024, ... in turn; a warp reduces by xor-butterfly 16, 8, 4, 2, 1; the 32 warp sums are added
// in warp order; rrms = 1 / sqrt(total / n + eps) with IEEE divide and square root.
#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {
namespace {

constexpr int kNormThreads = 1024;

__device__ __forceinline__ void q8_store_block(uint8_t *rec, uint32_t lane, float v)
{
    float amax = fabsf(v), sum = v;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        sum = __fadd_rn(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, o));
    }
    const float d = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    int q = __float2int_rn(__fmul_rn(v, inv));
    q = max(-127, min(127, q));
    uint32_t b = (uint32_t)(q & 0xFF) << (8 * (lane & 3u));
    b |= __shfl_xor_sync(0xFFFFFFFFu, b, 1);
    b |= __shfl_xor_sync(0xFFFFFFFFu, b, 2);
    const uint32_t word = __shfl_sync(0xFFFFFFFFu, b, ((lane >= 2u ? lane - 2u : 0u) & 7u) * 4u);
    uint32_t *dst = reinterpret_cast<uint32_t *>(rec);
    if (lane == 0) dst[0] = __float_as_uint(d);
    else if (lane == 1) dst[1] = __float_as_uint(sum);
    else if (lane < 10) dst[lane] = word;
}

// One CTA per vector.  hidden_io: when `add` is given the sum is written back there; y (optional)
// receives the normalised f32 values.
__global__ void __launch_bounds__(kNormThreads) rmsnorm_q8_kernel(const float *__restrict__ x, const float *__restrict__ add,
                                                                    const float *__restrict__ w, float *__restrict__ hidden_io,
                                                                    float *__restrict__ y, uint8_t *__restrict__ out, uint32_t n,
                                                                    float eps)
{
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_warp[32];
    __shared__ float s_rrms;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, n_sub = n >> 5;
    const size_t vec = blockIdx.x;
    x += vec * n;
    if (add) add += vec * n;
    if (hidden_io) hidden_io += vec * n;
    if (y) y += vec * n;
    out += vec * n_sub * RC_BLOCKQ8_BYTES;
    float part = 0.0f;
    for (uint32_t i = tid; i < n; i += kNormThreads) {
        const float v = add ? __fadd_rn(x[i], add[i]) : x[i];
        part = __fadd_rn(part, __fmul_rn(v, v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xFFFFFFFFu, part, o));
    if (lane == 0) s_warp[warp] = part;
    __syncthreads();
    if (tid == 0) {
        float tot = s_warp[0];
        for (int k = 1; k < 32; k++) tot = __fadd_rn(tot, s_warp[k]);
        s_rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)n), eps)));
    }
    __syncthreads();
    const float rrms = s_rrms;
    for (uint32_t sb = warp; sb < n_sub; sb += kNormThreads / 32) {
        const uint32_t i = sb * 32u + lane;
        const float xv = add ? __fadd_rn(x[i], add[i]) : x[i];
        if (add && hidden_io) hidden_io[i] = xv;
        const float v = __fmul_rn(__fmul_rn(xv, rrms), w[i]);
        if (y) y[i] = v;
        q8_store_block(out + (size_t)sb * RC_BLOCKQ8_BYTES, lane, v);
    }
}

__global__ void __launch_bounds__(256) swiglu_q8_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                         float *__restrict__ out, uint8_t *__restrict__ q8, uint32_t n)
{
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return; // n is a multiple of 32: whole warps leave together
    const float g = gate[i];
    const float v = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), up[i]);
    if (out) out[i] = v;
    q8_store_block(q8 + (i >> 5) * RC_BLOCKQ8_BYTES, threadIdx.x & 31u, v);
}

__global__ void __launch_bounds__(256) sigmoid_mul_q8_kernel(float *__restrict__ x, const float *__restrict__ gate,
                                                              uint8_t *__restrict__ q8, uint32_t n)
{
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = __fdiv_rn(x[i], __fadd_rn(1.0f, expf(-gate[i])));
    x[i] = v;
    q8_store_block(q8 + (i >> 5) * RC_BLOCKQ8_BYTES, threadIdx.x & 31u, v);
}

// One CTA of head_dim threads per head (head_dim a multiple of 32, at most 1024).  The head's sum of
// squares: xor-butterfly per warp, the warp sums added in warp order.
__global__ void __launch_bounds__(1024) rmsnorm_gated_q8_kernel(const float *__restrict__ x, const float *__restrict__ z,
                                                                  const float *__restrict__ w, float *__restrict__ y,
                                                                  uint8_t *__restrict__ q8, uint32_t head_dim, float eps)
{
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_warp[32];
    __shared__ float s_rrms;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, n_warps = head_dim >> 5;
    const size_t i = (size_t)blockIdx.x * head_dim + tid;
    const float xv = x[i];
    float part = __fmul_rn(xv, xv);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xFFFFFFFFu, part, o));
    if (lane == 0) s_warp[warp] = part;
    __syncthreads();
    if (tid == 0) {
        float tot = s_warp[0];
        for (uint32_t k = 1; k < n_warps; k++) tot = __fadd_rn(tot, s_warp[k]);
        s_rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)head_dim), eps)));
    }
    __syncthreads();
    const float zg = z[i];
    const float silu = __fdiv_rn(zg, __fadd_rn(1.0f, expf(-zg)));
    const float v = __fmul_rn(__fmul_rn(__fmul_rn(xv, s_rrms), w[tid]), silu);
    if (y) y[i] = v;
    q8_store_block(q8 + (i >> 5) * RC_BLOCKQ8_BYTES, lane, v);
}

} // namespace

int launch_sigmoid_mul_q8(cudaStream_t s, float *x, const float *gate, void *q8, size_t n)
{
    const size_t blocks = (n + 255) / 256;
    if (blocks > 0x7FFFFFFFull) return RC_ERR_BAD_SHAPE;
    return (int)launch_pdl(sigmoid_mul_q8_kernel, dim3((uint32_t)blocks), dim3(256), 0, s, x, gate, (uint8_t *)q8, (uint32_t)n);
}

int launch_rmsnorm_gated_q8(cudaStream_t s, const float *x, const float *z, const float *w, float *y, void *q8, uint32_t n_heads,
                            uint32_t head_dim, float eps)
{
    return (int)launch_pdl(rmsnorm_gated_q8_kernel, dim3(n_heads), dim3(head_dim), 0, s, x, z, w, y, (uint8_t *)q8, head_dim, eps);
}

int launch_rmsnorm_q8(cudaStream_t s, const float *x, const float *add, const float *w, float *hidden_io, float *y, void *out,
                      uint32_t n, uint32_t n_vec, float eps)
{
    return (int)launch_pdl(rmsnorm_q8_kernel, dim3(n_vec), dim3(kNormThreads), 0, s, x, add, w, hidden_io, y, (uint8_t *)out, n, eps);
}

int launch_swiglu_q8(cudaStream_t s, const float *gate, const float *up, float *out, void *q8, size_t n)
{
    const size_t blocks = (n + 255) / 256;
    if (blocks > 0x7FFFFFFFull) return RC_ERR_BAD_SHAPE;
    return (int)launch_pdl(swiglu_q8_kernel, dim3((uint32_t)blocks), dim3(256), 0, s, gate, up, out, (uint8_t *)q8, (uint32_t)n);
}

} // namespace rc
