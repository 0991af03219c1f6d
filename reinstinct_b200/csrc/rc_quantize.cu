// quantize_q8: f32 activations -> BlockQ8 {f32 d, f32 xsum, i8 qs[32]} per 32 values.
// Follows kernels/quantize_q8.cpp:23-54 of the reference with its approximate reciprocal
// replaced by the IEEE divide (as kernels/moe_geglu_q8.cpp:58 writes it), so the bytes are
// reproducible on any IEEE machine:
//   amax, xsum  xor-butterfly over the 32 lanes in the order 16,8,4,2,1
//   d   = amax > 0 ? amax / 127 : 1          inv = amax > 0 ? 127 / amax : 0
//   q   = clamp(rint(v * inv), -127, 127)    (round-half-even)
#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {

// One warp per sub-block, one value per lane.  The 40-byte block is written as ten 32-bit
// words by lanes 0..9 after the quants are packed four to a word with shuffles, so a warp
// issues one store instruction per block.
__global__ void __launch_bounds__(256) quantize_q8_kernel(const float *__restrict__ x,
                                                           uint8_t *__restrict__ out,
                                                           uint32_t in_dim)
{
    pdl_launch_dependents(); // a following matvec may start fetching its weights now
    pdl_wait();              // x comes from the preceding kernel
    const uint32_t n_sub = in_dim >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps_per_cta = blockDim.x >> 5;
    const size_t vec = blockIdx.y;
    x += vec * in_dim;
    out += vec * n_sub * RC_BLOCKQ8_BYTES;
    for (uint32_t sb = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); sb < n_sub;
         sb += gridDim.x * warps_per_cta) {
        const float v = x[(size_t)sb * 32 + lane];
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
        // Pack lanes 4k..4k+3 into one word held by every lane of the quad.
        uint32_t b = (uint32_t)(q & 0xFF) << (8 * (lane & 3u));
        b |= __shfl_xor_sync(0xFFFFFFFFu, b, 1);
        b |= __shfl_xor_sync(0xFFFFFFFFu, b, 2);
        // Lane l (2 <= l < 10) stores the word of quad l-2.
        const uint32_t word = __shfl_sync(0xFFFFFFFFu, b, ((lane >= 2u ? lane - 2u : 0u) & 7u) * 4u);
        uint32_t *dst = reinterpret_cast<uint32_t *>(out + (size_t)sb * RC_BLOCKQ8_BYTES);
        if (lane == 0) dst[0] = __float_as_uint(d);
        else if (lane == 1) dst[1] = __float_as_uint(sum);
        else if (lane < 10) dst[lane] = word;
    }
}

// The same quantizer writing the planar form the tensor-core GEMM takes through TMA instead of
// 40-byte records: qs int8 [n_vec][in_dim], then d f32 [in_dim/32][ld], then xsum f32
// [in_dim/32][ld], ld = n_vec rounded up to 4 (16-byte row pitch).  Same arithmetic, same values.
__global__ void __launch_bounds__(256) quantize_q8_planar_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                                  uint32_t in_dim, uint32_t n_vec)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t n_sub = in_dim >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps_per_cta = blockDim.x >> 5;
    const uint32_t vec = blockIdx.y;
    const uint32_t ld = (n_vec + 3u) & ~3u;
    uint32_t *qs = reinterpret_cast<uint32_t *>(out + (size_t)vec * in_dim);
    float *dT = reinterpret_cast<float *>(out + (size_t)n_vec * in_dim);
    float *sT = dT + (size_t)n_sub * ld;
    x += (size_t)vec * in_dim;
    for (uint32_t sb = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); sb < n_sub; sb += gridDim.x * warps_per_cta) {
        const float v = x[(size_t)sb * 32 + lane];
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
        if ((lane & 3u) == 0) qs[sb * 8 + (lane >> 2)] = b;
        if (lane == 0) {
            dT[(size_t)sb * ld + vec] = d;
            sT[(size_t)sb * ld + vec] = sum;
        }
    }
}

size_t quantize_planar_bytes(uint32_t in_dim, uint32_t n_vec)
{
    const size_t ld = ((size_t)n_vec + 3u) & ~(size_t)3u;
    return (size_t)n_vec * in_dim + 2u * (size_t)(in_dim >> 5) * ld * sizeof(float);
}

int launch_quantize_q8_planar(cudaStream_t s, const float *x, void *out, uint32_t in_dim, uint32_t n_vec)
{
    if (n_vec == 0) return RC_OK;
    if (n_vec > 65535u) return RC_ERR_TOO_MANY_ROWS;
    const uint32_t n_sub = in_dim >> 5;
    quantize_q8_planar_kernel<<<dim3((n_sub + 7u) / 8u, n_vec), 256, 0, s>>>(x, (uint8_t *)out, in_dim, n_vec);
    return (int)cudaGetLastError();
}

int launch_quantize_q8(cudaStream_t s, const float *x, void *xq, uint32_t in_dim, uint32_t n_vec)
{
    if (n_vec == 0) return RC_OK;
    const uint32_t n_sub = in_dim >> 5;
    const uint32_t gx = (n_sub + 7u) / 8u;
    // gridDim.y is limited to 65535: fold larger batches by looping on the host.
    for (uint32_t v0 = 0; v0 < n_vec; v0 += 65535u) {
        const uint32_t nv = min(65535u, n_vec - v0);
        const float *xp = x + (size_t)v0 * in_dim;
        uint8_t *op = (uint8_t *)xq + (size_t)v0 * n_sub * RC_BLOCKQ8_BYTES;
        if (matvec_pdl_enabled()) {
            cudaError_t e = launch_pdl(quantize_q8_kernel, dim3(gx, nv), dim3(256), 0, s, xp, op, in_dim);
            if (e != cudaSuccess) return (int)e;
        } else {
            quantize_q8_kernel<<<dim3(gx, nv), 256, 0, s>>>(xp, op, in_dim);
        }
    }
    return (int)cudaGetLastError();
}

} // namespace rc
