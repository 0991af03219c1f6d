// The small kernels around the grouped expert GEMMs of a MoE layer: router top-k, the fused
// gated activation + BlockQ8 quantizer between the two GEMMs, and the weighted combine of the
// routed experts' outputs.
//   moe_topk      kernels/moe_topk.cpp:17-107      softmax, n_used largest, renormalised
//   moe_act_q8    kernels/moe_geglu_q8.cpp:34-66   act(gate) * up -> BlockQ8 (GeGLU or SwiGLU,
//                                                  kernels/swiglu.cpp:11-21)
//   moe_combine   kernels/moe_combine.cpp:16-37    out = sum_j w_j * s[id_j] * expert_out_j
// All three are latency-bound and follow the PDL protocol of the chain (rc_common.cuh).
#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {
namespace {

// One warp per token; lane l holds experts l, l+32, ...  Ties go to the lowest expert index (the
// reference's tree reduction leaves the winner of an exact tie to its thread layout).
template <int kTopkMaxPerLane> // 32 * kTopkMaxPerLane >= n_expert
__global__ void __launch_bounds__(128) moe_topk_kernel(const float *__restrict__ logits, uint32_t n_tok,
                                                        uint32_t n_expert, uint32_t n_used,
                                                        int32_t *__restrict__ out_ids, float *__restrict__ out_w)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (tok >= n_tok) return;
    logits += (size_t)tok * n_expert;
    float p[kTopkMaxPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < kTopkMaxPerLane; k++) {
        const uint32_t e = k * 32u + lane;
        float v = e < n_expert ? logits[e] : -INFINITY;
        if (isnan(v)) v = -INFINITY; // a NaN logit can never win (kernels/moe_topk.cpp:37-49)
        p[k] = v;
        m = fmaxf(m, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < kTopkMaxPerLane; k++) {
        const uint32_t e = k * 32u + lane;
        p[k] = e < n_expert ? expf(p[k] - m) : 0.0f;
        sum += p[k];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
    for (int k = 0; k < kTopkMaxPerLane; k++) {
        const uint32_t e = k * 32u + lane;
        p[k] = e < n_expert ? p[k] * inv : -1.0f;
    }
    float wsum = 0.0f, mine = 0.0f; // lane j keeps the j-th chosen probability
    for (uint32_t r = 0; r < n_used; r++) {
        float bv = -1.0f;
        uint32_t bi = 0xFFFFFFFFu;
#pragma unroll
        for (int k = 0; k < kTopkMaxPerLane; k++) {
            const uint32_t e = k * 32u + lane;
            if (p[k] > bv) { bv = p[k]; bi = e; } // ascending e within the lane: first maximum wins
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
            const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        // no probability of the row is a number (all logits NaN): the reference's scan leaves its index at 0
        // (kernels/moe_topk.cpp: `float bv = -1.0f; int bi = 0;`)
        if (bi == 0xFFFFFFFFu) bi = 0u;
        if (lane == 0) out_ids[(size_t)tok * n_used + r] = (int32_t)bi;
        if ((r & 31u) == lane) mine = bv; // n_used <= 32 (checked on the host)
        wsum += bv;
#pragma unroll
        for (int k = 0; k < kTopkMaxPerLane; k++)
            if ((uint32_t)(k * 32) + lane == bi) p[k] = -1.0f; // exclude from later rounds
    }
    if (wsum < 6.103515625e-5f) wsum = 6.103515625e-5f;
    if (lane < n_used) out_w[(size_t)tok * n_used + lane] = __fdiv_rn(mine, wsum);
}

__device__ __forceinline__ float gelu_tanh(float x)
{
    const float k = 0.7978845608028654f; // sqrt(2/pi)
    const float c = x + 0.044715f * x * x * x;
    return 0.5f * x * (1.0f + tanhf(k * c));
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }

// gu [n_slot][2*ff] (gate then up) -> BlockQ8 [n_slot][ff/32]; one warp per 32 values, the
// quantizer of quantize_q8_kernel (same butterfly order, IEEE divide).
template <int ACT>
__global__ void __launch_bounds__(256) moe_act_q8_kernel(const float *__restrict__ gu, uint8_t *__restrict__ out, uint32_t ff)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t n_sub = ff >> 5, lane = threadIdx.x & 31u;
    const uint32_t sb = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (sb >= n_sub) return;
    const size_t slot = blockIdx.y;
    const float *g = gu + slot * 2u * ff;
    const float gate = g[sb * 32u + lane], up = g[ff + sb * 32u + lane];
    const float v = __fmul_rn(ACT == 0 ? gelu_tanh(gate) : silu(gate), up);
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
    uint32_t *dst = reinterpret_cast<uint32_t *>(out + (slot * n_sub + sb) * RC_BLOCKQ8_BYTES);
    if (lane == 0) dst[0] = __float_as_uint(d);
    else if (lane == 1) dst[1] = __float_as_uint(sum);
    else if (lane < 10) dst[lane] = word;
}

// experts [n_tok][n_used][hidden]; accumulation in slot order with one fused multiply-add per slot.
__global__ void __launch_bounds__(256) moe_combine_kernel(const float *__restrict__ experts, const int32_t *__restrict__ ids,
                                                           const float *__restrict__ weights,
                                                           const float *__restrict__ expert_scale, float *__restrict__ out,
                                                           uint32_t hidden, uint32_t n_used)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= hidden) return;
    const size_t tok = blockIdx.y;
    experts += tok * n_used * hidden;
    ids += tok * n_used;
    weights += tok * n_used;
    float acc = 0.0f;
    for (uint32_t j = 0; j < n_used; j++) {
        if (ids[j] < 0) continue; // a dropped slot (no expert row was ever written for it) adds nothing
        const float s = expert_scale ? __fmul_rn(weights[j], expert_scale[ids[j]]) : weights[j];
        acc = __fmaf_rn(s, experts[(size_t)j * hidden + i], acc);
    }
    out[tok * hidden + i] = acc;
}

} // namespace

int launch_moe_topk(cudaStream_t s, const float *logits, uint32_t n_tok, uint32_t n_expert, uint32_t n_used,
                    int32_t *ids, float *weights)
{
    const dim3 grid((n_tok + 3u) / 4u), block(128);
    if (n_expert <= 128) return (int)launch_pdl(moe_topk_kernel<4>, grid, block, 0, s, logits, n_tok, n_expert, n_used, ids, weights);
    if (n_expert <= 256) return (int)launch_pdl(moe_topk_kernel<8>, grid, block, 0, s, logits, n_tok, n_expert, n_used, ids, weights);
    return (int)launch_pdl(moe_topk_kernel<32>, grid, block, 0, s, logits, n_tok, n_expert, n_used, ids, weights);
}

int launch_moe_act_q8(cudaStream_t s, const float *gu, void *out, uint32_t ff, uint32_t n_slot, int act)
{
    const uint32_t gx = ((ff >> 5) + 7u) / 8u;
    for (uint32_t s0 = 0; s0 < n_slot; s0 += 65535u) {
        const uint32_t ns = min(65535u, n_slot - s0);
        const float *gp = gu + (size_t)s0 * 2u * ff;
        uint8_t *op = (uint8_t *)out + (size_t)s0 * (ff >> 5) * RC_BLOCKQ8_BYTES;
        cudaError_t e = act == 0 ? launch_pdl(moe_act_q8_kernel<0>, dim3(gx, ns), dim3(256), 0, s, gp, op, ff)
                                 : launch_pdl(moe_act_q8_kernel<1>, dim3(gx, ns), dim3(256), 0, s, gp, op, ff);
        if (e != cudaSuccess) return (int)e;
    }
    return RC_OK;
}

int launch_moe_combine(cudaStream_t s, const float *experts, const int32_t *ids, const float *weights,
                       const float *expert_scale, float *out, uint32_t hidden, uint32_t n_used, uint32_t n_tok)
{
    for (uint32_t t0 = 0; t0 < n_tok; t0 += 65535u) {
        const uint32_t nt = min(65535u, n_tok - t0);
        cudaError_t e = launch_pdl(moe_combine_kernel, dim3((hidden + 255u) / 256u, nt), dim3(256), 0, s,
                                   experts + (size_t)t0 * n_used * hidden, ids + (size_t)t0 * n_used,
                                   weights + (size_t)t0 * n_used, expert_scale, out + (size_t)t0 * hidden, hidden, n_used);
        if (e != cudaSuccess) return (int)e;
    }
    return RC_OK;
}

} // namespace rc
