// On-device construction of the repacked-v2 weight planes from on-disk GGUF blocks.
// Byte-for-byte the result of src/quant/<fmt>.rs::repack_for_matvec of the reference
// (q4_0.rs:86-104, q8_0.rs:93-119, q4_k.rs:126-176, q5_k.rs:97-151, q6_k.rs:86-148,
// iq4_xs.rs:106-136), which the reference runs on the host while loading a model
// (src/runtime/qwen35.rs:251-331).  Here the raw blocks are uploaded and the planes are
// built at HBM speed: one thread per (row, padded sub-block), padding written as zeros.
#include <algorithm>

#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {
namespace {

__device__ __forceinline__ uint32_t rd16(const uint8_t *p)
{
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8);
}

// f32 -> binary16 as src/quant/half.rs:51-84 does it: round-to-nearest-even for normal
// results, TRUNCATION in the subnormal range, NaN -> 0x7E00-style quiet pattern.  The
// IQ4_XS scale plane is defined through this function, so it is reproduced bit for bit
// rather than replaced by the hardware conversion (which rounds subnormals).
__device__ __forceinline__ uint32_t f32_to_f16_ref(float v)
{
    const uint32_t b = __float_as_uint(v);
    const uint32_t s = (b >> 16) & 0x8000u;
    const int e = (int)((b >> 23) & 0xFFu);
    const uint32_t m = b & 0x7FFFFFu;
    if (e == 255) return s | 0x7C00u | (m ? 0x200u : 0u);
    const int u = e - 127;
    if (u >= 16) return s | 0x7C00u;
    if (u < -24) return s;
    if (u < -14) return s | ((m | 0x800000u) >> (uint32_t)(-1 - u));
    uint32_t out = s | ((uint32_t)(u + 15) << 10) | (m >> 13);
    if (((m >> 12) & 1u) && ((m & 0xFFFu) || (out & 1u))) out += 1u;
    return out & 0xFFFFu;
}

// 6-bit (scale, min) pair j of a K-quant block (src/quant/q4_k.rs:40-48).
__device__ __forceinline__ void k4_pair(const uint8_t *q, int j, uint32_t &sc, uint32_t &mn)
{
    if (j < 4) {
        sc = q[j] & 63u;
        mn = q[j + 4] & 63u;
    } else {
        sc = (q[j + 4] & 15u) | ((uint32_t)(q[j - 4] >> 6) << 4);
        mn = (uint32_t)(q[j + 4] >> 4) | ((uint32_t)(q[j] >> 6) << 4);
    }
}

// weight index of byte c of dp4a group g inside a 32-weight sub-block
__device__ __forceinline__ int group_weight(int g, int c) { return (g & 1) * 16 + (g >> 1) * 4 + c; }

__device__ __forceinline__ void store16(uint8_t *dst, const uint8_t v[16])
{
    uint4 o;
    o.x = v[0] | (v[1] << 8) | (v[2] << 16) | ((uint32_t)v[3] << 24);
    o.y = v[4] | (v[5] << 8) | (v[6] << 16) | ((uint32_t)v[7] << 24);
    o.z = v[8] | (v[9] << 8) | (v[10] << 16) | ((uint32_t)v[11] << 24);
    o.w = v[12] | (v[13] << 8) | (v[14] << 16) | ((uint32_t)v[15] << 24);
    *reinterpret_cast<uint4 *>(dst) = o;
}

template <int FMT>
__global__ void __launch_bounds__(256)
repack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ out, uint32_t in_dim,
              uint32_t out_dim)
{
    constexpr int OUT = FMT == SRC_Q3_K ? (int)Q6_K : FMT == SRC_BF16 ? (int)Q8_0 : FMT == SRC_IQ4_NL ? (int)IQ4_XS : FMT; // planes written
    const uint32_t n_sub = in_dim >> 5, nsp = nsp_of(n_sub), n_super = n_sub >> 3;
    const size_t total = (size_t)out_dim * nsp;
    const size_t q = total;
    uint8_t *nib = out;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / nsp), sb = (uint32_t)(i % nsp);
        uint8_t v[16];
        if (sb >= n_sub) { // the anti-aliasing pad sub-block: all planes zero
#pragma unroll
            for (int k = 0; k < 16; k++) v[k] = 0;
            store16(nib + i * 16, v);
            if (OUT == Q8_0) store16(out + q * 16 + i * 16, v);
            if (OUT == Q5_K || OUT == Q5_1) *reinterpret_cast<uint32_t *>(out + q * 16 + i * 4) = 0;
            if (OUT == Q5_1) { // d | m word
                *reinterpret_cast<uint32_t *>(out + q * 20 + i * 4) = 0;
                continue;
            }
            if (OUT == Q6_K) *reinterpret_cast<uint2 *>(out + q * 16 + i * 8) = make_uint2(0, 0);
            const size_t sc_off = OUT == Q8_0 ? q * 32 : OUT == Q5_K ? q * 20 : OUT == Q6_K ? q * 24 : q * 16;
            *reinterpret_cast<uint16_t *>(out + sc_off + i * 2) = 0;
            continue;
        }
        if (FMT == Q4_0 || FMT == SRC_IQ4_NL) { // IQ4_NL: the same block shape and byte order; d is the sub-block scale as-is (src/quant/iq4_nl.rs:51-73)
            const uint8_t *b = src + ((size_t)row * n_sub + sb) * 18;
#pragma unroll
            for (int k = 0; k < 16; k++) v[k] = b[2 + k];
            store16(nib + i * 16, v);
            *reinterpret_cast<uint16_t *>(out + q * 16 + i * 2) = (uint16_t)rd16(b);
        } else if (FMT == Q5_1) {
            // src/quant/q5_1.rs:62-100: nibbles verbatim (already weight k low / k+16 high); 5th bits
            // regrouped so that bit 4g+b belongs to dp4a group g lane b (group 2j = weights 4j.., group
            // 2j+1 = weights 16+4j..); d and m kept as raw fp16
            const uint8_t *b = src + ((size_t)row * n_sub + sb) * 24;
#pragma unroll
            for (int k = 0; k < 16; k++) v[k] = b[8 + k];
            store16(nib + i * 16, v);
            const uint32_t qh = rd16(b + 4) | (rd16(b + 6) << 16);
            uint32_t packed = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                packed |= ((qh >> (4 * j)) & 0xFu) << (8 * j);
                packed |= ((qh >> (16 + 4 * j)) & 0xFu) << (8 * j + 4);
            }
            *reinterpret_cast<uint32_t *>(out + q * 16 + i * 4) = packed;
            *reinterpret_cast<uint32_t *>(out + q * 20 + i * 4) = rd16(b) | (rd16(b + 2) << 16);
        } else if (FMT == SRC_BF16) {
            // requantization to Q8_0 (src/quant/q8_0.rs:45-61): d = amax / 127 (kept as f16),
            // q = round-half-away(v * (1 / d)) clamped to +-127
            const uint8_t *b = src + ((size_t)row * n_sub + sb) * 64;
            float f[32], amax = 0.0f;
#pragma unroll
            for (int k = 0; k < 32; k++) {
                f[k] = __uint_as_float(rd16(b + 2 * k) << 16);
                amax = fmaxf(amax, fabsf(f[k]));
            }
            const float d = __fdiv_rn(amax, 127.0f);
            const float inv = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
#pragma unroll
            for (int h = 0; h < 2; h++) {
#pragma unroll
                for (int k = 0; k < 16; k++) {
                    float r = roundf(__fmul_rn(f[16 * h + k], inv));
                    r = r > 127.0f ? 127.0f : r < -127.0f ? -127.0f : r;
                    v[k] = (uint8_t)(int8_t)(r != r ? 0 : (int)r);
                }
                store16(h ? out + q * 16 + i * 16 : nib + i * 16, v);
            }
            *reinterpret_cast<uint16_t *>(out + q * 32 + i * 2) = (uint16_t)f32_to_f16_ref(d);
        } else if (FMT == SRC_Q3_K) {
            // exact relabel onto Q6_K (src/quant/q3_k.rs:92-121): q6 = q3 + 28, sc6 = sc3 - 32, same d.
            // Sub-block sb of the row = weights 32*s .. 32*s+31 of block blk: chunk c = s >> 2, level j = s & 3.
            const uint32_t blk = sb >> 3, s = sb & 7u, c = s >> 2, j = s & 3u;
            const uint8_t *b = src + ((size_t)row * n_super + blk) * 110;
            uint32_t q6[32];
#pragma unroll
            for (int l = 0; l < 32; l++) {
                const uint32_t lo = ((uint32_t)b[32 + 32 * c + l] >> (2 * j)) & 3u;
                const uint32_t hi = ((uint32_t)b[l] >> (4 * c + j)) & 1u;
                q6[l] = (lo | (hi << 2)) + 28u;
            }
#pragma unroll
            for (int k = 0; k < 16; k++) v[k] = (uint8_t)((q6[k] & 15u) | ((q6[k + 16] & 15u) << 4));
            store16(nib + i * 16, v);
            uint32_t h[2] = {0, 0};
#pragma unroll
            for (int g = 0; g < 8; g++)
#pragma unroll
                for (int cc = 0; cc < 4; cc++) h[g >> 2] |= (q6[group_weight(g, cc)] >> 4) << (8 * (g & 3) + 2 * cc);
            *reinterpret_cast<uint2 *>(out + q * 16 + i * 8) = make_uint2(h[0], h[1]);
            uint32_t scw = 0;
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const uint32_t si = 2u * s + u, jj = si & 3u, grp = si >> 2;
                const uint32_t low = grp < 2 ? (b[96 + grp * 4 + jj] & 15u) : ((b[96 + (grp - 2) * 4 + jj] >> 4) & 15u);
                const uint32_t high = ((uint32_t)b[104 + jj] >> (2 * grp)) & 3u;
                scw |= ((uint32_t)(uint8_t)(int8_t)((int)(low | (high << 4)) - 32)) << (8 * u);
            }
            *reinterpret_cast<uint16_t *>(out + q * 24 + i * 2) = (uint16_t)scw;
            if (s == 0)
                *reinterpret_cast<uint16_t *>(out + q * 26 + ((size_t)row * n_super + blk) * 2) = (uint16_t)rd16(b + 108);
        } else if (FMT == Q8_0) {
            const uint8_t *b = src + ((size_t)row * n_sub + sb) * 34;
#pragma unroll
            for (int k = 0; k < 16; k++) v[k] = b[2 + k];
            store16(nib + i * 16, v);
#pragma unroll
            for (int k = 0; k < 16; k++) v[k] = b[18 + k];
            store16(out + q * 16 + i * 16, v);
            *reinterpret_cast<uint16_t *>(out + q * 32 + i * 2) = (uint16_t)rd16(b);
        } else if (FMT == Q4_K || FMT == Q5_K) {
            const uint32_t blk = sb >> 3, s = sb & 7u;
            const uint32_t bb = FMT == Q5_K ? 176u : 144u;
            const uint8_t *b = src + ((size_t)row * n_super + blk) * bb;
            const uint8_t *qs = b + (FMT == Q5_K ? 48 : 16) + (s >> 1) * 32;
            // sub-block s takes the low (even s) or high (odd s) nibbles of its 32 bytes;
            // output byte k = weight k | weight k+16 << 4
#pragma unroll
            for (int k = 0; k < 16; k++) {
                const uint32_t a = qs[k], c = qs[k + 16];
                v[k] = (s & 1u) ? (uint8_t)((a >> 4) | (c & 0xF0u)) : (uint8_t)((a & 15u) | ((c & 15u) << 4));
            }
            store16(nib + i * 16, v);
            size_t off = q * 16;
            if (FMT == Q5_K) {
                const uint8_t *qh = b + 16;
                uint32_t bits = 0;
#pragma unroll
                for (int g = 0; g < 8; g++)
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        bits |= (((uint32_t)qh[group_weight(g, c)] >> s) & 1u) << (4 * g + c);
                *reinterpret_cast<uint32_t *>(out + off + i * 4) = bits;
                off += q * 4;
            }
            uint32_t sc, mn;
            k4_pair(b + 4, (int)s, sc, mn);
            *reinterpret_cast<uint16_t *>(out + off + i * 2) = (uint16_t)(sc | (mn << 8));
            if (s == 0) {
                uint8_t *dd = out + off + q * 2 + ((size_t)row * n_super + blk) * 4;
                *reinterpret_cast<uint16_t *>(dd) = (uint16_t)rd16(b);
                *reinterpret_cast<uint16_t *>(dd + 2) = (uint16_t)rd16(b + 2);
            }
        } else if (FMT == Q6_K) {
            const uint32_t blk = sb >> 3, s = sb & 7u, half = s >> 2, quad = s & 3u;
            const uint8_t *b = src + ((size_t)row * n_super + blk) * 210;
            const uint8_t *ql = b + half * 64 + (quad & 1u) * 32;
            const uint8_t *qh = b + 128 + half * 32;
#pragma unroll
            for (int k = 0; k < 16; k++) {
                const uint32_t a = ql[k], c = ql[k + 16];
                v[k] = (quad & 2u) ? (uint8_t)((a >> 4) | (c & 0xF0u)) : (uint8_t)((a & 15u) | ((c & 15u) << 4));
            }
            store16(nib + i * 16, v);
            uint32_t h[2] = {0, 0};
#pragma unroll
            for (int g = 0; g < 8; g++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const uint32_t f = ((uint32_t)qh[group_weight(g, c)] >> (2 * quad)) & 3u;
                    h[g >> 2] |= f << (8 * (g & 3) + 2 * c);
                }
            *reinterpret_cast<uint2 *>(out + q * 16 + i * 8) = make_uint2(h[0], h[1]);
            const uint8_t *scp = b + 192 + half * 8 + quad * 2;
            *reinterpret_cast<uint16_t *>(out + q * 24 + i * 2) = (uint16_t)(scp[0] | (scp[1] << 8));
            if (s == 0)
                *reinterpret_cast<uint16_t *>(out + q * 26 + ((size_t)row * n_super + blk) * 2) =
                    (uint16_t)rd16(b + 208);
        } else { // IQ4_XS
            const uint32_t blk = sb >> 3, ib = sb & 7u;
            const uint8_t *b = src + ((size_t)row * n_super + blk) * 136;
#pragma unroll
            for (int k = 0; k < 16; k++) v[k] = b[8 + 16 * ib + k];
            store16(nib + i * 16, v);
            const uint32_t lo = ((uint32_t)b[4 + (ib >> 1)] >> (4 * (ib & 1u))) & 15u;
            const uint32_t hi = (rd16(b + 2) >> (2 * ib)) & 3u;
            const int ls = (int)(lo | (hi << 4));
            const float d = f16_bits_to_f32(rd16(b));
            *reinterpret_cast<uint16_t *>(out + q * 16 + i * 2) =
                (uint16_t)f32_to_f16_ref(__fmul_rn(d, (float)(ls - 32)));
        }
    }
}

} // namespace

int launch_repack(cudaStream_t s, int type, const void *blocks, size_t in_dim, size_t out_dim,
                  void *out)
{
    const size_t total = out_dim * nsp_of((uint32_t)(in_dim >> 5));
    if (total == 0) return RC_OK;
    const uint32_t grid = (uint32_t)std::min<size_t>((total + 255) / 256, (size_t)sm_count() * 32);
    const uint8_t *src = (const uint8_t *)blocks;
    uint8_t *dst = (uint8_t *)out;
    switch (type) {
    case Q4_0: repack_kernel<Q4_0><<<grid, 256, 0, s>>>(src, dst, (uint32_t)in_dim, (uint32_t)out_dim); break;
    case Q5_1: repack_kernel<Q5_1><<<grid, 256, 0, s>>>(src, dst, (uint32_t)in_dim, (uint32_t)out_dim); break;
    case Q8_0: repack_kernel<Q8_0><<<grid, 256, 0, s>>>(src, dst, (uint32_t)in_dim, (uint32_t)out_dim); break;
    case Q4_K: repack_kernel<Q4_K><<<grid, 256, 0, s>>>(src, dst, (uint32_t)in_dim, (uint32_t)out_dim); break;
    case Q5_K: repack_kernel<Q5_K><<<grid, 256, 0, s>>>(src, dst, (uint32_t)in_dim, (uint32_t)out_dim); break;
    case Q6_K: repack_kernel<Q6_K><<<grid, 256, 0, s>>>(src, dst, (uint32_t)in_dim, (uint32_t)out_dim); break;
    case IQ4_XS: repack_kernel<IQ4_XS><<<grid, 256, 0, s>>>(src, dst, (uint32_t)in_dim, (uint32_t)out_dim); break;
    case SRC_Q3_K: repack_kernel<SRC_Q3_K><<<grid, 256, 0, s>>>(src, dst, (uint32_t)in_dim, (uint32_t)out_dim); break;
    case SRC_IQ4_NL: repack_kernel<SRC_IQ4_NL><<<grid, 256, 0, s>>>(src, dst, (uint32_t)in_dim, (uint32_t)out_dim); break;
    case SRC_BF16: repack_kernel<SRC_BF16><<<grid, 256, 0, s>>>(src, dst, (uint32_t)in_dim, (uint32_t)out_dim); break;
    default: return RC_ERR_BAD_TYPE;
    }
    return (int)cudaGetLastError();
}

} // namespace rc
