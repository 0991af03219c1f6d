/*
 * TEST INFRASTRUCTURE — CPU oracle for the quantized-weight hot path (see
 * ro_oracle.h for what may call it and how it is pinned).  Plain C, no SIMD
 * intrinsics, compiled with -ffp-contract=off so every f32 expression rounds
 * where it is written.
 */
#include "ro_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ f16 --- */

/* src/quant/half.rs:9-41.  Subnormals are renormalised by counting the shifts
 * needed to bring the leading one up to bit 10. */
float ro_f16_to_f32(uint16_t h)
{
    uint32_t s = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu;
    uint32_t m = h & 0x3FFu;
    uint32_t bits;
    if (e == 0) {
        if (m == 0) {
            bits = s;
        } else {
            int k = 0;
            while (!(m & 0x400u)) { m <<= 1; k++; }
            bits = s | ((uint32_t)(127 - 14 - k) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (e == 31) {
        bits = s | 0x7F800000u | (m << 13);
    } else {
        bits = s | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* src/quant/half.rs:51-84.  Round-to-nearest-even on normal results; results in
 * the binary16 subnormal range are TRUNCATED (no rounding), exactly as the
 * reference writes it (half.rs:70-74) — the IQ4_XS repack folds scales through
 * this function, so the truncation is part of that layout's definition. */
uint16_t ro_f32_to_f16(float v)
{
    uint32_t b;
    memcpy(&b, &v, 4);
    uint16_t s = (uint16_t)((b >> 16) & 0x8000u);
    int e = (int)((b >> 23) & 0xFFu);
    uint32_t m = b & 0x7FFFFFu;
    if (e == 255) return (uint16_t)(s | 0x7C00u | (m ? 0x200u : 0u));
    int u = e - 127;
    if (u >= 16) return (uint16_t)(s | 0x7C00u);
    if (u < -24) return s;
    if (u < -14) return (uint16_t)(s | (uint16_t)((m | 0x800000u) >> (unsigned)(-1 - u)));
    uint16_t out = (uint16_t)(s | (uint16_t)((u + 15) << 10) | (uint16_t)(m >> 13));
    uint32_t half_bit = (m >> 12) & 1u, rest = m & 0xFFFu;
    if (half_bit && (rest || (out & 1u))) out = (uint16_t)(out + 1u);
    return out;
}

/* src/quant/half.rs:44-47 */
float ro_bf16_to_f32(uint16_t h)
{
    uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static void wr16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }

/* ------------------------------------------------------------ constants --- */

size_t ro_block_bytes(int t)
{
    switch (t) {
    case RO_Q4_0: return 18;    /* src/quant/q4_0.rs:23 */
    case RO_Q5_1: return 24;    /* src/quant/q5_1.rs:27 */
    case RO_Q8_0: return 34;    /* src/quant/q8_0.rs:9 */
    case RO_Q4_K: return 144;   /* src/quant/q4_k.rs:18 */
    case RO_Q5_K: return 176;   /* src/quant/q5_k.rs:22 */
    case RO_Q6_K: return 210;   /* src/quant/q6_k.rs:18 */
    case RO_IQ4_XS: return 136; /* src/quant/iq4_xs.rs:24 */
    case RO_IQ3_S: return 110;  /* src/quant/iq3_s.rs:27 */
    default: return 0;
    }
}

size_t ro_block_weights(int t)
{
    switch (t) {
    case RO_Q4_0: case RO_Q8_0: case RO_Q5_1: return 32;
    case RO_Q4_K: case RO_Q5_K: case RO_Q6_K: case RO_IQ4_XS: case RO_IQ3_S: return 256;
    default: return 0;
    }
}

size_t ro_nsp(size_t in_dim)
{
    size_t n = in_dim / 32;
    return (n && (n & (n - 1)) == 0) ? n + 1 : n;
}

/* Bytes per padded sub-block and per 256-superblock of each repacked layout:
 * q4_0.rs:66-69, q8_0.rs:74-77, q4_k.rs:98-102, q5_k.rs:101-104,
 * q6_k.rs:90-93, iq4_xs.rs:85-88. */
static void plane_bytes(int t, size_t *per_sub, size_t *per_super)
{
    *per_sub = 0; *per_super = 0;
    switch (t) {
    case RO_Q4_0: case RO_IQ4_XS: case RO_IQ3_S: *per_sub = 18; break;
    case RO_Q8_0: *per_sub = 34; break;
    case RO_Q5_1: *per_sub = 24; break; /* src/quant/q5_1.rs:73-78 */
    case RO_Q4_K: *per_sub = 18; *per_super = 4; break;
    case RO_Q5_K: *per_sub = 22; *per_super = 4; break;
    case RO_Q6_K: *per_sub = 26; *per_super = 2; break;
    }
}

size_t ro_repacked_len(int t, size_t in_dim, size_t out_dim)
{
    size_t bw = ro_block_weights(t);
    if (!bw || in_dim == 0 || in_dim % bw) return 0;
    size_t ps, pp;
    plane_bytes(t, &ps, &pp);
    return out_dim * ro_nsp(in_dim) * ps + out_dim * (in_dim / 256) * pp;
}

/* 6-bit (scale, min) pair j of a K-quant block: src/quant/q4_k.rs:40-48. */
static void k4_scale_min(const uint8_t *q, int j, uint8_t *sc, uint8_t *mn)
{
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 15) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* src/quant/iq4_xs.rs:28-31 */
static const int8_t IQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10,
                                 1, 13, 25, 38, 53, 69, 89, 113};

/* 6-bit sub-scale ib of an IQ4_XS block: src/quant/iq4_xs.rs:56-58. */
static int iq4xs_ls(const uint8_t *blk, int ib)
{
    unsigned sh = rd16(blk + 2);
    unsigned lo = (blk[4 + ib / 2] >> (4 * (ib & 1))) & 15u;
    unsigned hi = (sh >> (2 * ib)) & 3u;
    return (int)(lo | (hi << 4));
}

/* -------------------------------------------------------------- dequant --- */

/* src/quant/q4_0.rs:36-53 */
static void deq_q4_0(const uint8_t *b, float *o)
{
    float d = ro_f16_to_f32(rd16(b));
    for (int k = 0; k < 16; k++) {
        o[k] = d * (float)((int)(b[2 + k] & 15) - 8);
        o[k + 16] = d * (float)((int)(b[2 + k] >> 4) - 8);
    }
}

/* src/quant/q5_1.rs:41-59 */
static void deq_q5_1(const uint8_t *b, float *o)
{
    float d = ro_f16_to_f32(rd16(b)), m = ro_f16_to_f32(rd16(b + 2));
    uint32_t qh = (uint32_t)b[4] | ((uint32_t)b[5] << 8) | ((uint32_t)b[6] << 16) | ((uint32_t)b[7] << 24);
    for (int k = 0; k < 16; k++) {
        uint32_t lo = (uint32_t)(b[8 + k] & 15) | (((qh >> k) & 1u) << 4);
        uint32_t hi = (uint32_t)(b[8 + k] >> 4) | (((qh >> (k + 16)) & 1u) << 4);
        o[k] = d * (float)lo + m;
        o[k + 16] = d * (float)hi + m;
    }
}

/* src/quant/q8_0.rs:24-38 */
static void deq_q8_0(const uint8_t *b, float *o)
{
    float d = ro_f16_to_f32(rd16(b));
    for (int k = 0; k < 32; k++) o[k] = d * (float)(int8_t)b[2 + k];
}

/* src/quant/q4_k.rs:50-84 (hi5 == NULL) and src/quant/q5_k.rs:47-86. */
static void deq_q45_k(const uint8_t *b, float *o, int is_q5)
{
    float d = ro_f16_to_f32(rd16(b)), dmin = ro_f16_to_f32(rd16(b + 2));
    const uint8_t *scales = b + 4;
    const uint8_t *qh = is_q5 ? b + 16 : NULL;
    const uint8_t *qs = b + (is_q5 ? 48 : 16);
    for (int pair = 0; pair < 4; pair++) {
        uint8_t sa, ma, sb, mb;
        k4_scale_min(scales, 2 * pair, &sa, &ma);
        k4_scale_min(scales, 2 * pair + 1, &sb, &mb);
        float d1 = d * (float)sa, m1 = dmin * (float)ma;
        float d2 = d * (float)sb, m2 = dmin * (float)mb;
        for (int l = 0; l < 32; l++) {
            int lo = qs[pair * 32 + l] & 15, hi = qs[pair * 32 + l] >> 4;
            if (qh) {
                if (qh[l] & (1u << (2 * pair))) lo += 16;
                if (qh[l] & (2u << (2 * pair))) hi += 16;
            }
            o[pair * 64 + l] = d1 * (float)lo - m1;
            o[pair * 64 + 32 + l] = d2 * (float)hi - m2;
        }
    }
}

/* src/quant/q6_k.rs:31-69: ql[128] qh[64] i8 scales[16] f16 d (at byte 208). */
static void deq_q6_k(const uint8_t *b, float *o)
{
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    float d = ro_f16_to_f32(rd16(b + 208));
    for (int half = 0; half < 2; half++) {
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            uint8_t h = qh[half * 32 + l];
            uint8_t a = ql[half * 64 + l], c = ql[half * 64 + 32 + l];
            int q[4] = {
                (int)((a & 15) | ((h & 3) << 4)) - 32,
                (int)((c & 15) | (((h >> 2) & 3) << 4)) - 32,
                (int)((a >> 4) | (((h >> 4) & 3) << 4)) - 32,
                (int)((c >> 4) | (((h >> 6) & 3) << 4)) - 32,
            };
            for (int g = 0; g < 4; g++)
                o[half * 128 + 32 * g + l] =
                    d * (float)sc[half * 8 + is + 2 * g] * (float)q[g];
        }
    }
}

/* src/quant/iq4_xs.rs:44-71 */
static void deq_iq4_xs(const uint8_t *b, float *o)
{
    float d = ro_f16_to_f32(rd16(b));
    for (int ib = 0; ib < 8; ib++) {
        float dl = d * (float)(iq4xs_ls(b, ib) - 32);
        const uint8_t *q = b + 8 + 16 * ib;
        for (int l = 0; l < 16; l++) {
            o[32 * ib + l] = dl * (float)IQ4NL[q[l] & 15];
            o[32 * ib + 16 + l] = dl * (float)IQ4NL[q[l] >> 4];
        }
    }
}

int ro_dequantize(int t, const uint8_t *blocks, float *out, size_t n_weights)
{
    size_t bw = ro_block_weights(t), bb = ro_block_bytes(t);
    if (!bw || n_weights % bw) return -1;
    for (size_t i = 0; i < n_weights / bw; i++) {
        const uint8_t *b = blocks + i * bb;
        float *o = out + i * bw;
        switch (t) {
        case RO_Q4_0: deq_q4_0(b, o); break;
        case RO_Q8_0: deq_q8_0(b, o); break;
        case RO_Q5_1: deq_q5_1(b, o); break;
        case RO_Q4_K: deq_q45_k(b, o, 0); break;
        case RO_Q5_K: deq_q45_k(b, o, 1); break;
        case RO_Q6_K: deq_q6_k(b, o); break;
        case RO_IQ4_XS: deq_iq4_xs(b, o); break;
        default: return -1; /* IQ3_S: planes only, no on-disk decode */
        }
    }
    return 0;
}

/* --------------------------------------------------------------- repack --- */

/* 32 unsigned 4-bit values in weight order -> 16 bytes in "dp4a order":
 * byte k carries weight k (low nibble) and weight k+16 (high nibble), so 32-bit
 * word j pairs with activation bytes 4j..4j+3 and 16+4j..16+4j+3
 * (src/quant/q4_k.rs:158-165). */
static void pack_nibbles(const uint8_t w[32], uint8_t *dst)
{
    for (int k = 0; k < 16; k++) dst[k] = (uint8_t)(w[k] | (w[k + 16] << 4));
}

/* "dp4a group" g of a sub-block: even g = weights 2g.., odd g = 16 + ...
 * group 2j holds weights 4j..4j+3, group 2j+1 weights 16+4j..16+4j+3
 * (src/quant/q5_k.rs:134-137, src/quant/q6_k.rs:128-133). */
static int group_weight(int g, int b) { return (g & 1) * 16 + (g >> 1) * 4 + b; }

/* src/quant/q4_0.rs:86-104 */
static void repack_q4_0(const uint8_t *src, size_t in_dim, size_t out_dim, uint8_t *out)
{
    size_t nb = in_dim / 32, nsp = ro_nsp(in_dim), nib = out_dim * nsp * 16;
    for (size_t r = 0; r < out_dim; r++)
        for (size_t k = 0; k < nb; k++) {
            const uint8_t *b = src + (r * nb + k) * 18;
            memcpy(out + (r * nsp + k) * 16, b + 2, 16);
            memcpy(out + nib + (r * nsp + k) * 2, b, 2);
        }
}

/* src/quant/q5_1.rs:62-100: nibbles verbatim, the 5th bits regrouped to bit 4g+b = dp4a group g lane b,
 * then d | m << 16 as raw fp16. */
static void repack_q5_1(const uint8_t *src, size_t in_dim, size_t out_dim, uint8_t *out)
{
    size_t nb = in_dim / 32, nsp = ro_nsp(in_dim), nib = out_dim * nsp * 16, qhl = out_dim * nsp * 4;
    for (size_t r = 0; r < out_dim; r++)
        for (size_t k = 0; k < nb; k++) {
            const uint8_t *b = src + (r * nb + k) * 24;
            size_t i = r * nsp + k;
            memcpy(out + i * 16, b + 8, 16);
            uint32_t qh = (uint32_t)b[4] | ((uint32_t)b[5] << 8) | ((uint32_t)b[6] << 16) | ((uint32_t)b[7] << 24);
            uint32_t bits = 0;
            for (int g = 0; g < 8; g++)
                for (int c = 0; c < 4; c++)
                    bits |= ((qh >> group_weight(g, c)) & 1u) << (4 * g + c);
            uint8_t *p = out + nib + i * 4;
            p[0] = (uint8_t)bits; p[1] = (uint8_t)(bits >> 8); p[2] = (uint8_t)(bits >> 16); p[3] = (uint8_t)(bits >> 24);
            memcpy(out + nib + qhl + i * 4, b, 4);
        }
}

/* src/quant/q8_0.rs:93-119 */
static void repack_q8_0(const uint8_t *src, size_t in_dim, size_t out_dim, uint8_t *out)
{
    size_t nb = in_dim / 32, nsp = ro_nsp(in_dim), plane = out_dim * nsp * 16;
    for (size_t r = 0; r < out_dim; r++)
        for (size_t k = 0; k < nb; k++) {
            const uint8_t *b = src + (r * nb + k) * 34;
            size_t i = r * nsp + k;
            memcpy(out + i * 16, b + 2, 16);
            memcpy(out + plane + i * 16, b + 18, 16);
            memcpy(out + 2 * plane + i * 2, b, 2);
        }
}

/* src/quant/q4_k.rs:126-176 and src/quant/q5_k.rs:97-151 */
static void repack_q45_k(const uint8_t *src, size_t in_dim, size_t out_dim, uint8_t *out,
                         int is_q5)
{
    size_t nblk = in_dim / 256, nsp = ro_nsp(in_dim), bb = is_q5 ? 176 : 144;
    size_t nib = out_dim * nsp * 16, qhl = is_q5 ? out_dim * nsp * 4 : 0;
    size_t sml = out_dim * nsp * 2;
    for (size_t r = 0; r < out_dim; r++)
        for (size_t k = 0; k < nblk; k++) {
            const uint8_t *b = src + (r * nblk + k) * bb;
            const uint8_t *qh = b + 16, *qs = b + (is_q5 ? 48 : 16);
            memcpy(out + nib + qhl + sml + (r * nblk + k) * 4, b, 4); /* d, dmin */
            for (int s = 0; s < 8; s++) {
                size_t i = r * nsp + k * 8 + (size_t)s;
                uint8_t w[32];
                for (int l = 0; l < 32; l++) {
                    uint8_t byte = qs[(s / 2) * 32 + l];
                    w[l] = (s & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 15);
                }
                pack_nibbles(w, out + i * 16);
                if (is_q5) {
                    uint32_t bits = 0;
                    for (int g = 0; g < 8; g++)
                        for (int c = 0; c < 4; c++)
                            bits |= (uint32_t)((qh[group_weight(g, c)] >> s) & 1u)
                                    << (4 * g + c);
                    uint8_t *p = out + nib + i * 4;
                    p[0] = (uint8_t)bits; p[1] = (uint8_t)(bits >> 8);
                    p[2] = (uint8_t)(bits >> 16); p[3] = (uint8_t)(bits >> 24);
                }
                uint8_t sc, mn;
                k4_scale_min(b + 4, s, &sc, &mn);
                out[nib + qhl + i * 2] = sc;
                out[nib + qhl + i * 2 + 1] = mn;
            }
        }
}

/* src/quant/q6_k.rs:86-148 */
static void repack_q6_k(const uint8_t *src, size_t in_dim, size_t out_dim, uint8_t *out)
{
    size_t nblk = in_dim / 256, nsp = ro_nsp(in_dim);
    size_t nib = out_dim * nsp * 16, h2l = out_dim * nsp * 8, sml = out_dim * nsp * 2;
    for (size_t r = 0; r < out_dim; r++)
        for (size_t k = 0; k < nblk; k++) {
            const uint8_t *b = src + (r * nblk + k) * 210;
            memcpy(out + nib + h2l + sml + (r * nblk + k) * 2, b + 208, 2);
            for (int s = 0; s < 8; s++) {
                size_t i = r * nsp + k * 8 + (size_t)s;
                int half = s / 4, quad = s % 4;
                uint8_t lo[32], hi[32];
                for (int l = 0; l < 32; l++) {
                    uint8_t q = b[half * 64 + (quad & 1) * 32 + l];
                    lo[l] = (quad & 2) ? (uint8_t)(q >> 4) : (uint8_t)(q & 15);
                    hi[l] = (uint8_t)((b[128 + half * 32 + l] >> (2 * quad)) & 3);
                }
                pack_nibbles(lo, out + i * 16);
                for (int g = 0; g < 8; g++) {
                    uint8_t v = 0;
                    for (int c = 0; c < 4; c++)
                        v |= (uint8_t)(hi[group_weight(g, c)] << (2 * c));
                    out[nib + i * 8 + (size_t)g] = v;
                }
                out[nib + h2l + i * 2] = b[192 + half * 8 + quad * 2];
                out[nib + h2l + i * 2 + 1] = b[192 + half * 8 + quad * 2 + 1];
            }
        }
}

/* src/quant/iq4_xs.rs:106-136 */
static void repack_iq4_xs(const uint8_t *src, size_t in_dim, size_t out_dim, uint8_t *out)
{
    size_t nblk = in_dim / 256, nsp = ro_nsp(in_dim), nib = out_dim * nsp * 16;
    for (size_t r = 0; r < out_dim; r++)
        for (size_t k = 0; k < nblk; k++) {
            const uint8_t *b = src + (r * nblk + k) * 136;
            float d = ro_f16_to_f32(rd16(b));
            for (int ib = 0; ib < 8; ib++) {
                size_t i = r * nsp + k * 8 + (size_t)ib;
                memcpy(out + i * 16, b + 8 + 16 * ib, 16);
                wr16(out + nib + i * 2, ro_f32_to_f16(d * (float)(iq4xs_ls(b, ib) - 32)));
            }
        }
}

int ro_repack(int t, const uint8_t *blocks, size_t in_dim, size_t out_dim, uint8_t *out)
{
    size_t len = ro_repacked_len(t, in_dim, out_dim);
    if (!len) return -1;
    memset(out, 0, len);
    switch (t) {
    case RO_Q4_0: repack_q4_0(blocks, in_dim, out_dim, out); break;
    case RO_Q8_0: repack_q8_0(blocks, in_dim, out_dim, out); break;
    case RO_Q5_1: repack_q5_1(blocks, in_dim, out_dim, out); break;
    case RO_Q4_K: repack_q45_k(blocks, in_dim, out_dim, out, 0); break;
    case RO_Q5_K: repack_q45_k(blocks, in_dim, out_dim, out, 1); break;
    case RO_Q6_K: repack_q6_k(blocks, in_dim, out_dim, out); break;
    case RO_IQ4_XS: repack_iq4_xs(blocks, in_dim, out_dim, out); break;
    default: return -1;
    }
    return 0;
}

/* ---------------------------------------------------------- quantize_q8 --- */

/* kernels/quantize_q8.cpp:23-54.  amax and the plain sum are reduced by the xor
 * butterfly 16,8,4,2,1 over the 32 lanes (lane 0's value is the one stored); the
 * gfx906 approximate reciprocal (quantize_q8.cpp:48) is pinned to the IEEE
 * divide 127/amax, as kernels/moe_geglu_q8.cpp:58 writes it. */
void ro_quantize_q8(const float *x, uint8_t *out, size_t in_dim, size_t n_vec)
{
    size_t n_sub = in_dim / 32;
    for (size_t v = 0; v < n_vec; v++)
        for (size_t s = 0; s < n_sub; s++) {
            const float *p = x + v * in_dim + s * 32;
            uint8_t *o = out + (v * n_sub + s) * RO_BLOCKQ8_BYTES;
            float mx[32], sm[32];
            for (int l = 0; l < 32; l++) { mx[l] = fabsf(p[l]); sm[l] = p[l]; }
            for (int off = 16; off > 0; off >>= 1) {
                float nm[32], ns[32];
                for (int l = 0; l < 32; l++) {
                    nm[l] = fmaxf(mx[l], mx[l ^ off]);
                    ns[l] = sm[l] + sm[l ^ off];
                }
                memcpy(mx, nm, sizeof mx);
                memcpy(sm, ns, sizeof sm);
            }
            float amax = mx[0], sum = sm[0];
            float d = amax > 0.0f ? amax / 127.0f : 1.0f;
            float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
            memcpy(o, &d, 4);
            memcpy(o + 4, &sum, 4);
            for (int l = 0; l < 32; l++) {
                /* rint in the default mode is round-half-even.  The float->int conversion
                 * saturates and maps NaN to 0, as the GPU conversion instruction does (a
                 * subnormal amax makes inv infinite). */
                float r = rintf(p[l] * inv);
                int q = isnan(r) ? 0 : r > 127.0f ? 127 : r < -127.0f ? -127 : (int)r;
                o[8 + l] = (uint8_t)(int8_t)q;
            }
        }
}

void ro_dequantize_q8(const uint8_t *xq, float *out, size_t in_dim, size_t n_vec)
{
    size_t n = n_vec * (in_dim / 32);
    for (size_t i = 0; i < n; i++) {
        float d;
        memcpy(&d, xq + i * RO_BLOCKQ8_BYTES, 4);
        for (int l = 0; l < 32; l++)
            out[i * 32 + l] = d * (float)(int8_t)xq[i * RO_BLOCKQ8_BYTES + 8 + l];
    }
}

/* ------------------------------------------------------ int8-path matvec --- */

typedef struct {
    const uint8_t *nib, *aux, *sc, *sup; /* plane bases */
    size_t nsp, n_super;
} planes_t;

static void find_planes(int t, const uint8_t *w, size_t in_dim, size_t out_dim, planes_t *p)
{
    size_t nsp = ro_nsp(in_dim), q = out_dim * nsp;
    p->nsp = nsp;
    p->n_super = in_dim / 256;
    p->nib = w;
    p->aux = NULL;
    p->sc = NULL;
    p->sup = NULL;
    switch (t) {
    case RO_Q4_0: case RO_IQ4_XS: case RO_IQ3_S: p->sc = w + q * 16; p->sup = NULL; break;
    case RO_Q8_0: p->aux = w + q * 16; p->sc = w + q * 32; p->sup = NULL; break;
    case RO_Q5_1: p->aux = w + q * 16; p->sc = w + q * 20; p->sup = NULL; break; /* sc: d | m << 16 per sub-block */
    case RO_Q4_K: p->sc = w + q * 16; p->sup = p->sc + q * 2; break;
    case RO_Q5_K: p->aux = w + q * 16; p->sc = p->aux + q * 4; p->sup = p->sc + q * 2; break;
    case RO_Q6_K: p->aux = w + q * 16; p->sc = p->aux + q * 8; p->sup = p->sc + q * 2; break;
    }
}

/* One (weight row, sub-block) against one activation block.  Returns the f32
 * term in the expression shape of the kernel bodies and the integers.
 *   Q4_K  kernels/matvec_q4k_repacked.cpp:105-122   dsc*dx*idot - deff*xsum
 *   Q5_K  kernels/matvec_q5k_repacked.cpp:79-96     same with the 5th bit
 *   Q6_K  kernels/matvec_q6k_repacked.cpp:83-109    two halves, (q-32)
 *   Q8_0  kernels/matvec_q8_0_repacked.cpp:77-86    dw*dx*idot
 *   Q4_0  kernels/matvec_q4_0_repacked.cpp:84-111   dw*dx*(idot - 8*xqsum)
 *   IQ4_XS kernels/matvec_iq4xs_repacked.cpp:104-116 dw*dx*sum LUT[q]*xq
 * The MMQ kernels fold the -8 / -32 into the expanded int8 weights
 * (kernels/mmq_gemm_q4_0_repacked.cpp:71-73, mmq_gemm_q6k_repacked.cpp:49-51),
 * which yields the same integers. */
static float block_term(int t, const planes_t *p, size_t row, size_t sb,
                        const uint8_t *xb, int32_t ints[2])
{
    size_t i = row * p->nsp + sb;
    const uint8_t *nb = p->nib + i * 16;
    const int8_t *xq = (const int8_t *)(xb + 8);
    float dx, xsum;
    memcpy(&dx, xb, 4);
    memcpy(&xsum, xb + 4, 4);
    ints[0] = ints[1] = 0;
    switch (t) {
    case RO_Q4_K: case RO_Q5_K: {
        int32_t idot = 0;
        uint32_t hb = 0;
        if (t == RO_Q5_K) {
            const uint8_t *h = p->aux + i * 4;
            hb = (uint32_t)h[0] | ((uint32_t)h[1] << 8) | ((uint32_t)h[2] << 16) |
                 ((uint32_t)h[3] << 24);
        }
        for (int g = 0; g < 8; g++)
            for (int c = 0; c < 4; c++) {
                int wi = group_weight(g, c);
                int q = (wi < 16) ? (nb[wi] & 15) : (nb[wi - 16] >> 4);
                q |= (int)((hb >> (4 * g + c)) & 1u) << 4;
                idot += q * xq[wi];
            }
        ints[0] = idot;
        const uint8_t *dd = p->sup + (row * p->n_super + sb / 8) * 4;
        float dsc = ro_f16_to_f32(rd16(dd)) * (float)p->sc[i * 2];
        float deff = ro_f16_to_f32(rd16(dd + 2)) * (float)p->sc[i * 2 + 1];
        float a = dsc * dx;
        a = a * (float)idot;
        float b = deff * xsum;
        return a - b;
    }
    case RO_Q5_1: {
        /* The Q5_K body with dsc = d, deff = -m (kernels/moe_matvec_q5k_repacked.cpp:86-91). */
        const uint8_t *h = p->aux + i * 4;
        uint32_t hb = (uint32_t)h[0] | ((uint32_t)h[1] << 8) | ((uint32_t)h[2] << 16) | ((uint32_t)h[3] << 24);
        int32_t idot = 0;
        for (int g = 0; g < 8; g++)
            for (int c = 0; c < 4; c++) {
                int wi = group_weight(g, c);
                int q = (wi < 16) ? (nb[wi] & 15) : (nb[wi - 16] >> 4);
                q |= (int)((hb >> (4 * g + c)) & 1u) << 4;
                idot += q * xq[wi];
            }
        ints[0] = idot;
        float dsc = ro_f16_to_f32(rd16(p->sc + i * 4));
        float deff = -ro_f16_to_f32(rd16(p->sc + i * 4 + 2));
        float a = dsc * dx;
        a = a * (float)idot;
        float b = deff * xsum;
        return a - b;
    }
    case RO_Q6_K: {
        const uint8_t *h2 = p->aux + i * 8;
        int32_t i0 = 0, i1 = 0;
        for (int g = 0; g < 8; g++)
            for (int c = 0; c < 4; c++) {
                int wi = group_weight(g, c);
                int q = (wi < 16) ? (nb[wi] & 15) : (nb[wi - 16] >> 4);
                q |= ((h2[g] >> (2 * c)) & 3) << 4;
                if (wi < 16) i0 += (q - 32) * xq[wi];
                else i1 += (q - 32) * xq[wi];
            }
        ints[0] = i0;
        ints[1] = i1;
        float d = ro_f16_to_f32(rd16(p->sup + (row * p->n_super + sb / 8) * 2));
        float lo = d * (float)(int8_t)p->sc[i * 2];
        float hi = d * (float)(int8_t)p->sc[i * 2 + 1];
        float a = lo * dx;
        a = a * (float)i0;
        float b = hi * dx;
        b = b * (float)i1;
        return a + b;
    }
    case RO_Q8_0: {
        const int8_t *lo = (const int8_t *)nb;
        const int8_t *hi = (const int8_t *)(p->aux + i * 16);
        int32_t idot = 0;
        for (int k = 0; k < 16; k++) idot += lo[k] * xq[k] + hi[k] * xq[16 + k];
        ints[0] = idot;
        float a = ro_f16_to_f32(rd16(p->sc + i * 2)) * dx;
        return a * (float)idot;
    }
    case RO_Q4_0: {
        int32_t idot = 0;
        for (int k = 0; k < 16; k++)
            idot += ((nb[k] & 15) - 8) * xq[k] + ((nb[k] >> 4) - 8) * xq[16 + k];
        ints[0] = idot;
        float a = ro_f16_to_f32(rd16(p->sc + i * 2)) * dx;
        return a * (float)idot;
    }
    case RO_IQ4_XS: {
        int32_t idot = 0;
        for (int k = 0; k < 16; k++)
            idot += IQ4NL[nb[k] & 15] * xq[k] + IQ4NL[nb[k] >> 4] * xq[16 + k];
        ints[0] = idot;
        float a = ro_f16_to_f32(rd16(p->sc + i * 2)) * dx;
        return a * (float)idot;
    }
    case RO_IQ3_S: {
        /* The IQ4_XS kernel body with the codebook v = 2n - 15 (src/quant/iq3_s.rs:193-214). */
        int32_t idot = 0;
        for (int k = 0; k < 16; k++)
            idot += (2 * (nb[k] & 15) - 15) * xq[k] + (2 * (nb[k] >> 4) - 15) * xq[16 + k];
        ints[0] = idot;
        float a = ro_f16_to_f32(rd16(p->sc + i * 2)) * dx;
        return a * (float)idot;
    }
    }
    return 0.0f;
}

int ro_matvec_q8(int t, const uint8_t *w, const uint8_t *xq, size_t in_dim, size_t out_dim,
                 size_t n_rows, size_t row_begin, size_t row_end, float *y32, double *y64,
                 int32_t *idots)
{
    if (!ro_repacked_len(t, in_dim, out_dim ? out_dim : 1)) return -1;
    planes_t p;
    find_planes(t, w, in_dim, out_dim, &p);
    size_t n_sub = in_dim / 32;
    for (size_t b = 0; b < n_rows; b++)
        for (size_t r = row_begin; r < row_end; r++) {
            float a32 = 0.0f;
            double a64 = 0.0;
            for (size_t s = 0; s < n_sub; s++) {
                int32_t ints[2];
                float term = block_term(t, &p, r, s, xq + (b * n_sub + s) * RO_BLOCKQ8_BYTES,
                                        ints);
                a32 = a32 + term;
                a64 += (double)term;
                if (idots) {
                    int32_t *o = idots + ((b * out_dim + r) * n_sub + s) * 2;
                    o[0] = ints[0];
                    o[1] = ints[1];
                }
            }
            if (y32) y32[b * out_dim + r] = a32;
            if (y64) y64[b * out_dim + r] = a64;
        }
    return 0;
}

int ro_grouped_q8(int t, const uint8_t *slab, size_t bytes_per_expert,
                  const int32_t *expert_off, size_t n_expert, const uint8_t *xq,
                  size_t in_dim, size_t out_dim, float *y32, double *y64)
{
    size_t n_sub = in_dim / 32;
    for (size_t e = 0; e < n_expert; e++) {
        size_t lo = (size_t)expert_off[e], hi = (size_t)expert_off[e + 1];
        if (hi <= lo) continue;
        int rc = ro_matvec_q8(t, slab + e * bytes_per_expert,
                              xq + lo * n_sub * RO_BLOCKQ8_BYTES, in_dim, out_dim, hi - lo, 0,
                              out_dim, y32 ? y32 + lo * out_dim : NULL,
                              y64 ? y64 + lo * out_dim : NULL, NULL);
        if (rc) return rc;
    }
    return 0;
}

/* ------------------------------------------------------- f32 CPU path ----- */

typedef struct {
    int type;
    const uint8_t *blocks;
    const float *x;
    const float *w;
    float *w_out;
    float *y;
    size_t in_dim, out_dim, n_rows, r0, r1;
    int dequant;
} job_t;

/* src/cpu/ops.rs:118-139: one sequential f32 accumulator per output row. */
static void rows_f32(const float *x, const float *w, size_t in_dim, size_t r0, size_t r1,
                     float *y)
{
    for (size_t j = r0; j < r1; j++) {
        const float *row = w + j * in_dim;
        float acc = 0.0f;
        for (size_t i = 0; i < in_dim; i++) acc += x[i] * row[i];
        y[j] = acc;
    }
}

static void *job_main(void *arg)
{
    job_t *j = (job_t *)arg;
    if (j->dequant) {
        size_t bw = ro_block_weights(j->type), bb = ro_block_bytes(j->type);
        size_t per_row = j->in_dim / bw * bb;
        ro_dequantize(j->type, j->blocks + j->r0 * per_row, j->w_out + j->r0 * j->in_dim,
                      (j->r1 - j->r0) * j->in_dim);
    }
    for (size_t b = 0; b < j->n_rows; b++)
        rows_f32(j->x + b * j->in_dim, j->w, j->in_dim, j->r0, j->r1, j->y + b * j->out_dim);
    return NULL;
}

static void run_jobs(job_t *proto, int n_threads)
{
    if (n_threads < 1) n_threads = 1;
    if ((size_t)n_threads > proto->out_dim) n_threads = (int)(proto->out_dim ? proto->out_dim : 1);
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)n_threads);
    job_t *jobs = (job_t *)malloc(sizeof(job_t) * (size_t)n_threads);
    for (int k = 0; k < n_threads; k++) {
        jobs[k] = *proto;
        jobs[k].r0 = proto->out_dim * (size_t)k / (size_t)n_threads;
        jobs[k].r1 = proto->out_dim * (size_t)(k + 1) / (size_t)n_threads;
        if (k) pthread_create(&th[k], NULL, job_main, &jobs[k]);
    }
    job_main(&jobs[0]);
    for (int k = 1; k < n_threads; k++) pthread_join(th[k], NULL);
    free(th);
    free(jobs);
}

void ro_matvec_f32(const float *x, const float *w, size_t in_dim, size_t out_dim, float *y,
                   int n_threads)
{
    job_t j;
    memset(&j, 0, sizeof j);
    j.x = x; j.w = w; j.y = y;
    j.in_dim = in_dim; j.out_dim = out_dim; j.n_rows = 1;
    /* src/cpu/ops.rs:116-128: small products stay on one thread. */
    if (in_dim * out_dim < ((size_t)1 << 16)) n_threads = 1;
    run_jobs(&j, n_threads);
}

int ro_cpu_path(int t, const uint8_t *blocks, const float *x, size_t in_dim, size_t out_dim,
                size_t n_rows, float *w_f32, float *y, int n_threads, int dequant)
{
    size_t bw = ro_block_weights(t);
    if (!bw || in_dim % bw) return -1;
    job_t j;
    memset(&j, 0, sizeof j);
    j.type = t; j.blocks = blocks; j.x = x; j.w = w_f32; j.w_out = w_f32; j.y = y;
    j.in_dim = in_dim; j.out_dim = out_dim; j.n_rows = n_rows; j.dequant = dequant;
    run_jobs(&j, n_threads);
    return 0;
}

/* ------------------------------------------------------------ MoE pieces --- */

void ro_moe_sort(const int32_t *ids, size_t n_entries, size_t n_expert, size_t bn,
                 int32_t *count, int32_t *expert_off, int32_t *tile_off, int32_t *perm)
{
    for (size_t e = 0; e < n_expert; e++) count[e] = 0;
    for (size_t i = 0; i < n_entries; i++)
        if (ids[i] >= 0 && (size_t)ids[i] < n_expert) count[ids[i]]++;
    int32_t eo = 0, to = 0;
    for (size_t e = 0; e < n_expert; e++) {
        expert_off[e] = eo;
        tile_off[e] = to;
        eo += count[e];
        to += (int32_t)(((size_t)count[e] + bn - 1) / bn);
    }
    expert_off[n_expert] = eo;
    tile_off[n_expert] = to;
    int32_t *cur = (int32_t *)calloc(n_expert ? n_expert : 1, sizeof(int32_t));
    for (size_t i = 0; i < n_entries; i++)
        if (ids[i] >= 0 && (size_t)ids[i] < n_expert)
            perm[expert_off[ids[i]] + cur[ids[i]]++] = (int32_t)i;
    free(cur);
}

void ro_router_topk(const float *logits, size_t n_tok, size_t n_expert, size_t n_used,
                    int32_t *ids, float *weights)
{
    float *p = (float *)malloc(sizeof(float) * n_expert);
    for (size_t t = 0; t < n_tok; t++) {
        const float *lg = logits + t * n_expert;
        float m = -INFINITY;
        for (size_t i = 0; i < n_expert; i++) {
            p[i] = isnan(lg[i]) ? -INFINITY : lg[i];
            m = fmaxf(m, p[i]);
        }
        float sum = 0.0f;
        for (size_t i = 0; i < n_expert; i++) { p[i] = expf(p[i] - m); sum += p[i]; }
        float inv = 1.0f / sum;
        for (size_t i = 0; i < n_expert; i++) p[i] *= inv;
        float wsum = 0.0f;
        for (size_t k = 0; k < n_used; k++) {
            size_t best = 0;
            float bv = -1.0f;
            for (size_t i = 0; i < n_expert; i++)
                if (p[i] > bv) { bv = p[i]; best = i; }
            ids[t * n_used + k] = (int32_t)best;
            weights[t * n_used + k] = bv;
            wsum += bv;
            p[best] = -1.0f;
        }
        if (wsum < 6.103515625e-5f) wsum = 6.103515625e-5f;
        for (size_t k = 0; k < n_used; k++) weights[t * n_used + k] /= wsum;
    }
    free(p);
}

/* kernels/moe_geglu_q8.cpp:20-66 (GeGLU) and kernels/swiglu.cpp:11-21 (SwiGLU): the gated
 * activation of a fused gate_up row, then the BlockQ8 quantizer of ro_quantize_q8.  act_out
 * (optional) receives the f32 values before quantization. */
static float ro_gelu_tanh(float x)
{
    const float k = 0.7978845608028654f;
    float c = x + 0.044715f * x * x * x;
    return 0.5f * x * (1.0f + tanhf(k * c));
}

void ro_moe_act_q8(const float *gu, uint8_t *out, size_t ff, size_t n_slot, int act, float *act_out)
{
    float *v = (float *)malloc(sizeof(float) * (ff ? ff : 1));
    for (size_t s = 0; s < n_slot; s++) {
        const float *g = gu + s * 2 * ff, *u = g + ff;
        for (size_t i = 0; i < ff; i++) {
            float a = act == 0 ? ro_gelu_tanh(g[i]) : g[i] / (1.0f + expf(-g[i]));
            v[i] = a * u[i];
        }
        if (act_out) memcpy(act_out + s * ff, v, sizeof(float) * ff);
        ro_quantize_q8(v, out + s * (ff / 32) * RO_BLOCKQ8_BYTES, ff, 1);
    }
    free(v);
}

/* kernels/moe_combine.cpp:16-37: slot-order accumulation; the device compiler contracts the
 * source's acc += s * v into one fused multiply-add, written out here. */
void ro_moe_combine(const float *experts, const int32_t *ids, const float *weights, const float *expert_scale,
                    float *out, size_t hidden, size_t n_used, size_t n_tok)
{
    for (size_t t = 0; t < n_tok; t++)
        for (size_t i = 0; i < hidden; i++) {
            float acc = 0.0f;
            for (size_t j = 0; j < n_used; j++) {
                float w = weights[t * n_used + j];
                float sc = expert_scale ? w * expert_scale[ids[t * n_used + j]] : w;
                acc = fmaf(sc, experts[(t * n_used + j) * hidden + i], acc);
            }
            out[t * hidden + i] = acc;
        }
}

/* ------------------------------------------- relabelled source formats --- */
/* Tensor types the loaders accept by mapping them exactly onto a layout that has kernels
 * (src/runtime/qwen35.rs:274-307): Q3_K -> Q6_K blocks, IQ4_NL -> the repacked IQ4_XS planes,
 * BF16 -> Q8_0 blocks (the only lossy one: a requantization). */

/* The sixteen 6-bit sub-block scales of a Q3_K block (src/quant/q3_k.rs:43-65): scale i has its
 * low nibble in byte (i & 7) of the first eight (low half for i < 8, high half for i >= 8) and
 * its two high bits in field (i >> 2) of byte 8 + (i & 3). */
static int q3k_scale(const uint8_t *sc, int i)
{
    int j = i & 3, grp = i >> 2;
    int low = grp < 2 ? (sc[grp * 4 + j] & 15) : ((sc[(grp - 2) * 4 + j] >> 4) & 15);
    int high = (sc[8 + j] >> (2 * grp)) & 3;
    return low | (high << 4);
}

/* Stored 3-bit quant (0..7) of weight y of a block (src/quant/q3_k.rs:67-90): weight
 * y = 128*c + 32*j + l has its low two bits in field j of qs[32*c + l] and its third bit in bit
 * 4*c + j of hmask[l]. */
static int q3k_quant(const uint8_t *b, int y)
{
    int c = y >> 7, j = (y >> 5) & 3, l = y & 31;
    int lo = (b[32 + 32 * c + l] >> (2 * j)) & 3;
    int hi = (b[l] >> (4 * c + j)) & 1;
    return lo | (hi << 2);
}

/* src/quant/q3_k.rs:123-162: w = (d * (sc - 32)) * (q3 - 4), sub-blocks of 16 weights. */
void ro_dequantize_q3_k(const uint8_t *blocks, float *out, size_t n_weights)
{
    for (size_t blk = 0; blk < n_weights / 256; blk++) {
        const uint8_t *b = blocks + blk * 110;
        float d = ro_f16_to_f32(rd16(b + 108));
        for (int y = 0; y < 256; y++) {
            float dl = d * (float)(q3k_scale(b + 96, y >> 4) - 32);
            out[blk * 256 + y] = dl * (float)(q3k_quant(b, y) - 4);
        }
    }
}

/* src/quant/q3_k.rs:92-121: q6 = q3 + 28, sc6 = sc3 - 32, same d; packed the way the Q6_K decoder
 * reads ql / qh (src/quant/q6_k.rs). */
void ro_q3k_to_q6k(const uint8_t *blocks, uint8_t *out, size_t n_weights)
{
    for (size_t blk = 0; blk < n_weights / 256; blk++) {
        const uint8_t *b = blocks + blk * 110;
        uint8_t *o = out + blk * 210;
        memset(o, 0, 210);
        for (int c = 0; c < 2; c++)
            for (int l = 0; l < 32; l++) {
                int q1 = q3k_quant(b, 128 * c + l) + 28, q2 = q3k_quant(b, 128 * c + 32 + l) + 28;
                int q3 = q3k_quant(b, 128 * c + 64 + l) + 28, q4 = q3k_quant(b, 128 * c + 96 + l) + 28;
                o[64 * c + l] = (uint8_t)((q1 & 15) | ((q3 & 15) << 4));
                o[64 * c + 32 + l] = (uint8_t)((q2 & 15) | ((q4 & 15) << 4));
                o[128 + 32 * c + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
            }
        for (int i = 0; i < 16; i++) o[192 + i] = (uint8_t)(int8_t)(q3k_scale(b + 96, i) - 32);
        o[208] = b[108];
        o[209] = b[109];
    }
}

/* src/quant/iq4_nl.rs:32-46: w = d * codebook[nibble]; byte k = weight k (low) and k + 16 (high). */
void ro_dequantize_iq4_nl(const uint8_t *blocks, float *out, size_t n_weights)
{
    for (size_t blk = 0; blk < n_weights / 32; blk++) {
        const uint8_t *b = blocks + blk * 18;
        float d = ro_f16_to_f32(rd16(b));
        for (int k = 0; k < 16; k++) {
            out[blk * 32 + k] = d * (float)IQ4NL[b[2 + k] & 15];
            out[blk * 32 + k + 16] = d * (float)IQ4NL[b[2 + k] >> 4];
        }
    }
}

/* src/quant/q8_0.rs:45-61: d = amax / 127, q = round-half-away(v * (1/d)) clamped to +-127,
 * d stored as f16. */
void ro_quantize_q8_0(const float *vals, uint8_t *out, size_t n)
{
    for (size_t blk = 0; blk < n / 32; blk++) {
        const float *v = vals + blk * 32;
        uint8_t *o = out + blk * 34;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(v[i]));
        float d = amax / 127.0f;
        float inv = d > 0.0f ? 1.0f / d : 0.0f;
        wr16(o, ro_f32_to_f16(d));
        for (int i = 0; i < 32; i++) {
            float r = roundf(v[i] * inv);
            r = r > 127.0f ? 127.0f : r < -127.0f ? -127.0f : r;
            o[2 + i] = (uint8_t)(int8_t)(isnan(r) ? 0 : (int)r);
        }
    }
}

/* Source type -> the type whose kernels run it (src/runtime/qwen35.rs:274-307); -1 if none. */
int ro_kernel_type(int src_type)
{
    switch (src_type) {
    case RO_Q4_0: case RO_Q5_1: case RO_Q8_0: case RO_Q4_K: case RO_Q5_K: case RO_Q6_K: case RO_IQ4_XS: case RO_IQ3_S: return src_type;
    case RO_Q3_K: return RO_Q6_K;
    case RO_IQ4_NL: return RO_IQ4_XS;
    case RO_BF16: return RO_Q8_0;
    }
    return -1;
}

/* On-disk rows of a source type -> the repacked planes of its kernel type. */
int ro_repack_any(int src_type, const uint8_t *src, size_t in_dim, size_t out_dim, uint8_t *out)
{
    size_t n = in_dim * out_dim;
    if (src_type == RO_Q3_K) {
        if (in_dim % 256) return -2;
        uint8_t *q6 = (uint8_t *)malloc((n / 256) * 210);
        ro_q3k_to_q6k(src, q6, n);
        int rc = ro_repack(RO_Q6_K, q6, in_dim, out_dim, out);
        free(q6);
        return rc;
    }
    if (src_type == RO_IQ4_NL) /* same block shape and byte order as Q4_0; d is the sub-block scale as-is */
        return ro_repack(RO_Q4_0, src, in_dim, out_dim, out);
    if (src_type == RO_BF16) {
        if (in_dim % 32) return -2;
        float *f = (float *)malloc(n * sizeof(float));
        uint8_t *q8 = (uint8_t *)malloc((n / 32) * 34);
        for (size_t i = 0; i < n; i++) f[i] = ro_bf16_to_f32(rd16(src + 2 * i));
        ro_quantize_q8_0(f, q8, n);
        int rc = ro_repack(RO_Q8_0, q8, in_dim, out_dim, out);
        free(f);
        free(q8);
        return rc;
    }
    return ro_repack(src_type, src, in_dim, out_dim, out);
}

/* ------------------------------------------- fused BlockQ8 producers --- */
/* kernels/rmsnorm_q8.cpp:38-103 and kernels/qwen35_fused.cpp:66-118: x (+ add) -> rmsnorm * w -> BlockQ8.
 * The sum of squares is reduced in the order the CUDA kernel fixes (the reference's own order, a
 * 512-thread tree or a wave64 reduction, is a property of its launch geometry): 1024 strided partial
 * sums, a 32-lane xor-butterfly per group of 32, the 32 group sums added in order; rrms with IEEE
 * divide and square root.  hidden_out / y_out may be NULL. */
void ro_rmsnorm_q8(const float *x, const float *add, const float *w, float *hidden_out, float *y_out,
                   uint8_t *out, size_t n, size_t n_vec, float eps)
{
    float *v = (float *)malloc(sizeof(float) * n);
    for (size_t vec = 0; vec < n_vec; vec++) {
        const float *xv = x + vec * n, *av = add ? add + vec * n : NULL;
        float part[1024];
        for (int t = 0; t < 1024; t++) {
            float p = 0.0f;
            for (size_t i = (size_t)t; i < n; i += 1024) {
                float e = av ? xv[i] + av[i] : xv[i];
                float sq = e * e;
                p = p + sq;
            }
            part[t] = p;
        }
        float tot = 0.0f;
        for (int wp = 0; wp < 32; wp++) {
            float s[32];
            memcpy(s, part + 32 * wp, sizeof s);
            for (int off = 16; off > 0; off >>= 1) {
                float ns[32];
                for (int l = 0; l < 32; l++) ns[l] = s[l] + s[l ^ off];
                memcpy(s, ns, sizeof s);
            }
            tot = wp == 0 ? s[0] : tot + s[0];
        }
        float mean = tot / (float)n;
        float rrms = 1.0f / sqrtf(mean + eps);
        for (size_t i = 0; i < n; i++) {
            float e = av ? xv[i] + av[i] : xv[i];
            if (hidden_out) hidden_out[vec * n + i] = e;
            float t = e * rrms;
            v[i] = t * w[i];
        }
        if (y_out) memcpy(y_out + vec * n, v, sizeof(float) * n);
        ro_quantize_q8(v, out + vec * (n / 32) * RO_BLOCKQ8_BYTES, n, 1);
    }
    free(v);
}

/* kernels/qwen35_fused.cpp:123-138: silu(gate) * up as f32 and BlockQ8. */
void ro_swiglu_q8(const float *gate, const float *up, float *out_f32, uint8_t *q8, size_t n)
{
    float *v = (float *)malloc(sizeof(float) * (n ? n : 1));
    for (size_t i = 0; i < n; i++) {
        float e = 1.0f + expf(-gate[i]);
        float s = gate[i] / e;
        v[i] = s * up[i];
    }
    if (out_f32) memcpy(out_f32, v, sizeof(float) * n);
    ro_quantize_q8(v, q8, n, 1);
    free(v);
}

/* kernels/qwen35_fused.cpp:139-152: x *= sigmoid(gate), in place and as BlockQ8. */
void ro_sigmoid_mul_q8(float *x, const float *gate, uint8_t *q8, size_t n)
{
    for (size_t i = 0; i < n; i++) {
        float e = 1.0f + expf(-gate[i]);
        x[i] = x[i] / e;
    }
    ro_quantize_q8(x, q8, n, 1);
}

/* kernels/qwen35_fused.cpp:204-224: per head y = ((x * rrms) * w) * silu(z); the head's sum of squares
 * by xor-butterfly per 32 values, the group sums added in order (the CUDA kernel's order). */
void ro_rmsnorm_gated_q8(const float *x, const float *z, const float *w, float *y, uint8_t *q8,
                         size_t n_heads, size_t head_dim, float eps)
{
    float *v = (float *)malloc(sizeof(float) * n_heads * head_dim);
    for (size_t h = 0; h < n_heads; h++) {
        const float *xh = x + h * head_dim, *zh = z + h * head_dim;
        float tot = 0.0f;
        for (size_t g = 0; g < head_dim / 32; g++) {
            float s[32];
            for (int l = 0; l < 32; l++) s[l] = xh[g * 32 + l] * xh[g * 32 + l];
            for (int off = 16; off > 0; off >>= 1) {
                float ns[32];
                for (int l = 0; l < 32; l++) ns[l] = s[l] + s[l ^ off];
                memcpy(s, ns, sizeof s);
            }
            tot = g == 0 ? s[0] : tot + s[0];
        }
        float mean = tot / (float)head_dim;
        float rrms = 1.0f / sqrtf(mean + eps);
        for (size_t i = 0; i < head_dim; i++) {
            float e = 1.0f + expf(-zh[i]);
            float silu = zh[i] / e;
            float a = xh[i] * rrms;
            float b = a * w[i];
            v[h * head_dim + i] = b * silu;
        }
    }
    if (y) memcpy(y, v, sizeof(float) * n_heads * head_dim);
    ro_quantize_q8(v, q8, n_heads * head_dim, 1);
    free(v);
}
