// Shared device helpers for the sm_100a kernels: repacked-v2 plane arithmetic, streaming
// loads, fp16 decode, and the staged (planar) form of the BlockQ8 activation blocks.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/reinstinct_cuda.h"

namespace rc {

constexpr int kWarp = 32;

// IQ3_S names the KERNEL type of an IQ3_S tensor: the IQ4_XS planes (a nibble and one fp16 scale per
// 32 weights) read through the codebook v = 2n - 15 (src/quant/iq3_s.rs:193-214).  The 110-byte
// on-disk blocks are turned into those planes by the caller's host code; there is no device repack.
// Q5_1 (24-byte blocks of 32: fp16 d, fp16 m, 4 bytes of 5th bits, 16 nibble bytes; w = d * q5 + m) runs
// on the Q5_K kernel bodies with dsc = d, deff = -m (src/quant/q5_1.rs:11-20): planes = the Q5_K nibble
// and 5th-bit planes, then one word d | m << 16 per sub-block; no superblock plane.
enum Fmt : int { Q4_0 = 2, Q5_1 = 7, Q8_0 = 8, Q4_K = 12, Q5_K = 13, Q6_K = 14, IQ3_S = 21, IQ4_XS = 23 };

// the two formats whose nibbles index a 16-entry int8 codebook
template <int FMT> constexpr bool kCodebook = (FMT == IQ4_XS || FMT == IQ3_S);

// Tensor types accepted as SOURCES of rc_repack_for_matvec only: each maps exactly (BF16: by a Q8_0
// requantization) onto one of the six layouts above (src/runtime/qwen35.rs:274-307).
enum SrcFmt : int { SRC_Q3_K = 11, SRC_IQ4_NL = 20, SRC_BF16 = 30 };

// The type whose kernels run a source type; -1 if there is none.
__host__ __device__ inline int fmt_kernel_type(int t)
{
    switch (t) {
    case Q4_0: case Q5_1: case Q8_0: case Q4_K: case Q5_K: case Q6_K: case IQ4_XS: case IQ3_S: return t;
    case SRC_Q3_K: return Q6_K;
    case SRC_IQ4_NL: return IQ4_XS;
    case SRC_BF16: return Q8_0;
    }
    return -1;
}
// weights and bytes of one source block (BF16: rows are handled 32 values at a time)
__host__ __device__ inline uint32_t src_block_weights(int t) { return t == SRC_Q3_K ? 256u : 32u; }
__host__ __device__ inline uint32_t src_block_bytes(int t) { return t == SRC_Q3_K ? 110u : t == SRC_IQ4_NL ? 18u : 64u; }

__host__ __device__ inline bool fmt_known(int t)
{
    return t == Q4_0 || t == Q5_1 || t == Q8_0 || t == Q4_K || t == Q5_K || t == Q6_K || t == IQ4_XS || t == IQ3_S;
}
__host__ __device__ inline uint32_t fmt_block_weights(int t)
{
    return (t == Q4_0 || t == Q8_0 || t == Q5_1) ? 32u : 256u;
}
__host__ __device__ inline uint32_t fmt_block_bytes(int t)
{
    switch (t) {
    case Q4_0: return 18;
    case Q5_1: return 24;
    case Q8_0: return 34;
    case Q4_K: return 144;
    case Q5_K: return 176;
    case Q6_K: return 210;
    case IQ4_XS: return 136;
    case IQ3_S: return 110;
    }
    return 0;
}

// Padded sub-blocks per repacked row: one extra when the natural count is a power of two
// (src/quant/q4_k.rs:92-95).
__host__ __device__ inline uint32_t nsp_of(uint32_t n_sub)
{
    return (n_sub && (n_sub & (n_sub - 1u)) == 0u) ? n_sub + 1u : n_sub;
}

// Plane bases of one repacked tensor.  `aux` is the Q5_K 5th-bit plane, the Q6_K
// high-2-bit plane or the Q8_0 hi-half plane; `sc` the per-sub-block scale plane; `sup`
// the per-256 superblock plane (src/quant/<fmt>.rs::repack_for_matvec).
struct Planes {
    const uint8_t *nib, *aux, *sc, *sup;
    uint32_t nsp, n_super;
};

template <int FMT>
__host__ __device__ inline Planes planes_of(const uint8_t *w, uint32_t in_dim, uint32_t out_dim)
{
    Planes p;
    const uint32_t n_sub = in_dim >> 5;
    p.nsp = nsp_of(n_sub);
    p.n_super = n_sub >> 3;
    const size_t q = (size_t)out_dim * p.nsp;
    p.nib = w;
    p.aux = nullptr;
    p.sup = nullptr;
    if (FMT == Q4_0 || FMT == IQ4_XS || FMT == IQ3_S) {
        p.sc = w + q * 16;
    } else if (FMT == Q8_0) {
        p.aux = w + q * 16;
        p.sc = w + q * 32;
    } else if (FMT == Q4_K) {
        p.sc = w + q * 16;
        p.sup = p.sc + q * 2;
    } else if (FMT == Q5_1) {
        p.aux = w + q * 16;
        p.sc = p.aux + q * 4; // d | m << 16, four bytes per sub-block
    } else if (FMT == Q5_K) {
        p.aux = w + q * 16;
        p.sc = p.aux + q * 4;
        p.sup = p.sc + q * 2;
    } else { // Q6_K
        p.aux = w + q * 16;
        p.sc = p.aux + q * 8;
        p.sup = p.sc + q * 2;
    }
    return p;
}

__host__ __device__ inline size_t repacked_len_of(int t, size_t in_dim, size_t out_dim)
{
    if (!fmt_known(t) || in_dim == 0 || in_dim % fmt_block_weights(t)) return 0;
    const size_t nsp = nsp_of((uint32_t)(in_dim >> 5));
    size_t per_sub = 18, per_super = 0;
    if (t == Q8_0) per_sub = 34;
    if (t == Q5_1) per_sub = 24;
    if (t == Q4_K) per_super = 4;
    if (t == Q5_K) { per_sub = 22; per_super = 4; }
    if (t == Q6_K) { per_sub = 26; per_super = 2; }
    return out_dim * nsp * per_sub + out_dim * (in_dim >> 8) * per_super;
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// The kernels of the decode chain run back to back on one stream and last a few microseconds,
// so launch ramp and tail are a sizeable share.  Launched with programmatic stream
// serialization, a kernel may start while its predecessor drains: it calls
// pdl_launch_dependents() early (its own successor may then start too) and pdl_wait() before it
// touches anything a predecessor wrote or still reads — weights are never such data, so their
// first loads go out before the wait.  Both instructions are no-ops in a plain launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- loads -------------------------------------------------------------------------

// Weight bytes are read exactly once per launch: bypass L1 allocation.
__device__ __forceinline__ uint4 ld_stream_u4(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_u2(const void *p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const void *p)
{
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_nc_u16(const void *p)
{
    return (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(p));
}

__device__ __forceinline__ float f16_bits_to_f32(uint32_t bits)
{
    return __half2float(__ushort_as_half((unsigned short)(bits & 0xFFFFu)));
}

// ---- BlockQ8 --------------------------------------------------------------------------

// One activation block as the kernels consume it from shared memory: the 32 int8 quants
// as two 16-byte halves (weights 0..15, 16..31), the f32 scale and plain sum, and the
// integer sums of the two halves (used by the Q6_K "-32" and Q4_0 "-8" offsets,
// kernels/matvec_q6k_repacked.cpp:83-88, kernels/matvec_q4_0_repacked.cpp:84-91).
struct XBlock {
    int4 lo, hi;
    float d, xsum;
    int s_lo, s_hi;
};

// Reads one 40-byte BlockQ8 (8-byte aligned) from global memory.
__device__ __forceinline__ XBlock load_blockq8(const uint8_t *p)
{
    const uint2 *q = reinterpret_cast<const uint2 *>(p);
    const uint2 a = __ldg(q), b = __ldg(q + 1), c = __ldg(q + 2), e = __ldg(q + 3), f = __ldg(q + 4);
    XBlock x;
    x.d = __uint_as_float(a.x);
    x.xsum = __uint_as_float(a.y);
    x.lo = make_int4((int)b.x, (int)b.y, (int)c.x, (int)c.y);
    x.hi = make_int4((int)e.x, (int)e.y, (int)f.x, (int)f.y);
    const int ones = 0x01010101;
    x.s_lo = __dp4a(x.lo.x, ones, __dp4a(x.lo.y, ones, __dp4a(x.lo.z, ones, __dp4a(x.lo.w, ones, 0))));
    x.s_hi = __dp4a(x.hi.x, ones, __dp4a(x.hi.y, ones, __dp4a(x.hi.z, ones, __dp4a(x.hi.w, ones, 0))));
    return x;
}

// ---- bit spreading ------------------------------------------------------------------------

// Bits 0..3 of h -> bit 4 of bytes 0..3 (the Q5_K 5th weight bit).  0x00204081 places bit
// i at 8i after the multiply; no two partial products share a bit position.
__device__ __forceinline__ uint32_t bits4_to_bit4(uint32_t h)
{
    return (((h & 0xFu) * 0x00204081u) & 0x01010101u) << 4;
}

// The four 2-bit fields of byte h -> bits 4..5 of bytes 0..3 (the Q6_K high pair).
// Field c must move left by 6c+4.  Even and odd fields are spread by separate multiplies
// so that no two shifted copies overlap (an overlap would carry into a target bit).
__device__ __forceinline__ uint32_t fields2_to_bits45(uint32_t h)
{
    const uint32_t even = ((h & 0x33u) * 0x00010010u) & 0x00300030u;  // fields 0,2: <<4, <<16
    const uint32_t odd = ((h & 0xCCu) * 0x00400400u) & 0x30003000u;   // fields 1,3: <<10, <<22
    return even | odd;
}

// The same spreading for the four bytes of a word at once: h holds the high-2 bytes of groups
// 0..3 (byte g = four 2-bit fields of group g); g0..g3 receive, for each group, its four fields
// in bits 4..5 of bytes 0..3.  Four shift-and-mask steps pull field c of every group into one
// word, a 4x4 byte transpose (eight PRMT) regroups them: 15 operations for 16 fields and no
// multiplies.
__device__ __forceinline__ void spread_fields4(uint32_t h, uint32_t &g0, uint32_t &g1, uint32_t &g2, uint32_t &g3)
{
    const uint32_t K = 0x30303030u;
    const uint32_t f0 = (h << 4) & K, f1 = (h << 2) & K, f2 = h & K, f3 = (h >> 2) & K; // [grp0..grp3] of field c
    const uint32_t t0 = __byte_perm(f0, f1, 0x5140u), t1 = __byte_perm(f2, f3, 0x5140u); // groups 0,1
    const uint32_t t2 = __byte_perm(f0, f1, 0x7362u), t3 = __byte_perm(f2, f3, 0x7362u); // groups 2,3
    g0 = __byte_perm(t0, t1, 0x5410u);
    g1 = __byte_perm(t0, t1, 0x7632u);
    g2 = __byte_perm(t2, t3, 0x5410u);
    g3 = __byte_perm(t2, t3, 0x7632u);
}

// IQ4_NL codebook {-127,-104,-83,-65,-49,-35,-22,-10,1,13,25,38,53,69,89,113}
// (src/quant/iq4_xs.rs:28-31) and the IQ3_S codebook {-15,-13,...,13,15}
// (src/quant/iq3_s.rs:193-194), each as four little-endian words.
template <int FMT> struct Codebook {
    static constexpr uint32_t w0 = 0xBFAD9881u, w1 = 0xF6EADDCFu, w2 = 0x26190D01u, w3 = 0x71594535u;
};
template <> struct Codebook<IQ3_S> {
    static constexpr uint32_t w0 = 0xF7F5F3F1u, w1 = 0xFFFDFBF9u, w2 = 0x07050301u, w3 = 0x0F0D0B09u;
};

// Eight 4-bit codebook indices packed in q (byte k = index a_k low, b_k high) -> two
// words of int8 codebook values, in the order the selector nibbles arrive:
//   first  = [T[a0], T[b0], T[a1], T[b1]],  second = [T[a2], T[b2], T[a3], T[b3]].
// PRMT reads selector nibbles directly, so no unpacking to bytes is needed: the low three
// bits pick within a half-table, bit 3 then picks the half.  The matching activation
// order is produced once per CTA when the activations are staged (xperm_iq4).
template <int FMT = IQ4_XS>
__device__ __forceinline__ void iq4_lookup8(uint32_t q, int &first, int &second)
{
    using C = Codebook<FMT>;
    const uint32_t sel = q & 0x77777777u;
    const uint32_t pick = 0x32103210u | ((q & 0x88888888u) >> 1);
    const uint32_t l0 = __byte_perm(C::w0, C::w1, sel);
    const uint32_t h0 = __byte_perm(C::w2, C::w3, sel);
    const uint32_t l1 = __byte_perm(C::w0, C::w1, sel >> 16);
    const uint32_t h1 = __byte_perm(C::w2, C::w3, sel >> 16);
    first = (int)__byte_perm(l0, h0, pick);
    second = (int)__byte_perm(l1, h1, pick >> 16);
}

// Activation words for iq4_lookup8: from lo word j = x[4j..4j+3] and hi word j =
// x[16+4j..16+4j+3] build [x(4j), x(16+4j), x(4j+1), x(16+4j+1)] and
// [x(4j+2), x(16+4j+2), x(4j+3), x(16+4j+3)].
__device__ __forceinline__ void xperm_iq4(int lo, int hi, int &first, int &second)
{
    first = (int)__byte_perm((uint32_t)lo, (uint32_t)hi, 0x5140u);
    second = (int)__byte_perm((uint32_t)lo, (uint32_t)hi, 0x7362u);
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

} // namespace rc
