// Pieces shared by the tensor-core GEMM kernels: mbarrier / TMA / tcgen05 PTX wrappers,
// explicit shared-space accessors, shared-memory operand descriptors, the byte -> f16 helpers
// and the host-side tensor-map encoders.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {

constexpr int kBM = 128;     // weight rows per tile = tensor-memory lanes
constexpr long long kWaitLimitCycles = 1000ll * 1000 * 1000; // about half a second: far beyond any legal wait (microseconds)

// ---- PTX wrappers ------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return done != 0;
}
// Non-blocking probe of a phase: returns at once, so a spin on it notices completion within a few
// cycles (try_wait may park the thread first).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return done != 0;
}
__device__ __forceinline__ uint64_t global_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1,
                                            int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, "
                 "%4, %5}], [%6];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[128 x N] (int32, tensor memory) = A[128 x 32] * B[N x 32]^T, both int8 from shared memory.
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// Arrives on `bar` when every MMA this thread issued before has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread l of the warp gets row (lane base + l).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                   "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
                   "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
                   "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                   "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle (version 1 = sm_100).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}

// Explicit shared-space loads (the operand areas are addressed through a realigned pointer, which
// the compiler would otherwise treat as generic).
__device__ __forceinline__ ulonglong2 lds_u64x2(uint32_t addr)
{
    ulonglong2 v;
    asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds_u4(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds_u2(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_u4(uint32_t addr, const uint4 &v)
{
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts_u32(uint32_t addr, uint32_t v)
{
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}


// D[128 x N] (f32) (+)= A[128 x 16] * B[N x 16]^T, f16 operands from shared memory.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// f32 accumulator, f16 A and B, both K-major, M = 128
__host__ __device__ constexpr uint32_t make_idesc_f16(uint32_t n)
{
    return (1u << 4) | ((n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}


__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

// Four unsigned bytes (each < 256) -> two half2 words holding 1024 + byte: 0x64 in the high byte of
// each half makes the exponent 2^10, the byte lands in the mantissa.
__device__ __forceinline__ void bytes_to_h2_biased(uint32_t t, uint32_t &p01, uint32_t &p23)
{
    p01 = __byte_perm(t, 0x64646464u, 0x4140u);
    p23 = __byte_perm(t, 0x64646464u, 0x4342u);
}

// Eight weights (two words of four unsigned bytes) -> one 16-byte kc block of the operand, computed
// as  (1024 + byte) * mul + add  in half2 (one rounding of an exactly representable result).
__device__ __forceinline__ uint4 kc_block(uint32_t t0, uint32_t t1, __half2 mul, __half2 add)
{
    uint32_t a, b, c, d;
    bytes_to_h2_biased(t0, a, b);
    bytes_to_h2_biased(t1, c, d);
    return make_uint4(h2_as_u32(__hfma2(u32_as_h2(a), mul, add)), h2_as_u32(__hfma2(u32_as_h2(b), mul, add)),
                      h2_as_u32(__hfma2(u32_as_h2(c), mul, add)), h2_as_u32(__hfma2(u32_as_h2(d), mul, add)));
}


typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 4-D view of the 16-byte planes of a repacked tensor (or slab of tensors):
// (byte in row, row, plane, expert); one box = 16 bytes x 128 rows of one plane.
// box_k: bytes of a row per box (16 = one sub-block; a multiple of 16 takes several sub-blocks at once and
// lands as [row][box_k bytes]).
template <int FMT>
int make_tmap(CUtensorMap *map, const void *w, size_t bytes_per_expert, uint32_t n_expert, uint32_t in_dim,
              uint32_t out_dim, uint32_t box_k = 16)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return RC_ERR_NO_DEVICE;
    const uint64_t nsp = nsp_of(in_dim >> 5);
    const cuuint64_t dims[4] = {nsp * 16, out_dim, (cuuint64_t)(FMT == Q8_0 ? 2 : 1), n_expert};
    const uint64_t plane = (uint64_t)out_dim * nsp * 16;
    const cuuint64_t strides[3] = {nsp * 16, plane, n_expert > 1 ? (cuuint64_t)bytes_per_expert : plane * 2};
    const cuuint32_t box[4] = {box_k, kBM, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(w), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? RC_OK : RC_ERR_BAD_ARGUMENT;
}


// One (row, sub-block): raw bytes -> the f16 operand rows.  out[part][kc]: part 0 (and 1 for Q6_K).
// sm: the sub-block's scale word (K-quants: sc | m << 8; Q6_K: sc_lo | sc_hi << 8).
template <int FMT>
__device__ __forceinline__ void expand_f16(const uint4 &q, const uint4 &q2, uint32_t extra0, uint32_t extra1, uint32_t sm,
                                           uint4 (&out)[2][4])
{
    const uint32_t M = 0x0F0F0F0Fu;
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t lo[4], hi[4]; // unsigned byte values of weights 4j..4j+3 and 16+4j..16+4j+3
    if constexpr (FMT == Q4_K || FMT == Q4_0) {
#pragma unroll
        for (int j = 0; j < 4; j++) { lo[j] = w[j] & M; hi[j] = (w[j] >> 4) & M; }
    } else if constexpr (FMT == Q5_K || FMT == Q5_1) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            lo[j] = (w[j] & M) | bits4_to_bit4(extra0 >> (8 * j));
            hi[j] = ((w[j] >> 4) & M) | bits4_to_bit4(extra0 >> (8 * j + 4));
        }
    } else if constexpr (FMT == Q6_K) {
        uint32_t g[8];
        spread_fields4(extra0, g[0], g[1], g[2], g[3]);
        spread_fields4(extra1, g[4], g[5], g[6], g[7]);
#pragma unroll
        for (int j = 0; j < 4; j++) { lo[j] = (w[j] & M) | g[2 * j]; hi[j] = ((w[j] >> 4) & M) | g[2 * j + 1]; }
    } else if constexpr (FMT == Q8_0) {
        const uint32_t w2[4] = {q2.x, q2.y, q2.z, q2.w};
#pragma unroll
        for (int j = 0; j < 4; j++) { lo[j] = w[j] ^ 0x80808080u; hi[j] = w2[j] ^ 0x80808080u; } // + 128
    } else { // IQ4_XS: codebook bytes, + 128
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int a0, a1;
            iq4_lookup8<FMT>(w[j], a0, a1);
            lo[j] = __byte_perm(a0, a1, 0x6420) ^ 0x80808080u;
            hi[j] = __byte_perm(a0, a1, 0x7531) ^ 0x80808080u;
        }
    }
    if constexpr (FMT == Q4_K || FMT == Q5_K) {
        // sc * v  =  (1024 + v) * sc - 1024 * sc
        const __half2 sc = __half2half2(__ushort2half_rn((unsigned short)(sm & 0xFFu)));
        const __half2 nb = __hmul2(sc, __half2half2(__float2half(-1024.0f)));
        out[0][0] = kc_block(lo[0], lo[1], sc, nb);
        out[0][1] = kc_block(lo[2], lo[3], sc, nb);
        out[0][2] = kc_block(hi[0], hi[1], sc, nb);
        out[0][3] = kc_block(hi[2], hi[3], sc, nb);
    } else if constexpr (FMT == Q6_K) {
        // (v - 32) * sc  =  (v - 32) * 2*(sc >> 1)  +  (v - 32) * (sc & 1), per 16-weight half
        const int s_lo = (int)(int8_t)(sm & 0xFFu), s_hi = (int)(int8_t)(sm >> 8);
        const __half2 one = __half2half2(__float2half(1.0f)), off = __half2half2(__float2half(-1056.0f));
        const __half2 x_lo = __half2half2(__int2half_rn(2 * (s_lo >> 1))), y_lo = __half2half2(__int2half_rn(s_lo & 1));
        const __half2 x_hi = __half2half2(__int2half_rn(2 * (s_hi >> 1))), y_hi = __half2half2(__int2half_rn(s_hi & 1));
        const __half2 zero = __half2half2(__float2half(0.0f));
        const uint4 u0 = kc_block(lo[0], lo[1], one, off), u1 = kc_block(lo[2], lo[3], one, off); // v - 32
        const uint4 u2 = kc_block(hi[0], hi[1], one, off), u3 = kc_block(hi[2], hi[3], one, off);
        auto scale = [&](const uint4 &u, __half2 s) {
            return make_uint4(h2_as_u32(__hfma2(u32_as_h2(u.x), s, zero)), h2_as_u32(__hfma2(u32_as_h2(u.y), s, zero)),
                              h2_as_u32(__hfma2(u32_as_h2(u.z), s, zero)), h2_as_u32(__hfma2(u32_as_h2(u.w), s, zero)));
        };
        out[0][0] = scale(u0, x_lo); out[0][1] = scale(u1, x_lo); out[0][2] = scale(u2, x_hi); out[0][3] = scale(u3, x_hi);
        out[1][0] = scale(u0, y_lo); out[1][1] = scale(u1, y_lo); out[1][2] = scale(u2, y_hi); out[1][3] = scale(u3, y_hi);
    } else {
        const float bias = (FMT == Q4_0) ? -1032.0f : (FMT == Q5_1) ? -1024.0f : -1152.0f; // remove 1024 and the format's offset (8, none, or 128)
        const __half2 one = __half2half2(__float2half(1.0f)), off = __half2half2(__float2half(bias));
        out[0][0] = kc_block(lo[0], lo[1], one, off);
        out[0][1] = kc_block(lo[2], lo[3], one, off);
        out[0][2] = kc_block(hi[0], hi[1], one, off);
        out[0][3] = kc_block(hi[2], hi[3], one, off);
    }
}

} // namespace rc
