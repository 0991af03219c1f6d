// Fused dequant+dot matvec over repacked-v2 weights, for 1..16 activation rows.
//
// What is computed (per weight row r, activation row b, 32-wide sub-block s) follows the
// per-lane bodies of the reference's kernels:
//   Q4_K   kernels/matvec_q4k_repacked.cpp:105-122    dsc*dx*idot - deff*xsum
//   Q5_K   kernels/matvec_q5k_repacked.cpp:79-96      same, 5th bit OR-ed into the nibbles
//   Q6_K   kernels/matvec_q6k_repacked.cpp:83-109     two 16-weight halves of (q-32)
//   Q8_0   kernels/matvec_q8_0_repacked.cpp:77-86     dw*dx*idot
//   Q4_0   kernels/matvec_q4_0_repacked.cpp:84-111    dw*dx*(idot - 8*sum(xq))
//   IQ4_XS kernels/matvec_iq4xs_repacked.cpp:104-116  dw*dx*sum(LUT[q]*xq)
// and of their _batched forms (kernels/matvec_q4k_repacked_batched.cpp:107-126).
//
// How it runs on B200 is not the reference's Wave64 scheme.  The kernel is HBM-bound, so
// the design is about bytes in flight: a CTA stages the BlockQ8 activations once into
// shared memory in planar form (two 16-byte halves, scale/sum pair, integer half sums), then
// each warp streams whole weight rows with 128-bit non-allocating loads — lane l owns
// sub-blocks l, l+32, ... of the row, so one warp instruction reads 512 contiguous bytes of
// the nibble plane — issues every plane load of ROWS rows before the first dot, and reduces
// with five shuffles per output.  CTAs are persistent over row groups.
#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {

namespace {

// Staged activations: [n_rows][chunk] arrays, sub-block index fastest, so a warp's reads
// are conflict-free 16-byte (or 8-byte) rows.
struct XStage {
    int4 *lo, *hi;
    float2 *ds;
    int2 *is;
};

__device__ __forceinline__ XStage carve_stage(uint8_t *smem, uint32_t n_rows, uint32_t chunk)
{
    XStage s;
    const size_t n = (size_t)n_rows * chunk;
    s.lo = reinterpret_cast<int4 *>(smem);
    s.hi = s.lo + n;
    s.ds = reinterpret_cast<float2 *>(s.hi + n);
    s.is = reinterpret_cast<int2 *>(s.ds + n);
    return s;
}

constexpr size_t kStageBytesPerBlock = 16 + 16 + 8 + 8;
constexpr size_t kMaxStageBytesHost = 200 * 1024;

// Weight registers of one (row, sub-block) and the math on them -----------------------------

template <int FMT> struct WBlk;

// Weight-plane loads: SM = false streams from global memory (non-allocating), SM = true
// reads the copy a bulk-async stage holds in shared memory.
template <bool SM> __device__ __forceinline__ uint4 ldw_u4(const uint8_t *p)
{
    if (SM) return *reinterpret_cast<const uint4 *>(p);
    return ld_stream_u4(p);
}
template <bool SM> __device__ __forceinline__ uint2 ldw_u2(const uint8_t *p)
{
    if (SM) return *reinterpret_cast<const uint2 *>(p);
    return ld_stream_u2(p);
}
template <bool SM> __device__ __forceinline__ uint32_t ldw_u32(const uint8_t *p)
{
    if (SM) return *reinterpret_cast<const uint32_t *>(p);
    return ld_stream_u32(p);
}
template <bool SM> __device__ __forceinline__ uint32_t ldw_u16(const uint8_t *p)
{
    if (SM) return (uint32_t)*reinterpret_cast<const unsigned short *>(p);
    return ld_nc_u16(p);
}
// d|dmin word of a superblock; in global memory its plane base may be only 2-byte aligned
template <bool SM> __device__ __forceinline__ uint32_t ld_sup32(const uint8_t *p, bool aligned4)
{
    if (SM) return *reinterpret_cast<const uint32_t *>(p);
    if (aligned4) return __ldg(reinterpret_cast<const uint32_t *>(p));
    return ld_nc_u16(p) | (ld_nc_u16(p + 2) << 16);
}

__device__ __forceinline__ int dot_nibbles(const uint4 &q, const int4 &lo, const int4 &hi)
{
    const uint32_t M = 0x0F0F0F0Fu;
    int a = 0;
    a = __dp4a((int)(q.x & M), lo.x, a);
    a = __dp4a((int)((q.x >> 4) & M), hi.x, a);
    a = __dp4a((int)(q.y & M), lo.y, a);
    a = __dp4a((int)((q.y >> 4) & M), hi.y, a);
    a = __dp4a((int)(q.z & M), lo.z, a);
    a = __dp4a((int)((q.z >> 4) & M), hi.z, a);
    a = __dp4a((int)(q.w & M), lo.w, a);
    a = __dp4a((int)((q.w >> 4) & M), hi.w, a);
    return a;
}

template <> struct WBlk<Q4_K> {
    uint4 q;
    float dsc, deff;
    template <bool SM> __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t sup, bool a4)
    {
        q = ldw_u4<SM>(p.nib + idx * 16);
        const uint32_t sm = ldw_u16<SM>(p.sc + idx * 2);
        const uint32_t dd = ld_sup32<SM>(p.sup + sup * 4, a4);
        dsc = f16_bits_to_f32(dd) * (float)(sm & 0xFFu);
        deff = f16_bits_to_f32(dd >> 16) * (float)(sm >> 8);
    }
    __device__ __forceinline__ float term(const int4 &lo, const int4 &hi, float2 ds, int2,
                                          int &i0, int &i1) const
    {
        i0 = dot_nibbles(q, lo, hi);
        i1 = 0;
        return dsc * ds.x * (float)i0 - deff * ds.y;
    }
};

template <> struct WBlk<Q5_K> {
    uint4 lo4, hi4; // the eight expanded 5-bit words: lo4 = weights 0..15, hi4 = 16..31
    float dsc, deff;
    template <bool SM> __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t sup, bool a4)
    {
        const uint4 q = ldw_u4<SM>(p.nib + idx * 16);
        const uint32_t qh = ldw_u32<SM>(p.aux + idx * 4);
        const uint32_t sm = ldw_u16<SM>(p.sc + idx * 2);
        const uint32_t dd = ld_sup32<SM>(p.sup + sup * 4, a4);
        const uint32_t M = 0x0F0F0F0Fu;
        // bit 4g+c of qh is the 5th bit of weight c of group g; group 2j pairs with the
        // low nibbles of word j, group 2j+1 with the high nibbles (src/quant/q5_k.rs:134-137)
        lo4.x = (q.x & M) | bits4_to_bit4(qh);
        hi4.x = ((q.x >> 4) & M) | bits4_to_bit4(qh >> 4);
        lo4.y = (q.y & M) | bits4_to_bit4(qh >> 8);
        hi4.y = ((q.y >> 4) & M) | bits4_to_bit4(qh >> 12);
        lo4.z = (q.z & M) | bits4_to_bit4(qh >> 16);
        hi4.z = ((q.z >> 4) & M) | bits4_to_bit4(qh >> 20);
        lo4.w = (q.w & M) | bits4_to_bit4(qh >> 24);
        hi4.w = ((q.w >> 4) & M) | bits4_to_bit4(qh >> 28);
        dsc = f16_bits_to_f32(dd) * (float)(sm & 0xFFu);
        deff = f16_bits_to_f32(dd >> 16) * (float)(sm >> 8);
    }
    __device__ __forceinline__ float term(const int4 &lo, const int4 &hi, float2 ds, int2,
                                          int &i0, int &i1) const
    {
        int a = 0;
        a = __dp4a((int)lo4.x, lo.x, a);
        a = __dp4a((int)hi4.x, hi.x, a);
        a = __dp4a((int)lo4.y, lo.y, a);
        a = __dp4a((int)hi4.y, hi.y, a);
        a = __dp4a((int)lo4.z, lo.z, a);
        a = __dp4a((int)hi4.z, hi.z, a);
        a = __dp4a((int)lo4.w, lo.w, a);
        a = __dp4a((int)hi4.w, hi.w, a);
        i0 = a;
        i1 = 0;
        return dsc * ds.x * (float)a - deff * ds.y;
    }
};

template <> struct WBlk<Q6_K> {
    uint4 lo6, hi6; // expanded 6-bit words, unsigned 0..63
    float dlo, dhi;
    template <bool SM> __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t sup, bool)
    {
        const uint4 q = ldw_u4<SM>(p.nib + idx * 16);
        const uint2 h = ldw_u2<SM>(p.aux + idx * 8);
        const uint32_t sm = ldw_u16<SM>(p.sc + idx * 2);
        const float d = f16_bits_to_f32(ldw_u16<SM>(p.sup + sup * 2));
        const uint32_t M = 0x0F0F0F0Fu;
        // byte g of the high-2 plane belongs to group g (src/quant/q6_k.rs:128-133)
        lo6.x = (q.x & M) | fields2_to_bits45(h.x & 0xFFu);
        hi6.x = ((q.x >> 4) & M) | fields2_to_bits45((h.x >> 8) & 0xFFu);
        lo6.y = (q.y & M) | fields2_to_bits45((h.x >> 16) & 0xFFu);
        hi6.y = ((q.y >> 4) & M) | fields2_to_bits45(h.x >> 24);
        lo6.z = (q.z & M) | fields2_to_bits45(h.y & 0xFFu);
        hi6.z = ((q.z >> 4) & M) | fields2_to_bits45((h.y >> 8) & 0xFFu);
        lo6.w = (q.w & M) | fields2_to_bits45((h.y >> 16) & 0xFFu);
        hi6.w = ((q.w >> 4) & M) | fields2_to_bits45(h.y >> 24);
        dlo = d * (float)(int)(int8_t)(sm & 0xFFu);
        dhi = d * (float)(int)(int8_t)(sm >> 8);
    }
    __device__ __forceinline__ float term(const int4 &lo, const int4 &hi, float2 ds, int2 is,
                                          int &i0, int &i1) const
    {
        int a = 0, b = 0;
        a = __dp4a((int)lo6.x, lo.x, a);
        b = __dp4a((int)hi6.x, hi.x, b);
        a = __dp4a((int)lo6.y, lo.y, a);
        b = __dp4a((int)hi6.y, hi.y, b);
        a = __dp4a((int)lo6.z, lo.z, a);
        b = __dp4a((int)hi6.z, hi.z, b);
        a = __dp4a((int)lo6.w, lo.w, a);
        b = __dp4a((int)hi6.w, hi.w, b);
        i0 = a - 32 * is.x;
        i1 = b - 32 * is.y;
        return dlo * ds.x * (float)i0 + dhi * ds.x * (float)i1;
    }
};

template <> struct WBlk<Q8_0> {
    uint4 wl, wh;
    float dw;
    template <bool SM> __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t, bool)
    {
        wl = ldw_u4<SM>(p.nib + idx * 16);
        wh = ldw_u4<SM>(p.aux + idx * 16);
        dw = f16_bits_to_f32(ldw_u16<SM>(p.sc + idx * 2));
    }
    __device__ __forceinline__ float term(const int4 &lo, const int4 &hi, float2 ds, int2,
                                          int &i0, int &i1) const
    {
        int a = 0;
        a = __dp4a((int)wl.x, lo.x, a);
        a = __dp4a((int)wl.y, lo.y, a);
        a = __dp4a((int)wl.z, lo.z, a);
        a = __dp4a((int)wl.w, lo.w, a);
        a = __dp4a((int)wh.x, hi.x, a);
        a = __dp4a((int)wh.y, hi.y, a);
        a = __dp4a((int)wh.z, hi.z, a);
        a = __dp4a((int)wh.w, hi.w, a);
        i0 = a;
        i1 = 0;
        return dw * ds.x * (float)a;
    }
};

template <> struct WBlk<Q4_0> {
    uint4 q;
    float dw;
    template <bool SM> __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t, bool)
    {
        q = ldw_u4<SM>(p.nib + idx * 16);
        dw = f16_bits_to_f32(ldw_u16<SM>(p.sc + idx * 2));
    }
    __device__ __forceinline__ float term(const int4 &lo, const int4 &hi, float2 ds, int2 is,
                                          int &i0, int &i1) const
    {
        i0 = dot_nibbles(q, lo, hi) - 8 * (is.x + is.y);
        i1 = 0;
        return dw * ds.x * (float)i0;
    }
};

template <> struct WBlk<IQ4_XS> {
    int4 a, b; // codebook values in iq4_lookup8 order: a = words 0,1; b = words 2,3
    float dw;
    template <bool SM> __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t, bool)
    {
        const uint4 q = ldw_u4<SM>(p.nib + idx * 16);
        dw = f16_bits_to_f32(ldw_u16<SM>(p.sc + idx * 2));
        iq4_lookup8(q.x, a.x, a.y);
        iq4_lookup8(q.y, a.z, a.w);
        iq4_lookup8(q.z, b.x, b.y);
        iq4_lookup8(q.w, b.z, b.w);
    }
    // lo/hi hold the activations already permuted by xperm_iq4 at staging time.
    __device__ __forceinline__ float term(const int4 &lo, const int4 &hi, float2 ds, int2,
                                          int &i0, int &i1) const
    {
        int s = 0;
        s = __dp4a(a.x, lo.x, s);
        s = __dp4a(a.y, lo.y, s);
        s = __dp4a(a.z, lo.z, s);
        s = __dp4a(a.w, lo.w, s);
        s = __dp4a(b.x, hi.x, s);
        s = __dp4a(b.y, hi.y, s);
        s = __dp4a(b.z, hi.z, s);
        s = __dp4a(b.w, hi.w, s);
        i0 = s;
        i1 = 0;
        return dw * ds.x * (float)s;
    }
};

// --------------------------------------------------------------------------------------------

// NB    compile-time bound on activation rows (n_rows <= NB)
// ROWS  weight rows a warp streams together
// DUMP  also write the per-block integers (debug entry point)
template <int FMT, int NB, int ROWS, bool DUMP>
__device__ __forceinline__ void
matvec_body(uint8_t *smem, const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq,
            float *__restrict__ y, int32_t *__restrict__ idots, uint32_t in_dim, uint32_t out_dim,
            uint32_t n_rows, uint32_t group_begin, uint32_t group_stride)
{
    const uint32_t n_sub = in_dim >> 5;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const Planes p = planes_of<FMT>(w, in_dim, out_dim);
    const bool sup_a4 = (reinterpret_cast<uintptr_t>(p.sup) & 3u) == 0;
    const XStage st = carve_stage(smem, n_rows, n_sub);

    // Stage every activation block once per CTA.
    for (uint32_t i = threadIdx.x; i < n_rows * n_sub; i += blockDim.x) {
        XBlock x = load_blockq8(xq + (size_t)i * RC_BLOCKQ8_BYTES);
        if (FMT == IQ4_XS) {
            int4 a, b;
            xperm_iq4(x.lo.x, x.hi.x, a.x, a.y);
            xperm_iq4(x.lo.y, x.hi.y, a.z, a.w);
            xperm_iq4(x.lo.z, x.hi.z, b.x, b.y);
            xperm_iq4(x.lo.w, x.hi.w, b.z, b.w);
            x.lo = a;
            x.hi = b;
        }
        st.lo[i] = x.lo;
        st.hi[i] = x.hi;
        st.ds[i] = make_float2(x.d, x.xsum);
        st.is[i] = make_int2(x.s_lo, x.s_hi);
    }
    __syncthreads();

    const uint32_t rows_per_cta = n_warps * ROWS;
    const uint32_t n_groups = (out_dim + rows_per_cta - 1) / rows_per_cta;
    for (uint32_t g = group_begin; g < n_groups; g += group_stride) {
        const uint32_t row0 = g * rows_per_cta + warp * ROWS;
        if (row0 >= out_dim) continue;
        float acc[ROWS][NB];
#pragma unroll
        for (int r = 0; r < ROWS; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = 0.0f;

        for (uint32_t sb = lane; sb < n_sub; sb += 32) {
            WBlk<FMT> wb[ROWS];
#pragma unroll
            for (int r = 0; r < ROWS; r++) {
                // rows past the end are clamped: their loads stay legal, their results unused
                const uint32_t row = min(row0 + r, out_dim - 1);
                wb[r].template load<false>(p, (size_t)row * p.nsp + sb, (size_t)row * p.n_super + (sb >> 3), sup_a4);
            }
#pragma unroll
            for (int b = 0; b < NB; b++) {
                if (b < (int)n_rows) {
                    const uint32_t xi = b * n_sub + sb;
                    const int4 lo = st.lo[xi], hi = st.hi[xi];
                    const float2 ds = st.ds[xi];
                    const int2 is = (FMT == Q6_K || FMT == Q4_0) ? st.is[xi] : make_int2(0, 0);
#pragma unroll
                    for (int r = 0; r < ROWS; r++) {
                        int i0, i1;
                        acc[r][b] += wb[r].term(lo, hi, ds, is, i0, i1);
                        if (DUMP && row0 + r < out_dim) {
                            int32_t *o = idots + (((size_t)b * out_dim + row0 + r) * n_sub + sb) * 2;
                            o[0] = i0;
                            o[1] = i1;
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float v = warp_sum(acc[r][b]);
                if (!DUMP && lane == 0 && b < (int)n_rows && row0 + r < out_dim)
                    y[(size_t)b * out_dim + row0 + r] = v;
            }
    }
}

template <int FMT, int NB, int ROWS, bool DUMP>
__global__ void __launch_bounds__(512)
matvec_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, float *__restrict__ y,
              int32_t *__restrict__ idots, uint32_t in_dim, uint32_t out_dim, uint32_t n_rows)
{
    extern __shared__ __align__(16) uint8_t smem[];
    matvec_body<FMT, NB, ROWS, DUMP>(smem, w, xq, y, idots, in_dim, out_dim, n_rows, blockIdx.x,
                                     gridDim.x);
}

// Expert-grouped form: blockIdx.y is a global token tile, mapped to (expert, local tile) by
// binary search over tile_off as in kernels/mmq_gemm_q4k_grouped.cpp:49-60; the tile's rows
// of xq / y are contiguous in expert-sorted order.
template <int FMT, int BN>
__global__ void __launch_bounds__(512)
matvec_grouped_kernel(const uint8_t *__restrict__ slab, size_t bytes_per_expert,
                      const int32_t *__restrict__ expert_off, const int32_t *__restrict__ tile_off,
                      uint32_t n_expert, const uint8_t *__restrict__ xq, float *__restrict__ y,
                      uint32_t in_dim, uint32_t out_dim)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t by = blockIdx.y;
    if (by >= (uint32_t)tile_off[n_expert]) return; // over-launched tile
    uint32_t lo = 0, hi = n_expert;
    while (lo + 1 < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if ((uint32_t)tile_off[mid] <= by) lo = mid; else hi = mid;
    }
    const uint32_t e = lo;
    const uint32_t tok0 = (uint32_t)expert_off[e] + (by - (uint32_t)tile_off[e]) * BN;
    const uint32_t n = min((uint32_t)BN, (uint32_t)expert_off[e + 1] - tok0);
    const uint32_t n_sub = in_dim >> 5;
    matvec_body<FMT, BN, 1, false>(smem, slab + (size_t)e * bytes_per_expert,
                                   xq + (size_t)tok0 * n_sub * RC_BLOCKQ8_BYTES,
                                   y + (size_t)tok0 * out_dim, nullptr, in_dim, out_dim, n,
                                   blockIdx.x, gridDim.x);
}


// ---------------------------------------------------------------------------------------------
// Bulk-async pipelined form (the decode fast path).
//
// A persistent CTA owns groups of R consecutive weight rows.  For R a multiple of 8 and
// out_dim a multiple of 8, the R rows' share of every plane is one contiguous, 16-byte aligned
// run of bytes, so a group is fetched by one cp.async.bulk per plane into a ring of shared
// memory stages, completion counted on an mbarrier.  One elected producer thread keeps every
// free stage in flight — the bytes in flight are bounded by shared memory (~190 KB per SM),
// not by registers or occupancy, which is what an 8 us HBM-bound kernel needs.  Consumer
// warps take one row each from a full stage, dot it against the staged activations and
// release the stage.  Every wait is bounded: after kSpinLimit polls the kernel records an
// error in g_pipe_error and returns (the context stays usable, the output is invalid).

constexpr uint32_t kSpinLimit = 1u << 22; // ~4M polls with back-off, far beyond any legal wait
__device__ unsigned int g_pipe_error;

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < kSpinLimit; spin++) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done)
                     : "r"(addr), "r"(parity)
                     : "memory");
        if (done) return true;
        if (spin > 64) __nanosleep(32);
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Bytes of plane `k` (0 nib, 1 aux, 2 sc, 3 sup) per weight row.
template <int FMT> __host__ __device__ inline uint32_t plane_row_bytes(int k, uint32_t nsp, uint32_t n_super)
{
    switch (k) {
    case 0: return nsp * 16;
    case 1: return FMT == Q5_K ? nsp * 4 : FMT == Q6_K ? nsp * 8 : FMT == Q8_0 ? nsp * 16 : 0;
    case 2: return nsp * 2;
    default: return (FMT == Q4_K || FMT == Q5_K) ? n_super * 4 : FMT == Q6_K ? n_super * 2 : 0;
    }
}

template <int FMT> __host__ __device__ inline uint32_t row_bytes_all(uint32_t nsp, uint32_t n_super)
{
    return plane_row_bytes<FMT>(0, nsp, n_super) + plane_row_bytes<FMT>(1, nsp, n_super) +
           plane_row_bytes<FMT>(2, nsp, n_super) + plane_row_bytes<FMT>(3, nsp, n_super);
}

// smem: [x stage][pad to 128][S stages of R*row_bytes][full[S], empty[S] barriers]
template <int FMT, int NB>
__global__ void __launch_bounds__(544)
matvec_pipe_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, float *__restrict__ y,
                   uint32_t in_dim, uint32_t out_dim, uint32_t n_rows, uint32_t R, uint32_t S)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t n_sub = in_dim >> 5;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t n_cwarps = (blockDim.x >> 5) - 1; // the last warp is the producer
    const Planes gp = planes_of<FMT>(w, in_dim, out_dim);
    const uint32_t nsp = gp.nsp, n_super = gp.n_super;

    const size_t x_bytes = ((size_t)n_rows * n_sub * kStageBytesPerBlock + 127) & ~(size_t)127;
    const uint32_t rb[4] = {plane_row_bytes<FMT>(0, nsp, n_super), plane_row_bytes<FMT>(1, nsp, n_super),
                            plane_row_bytes<FMT>(2, nsp, n_super), plane_row_bytes<FMT>(3, nsp, n_super)};
    // plane offsets inside one stage; every plane's run of R rows is a multiple of 16 bytes
    const uint32_t off1 = R * rb[0], off2 = off1 + R * rb[1], off3 = off2 + R * rb[2];
    const uint32_t stage_bytes = (off3 + R * rb[3] + 127u) & ~127u;
    uint8_t *stages = smem + x_bytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(stages + (size_t)S * stage_bytes);
    uint64_t *empty = full + S;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; s++) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, n_cwarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const uint32_t n_groups = (out_dim + R - 1) / R;

    if (warp == n_cwarps) {
        // ---- producer: one thread keeps the ring full ----
        if (lane == 0) {
            const uint8_t *gbase[4] = {gp.nib, gp.aux, gp.sc, gp.sup};
            uint32_t it = 0;
            for (uint32_t g = blockIdx.x; g < n_groups; g += gridDim.x, it++) {
                const uint32_t s = it % S;
                if (it >= S && !mbar_wait(empty + s, ((it / S) - 1u) & 1u)) {
                    atomicExch(&g_pipe_error, 1u);
                    break;
                }
                const uint32_t r0 = g * R, nr = min(R, out_dim - r0);
                uint8_t *dst = stages + (size_t)s * stage_bytes;
                const uint32_t offs[4] = {0, off1, off2, off3};
                uint32_t total = 0;
#pragma unroll
                for (int k = 0; k < 4; k++) total += nr * rb[k];
                mbar_expect_tx(full + s, total);
#pragma unroll
                for (int k = 0; k < 4; k++)
                    if (rb[k]) bulk_g2s(dst + offs[k], gbase[k] + (size_t)r0 * rb[k], nr * rb[k], full + s);
            }
        }
        return;
    }

    // ---- consumers ----
    const uint32_t n_cthreads = n_cwarps * 32;
    const XStage st = carve_stage(smem, n_rows, n_sub);
    for (uint32_t i = threadIdx.x; i < n_rows * n_sub; i += n_cthreads) {
        XBlock x = load_blockq8(xq + (size_t)i * RC_BLOCKQ8_BYTES);
        if (FMT == IQ4_XS) {
            int4 a, b;
            xperm_iq4(x.lo.x, x.hi.x, a.x, a.y);
            xperm_iq4(x.lo.y, x.hi.y, a.z, a.w);
            xperm_iq4(x.lo.z, x.hi.z, b.x, b.y);
            xperm_iq4(x.lo.w, x.hi.w, b.z, b.w);
            x.lo = a;
            x.hi = b;
        }
        st.lo[i] = x.lo;
        st.hi[i] = x.hi;
        st.ds[i] = make_float2(x.d, x.xsum);
        st.is[i] = make_int2(x.s_lo, x.s_hi);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(n_cthreads) : "memory");

    uint32_t it = 0;
    for (uint32_t g = blockIdx.x; g < n_groups; g += gridDim.x, it++) {
        const uint32_t s = it % S;
        if (!mbar_wait(full + s, (it / S) & 1u)) {
            atomicExch(&g_pipe_error, 2u);
            return;
        }
        const uint8_t *sb_base = stages + (size_t)s * stage_bytes;
        Planes sp;
        sp.nib = sb_base;
        sp.aux = sb_base + off1;
        sp.sc = sb_base + off2;
        sp.sup = sb_base + off3;
        sp.nsp = nsp;
        sp.n_super = n_super;
        const uint32_t r0 = g * R, nr = min(R, out_dim - r0);
        for (uint32_t r = warp; r < nr; r += n_cwarps) {
            float acc[NB];
#pragma unroll
            for (int b = 0; b < NB; b++) acc[b] = 0.0f;
#pragma unroll 5
            for (uint32_t sb = lane; sb < n_sub; sb += 32) {
                WBlk<FMT> wb;
                wb.template load<true>(sp, (size_t)r * nsp + sb, (size_t)r * n_super + (sb >> 3), true);
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    if (b < (int)n_rows) {
                        const uint32_t xi = b * n_sub + sb;
                        const int2 is = (FMT == Q6_K || FMT == Q4_0) ? st.is[xi] : make_int2(0, 0);
                        int i0, i1;
                        acc[b] += wb.term(st.lo[xi], st.hi[xi], st.ds[xi], is, i0, i1);
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float v = warp_sum(acc[b]);
                if (lane == 0 && b < (int)n_rows) y[(size_t)b * out_dim + r0 + r] = v;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
    }
}

struct PipeTuning {
    int rows_per_stage = 0, stages = 0, cwarps = 0, ctas_per_sm = 0, disable = 0;
};
PipeTuning g_pipe;

template <int FMT, int NB>
int launch_pipe(cudaStream_t s, const void *w, const void *xq, float *y, uint32_t in_dim,
                uint32_t out_dim, uint32_t n_rows)
{
    const uint32_t n_sub = in_dim >> 5, nsp = nsp_of(n_sub), n_super = n_sub >> 3;
    const uint32_t rowb = row_bytes_all<FMT>(nsp, n_super);
    const size_t x_bytes = ((size_t)n_rows * n_sub * kStageBytesPerBlock + 127) & ~(size_t)127;
    const size_t budget = 208 * 1024;
    uint32_t ctas_per_sm = g_pipe.ctas_per_sm > 0 ? (uint32_t)g_pipe.ctas_per_sm : 1;
    const size_t per_cta = budget / ctas_per_sm;
    if (x_bytes + 2 * (size_t)8 * rowb + 256 > per_cta) return RC_ERR_TOO_MANY_ROWS; // caller uses the generic kernel
    uint32_t R = g_pipe.rows_per_stage > 0 ? ((uint32_t)g_pipe.rows_per_stage + 7u) & ~7u : 8;
    const uint32_t stage_bytes = (R * rowb + 127u) & ~127u;
    uint32_t S = (uint32_t)((per_cta - x_bytes - 256) / stage_bytes);
    if (g_pipe.stages > 0) S = min(S, (uint32_t)g_pipe.stages);
    S = min(S, 16u);
    if (S < 2) {
        R = 8;
        S = (uint32_t)((per_cta - x_bytes - 256) / ((8 * rowb + 127u) & ~127u));
        if (S < 2) return RC_ERR_TOO_MANY_ROWS;
    }
    const uint32_t cwarps = g_pipe.cwarps > 0 ? min((uint32_t)g_pipe.cwarps, 16u) : min(R, 16u);
    const uint32_t n_groups = (out_dim + R - 1) / R;
    const uint32_t grid = min(n_groups, (uint32_t)sm_count() * ctas_per_sm);
    const size_t smem = x_bytes + (size_t)S * ((R * rowb + 127u) & ~127u) + 2 * S * sizeof(uint64_t);
    matvec_pipe_kernel<FMT, NB><<<grid, (cwarps + 1) * 32, smem, s>>>(
        (const uint8_t *)w, (const uint8_t *)xq, y, in_dim, out_dim, n_rows, R, S);
    return (int)cudaGetLastError();
}

// The pipelined kernel needs every plane's per-group run to start on a 16-byte boundary.
inline bool pipe_eligible(const void *w, uint32_t out_dim, uint32_t n_rows)
{
    return !g_pipe.disable && out_dim % 8 == 0 && n_rows <= 4 && ((uintptr_t)w & 15u) == 0;
}

template <int FMT>
int launch_pipe_fmt(cudaStream_t s, const void *w, const void *xq, float *y, uint32_t in_dim,
                    uint32_t out_dim, uint32_t n_rows)
{
    if (n_rows == 1) return launch_pipe<FMT, 1>(s, w, xq, y, in_dim, out_dim, n_rows);
    if (n_rows == 2) return launch_pipe<FMT, 2>(s, w, xq, y, in_dim, out_dim, n_rows);
    return launch_pipe<FMT, 4>(s, w, xq, y, in_dim, out_dim, n_rows);
}

template <int FMT> int set_attr_pipe()
{
    int rc = 0;
    rc |= (int)cudaFuncSetAttribute(matvec_pipe_kernel<FMT, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    rc |= (int)cudaFuncSetAttribute(matvec_pipe_kernel<FMT, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    rc |= (int)cudaFuncSetAttribute(matvec_pipe_kernel<FMT, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    return rc;
}

struct Tuning {
    int rows = 0;     // 0 = heuristic
    int threads = 0;  // 0 = heuristic
    int ctas_per_sm = 0;
};
Tuning g_tune;

template <int FMT, int NB, int ROWS, bool DUMP>
int launch_one(cudaStream_t s, const void *w, const void *xq, float *y, int32_t *idots,
               uint32_t in_dim, uint32_t out_dim, uint32_t n_rows, uint32_t threads, size_t smem)
{
    auto kern = matvec_kernel<FMT, NB, ROWS, DUMP>;
    const uint32_t rows_per_cta = (threads / 32) * ROWS;
    const uint32_t n_groups = (out_dim + rows_per_cta - 1) / rows_per_cta;
    uint32_t per_sm = 2048 / threads;
    if (smem) per_sm = min(per_sm, (uint32_t)((227 * 1024) / (smem + 1024)));
    if (per_sm == 0) per_sm = 1;
    if (g_tune.ctas_per_sm > 0) per_sm = (uint32_t)g_tune.ctas_per_sm;
    const uint32_t grid = min(n_groups, (uint32_t)sm_count() * per_sm);
    kern<<<grid, threads, smem, s>>>((const uint8_t *)w, (const uint8_t *)xq, y, idots, in_dim,
                                     out_dim, n_rows);
    return (int)cudaGetLastError();
}

template <int FMT, bool DUMP>
int launch_fmt(cudaStream_t s, const void *w, const void *xq, float *y, int32_t *idots,
               uint32_t in_dim, uint32_t out_dim, uint32_t n_rows)
{
    const uint32_t n_sub = in_dim >> 5;
    const size_t smem = (size_t)n_rows * n_sub * kStageBytesPerBlock;
    if (smem > kMaxStageBytesHost) return RC_ERR_TOO_MANY_ROWS; // caller splits the batch
    uint32_t threads = smem > 96 * 1024 ? 512 : 256;
    if (g_tune.threads > 0) threads = (uint32_t)g_tune.threads;
    int rows = (n_rows <= 2 && out_dim >= 8192) ? 2 : 1;
    if (g_tune.rows > 0) rows = g_tune.rows;
    if (DUMP) rows = 1;
#define RC_GO(NB, ROWS) \
    return launch_one<FMT, NB, ROWS, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows, threads, smem)
#define RC_GO_MULTI(NB, ROWS) \
    if (!DUMP) return launch_one<FMT, NB, ROWS, false>(s, w, xq, y, idots, in_dim, out_dim, n_rows, threads, smem)
    if (n_rows == 1) {
        if (rows >= 4) RC_GO_MULTI(1, 4);
        if (rows == 2) RC_GO_MULTI(1, 2);
        RC_GO(1, 1);
    }
    if (n_rows == 2) {
        if (rows >= 2) RC_GO_MULTI(2, 2);
        RC_GO(2, 1);
    }
    if (n_rows <= 4) {
        if (rows >= 2) RC_GO_MULTI(4, 2);
        RC_GO(4, 1);
    }
    if (n_rows <= 8) RC_GO(8, 1);
    RC_GO(16, 1);
#undef RC_GO
#undef RC_GO_MULTI
}

template <bool DUMP>
int launch_any(cudaStream_t s, int type, const void *w, const void *xq, float *y, int32_t *idots,
               uint32_t in_dim, uint32_t out_dim, uint32_t n_rows)
{
    if (!DUMP && pipe_eligible(w, out_dim, n_rows)) {
        int rc = RC_ERR_BAD_TYPE;
        switch (type) {
        case Q4_0: rc = launch_pipe_fmt<Q4_0>(s, w, xq, y, in_dim, out_dim, n_rows); break;
        case Q8_0: rc = launch_pipe_fmt<Q8_0>(s, w, xq, y, in_dim, out_dim, n_rows); break;
        case Q4_K: rc = launch_pipe_fmt<Q4_K>(s, w, xq, y, in_dim, out_dim, n_rows); break;
        case Q5_K: rc = launch_pipe_fmt<Q5_K>(s, w, xq, y, in_dim, out_dim, n_rows); break;
        case Q6_K: rc = launch_pipe_fmt<Q6_K>(s, w, xq, y, in_dim, out_dim, n_rows); break;
        case IQ4_XS: rc = launch_pipe_fmt<IQ4_XS>(s, w, xq, y, in_dim, out_dim, n_rows); break;
        }
        if (rc != RC_ERR_TOO_MANY_ROWS) return rc; // rows too long for the stage ring: generic kernel
    }
    switch (type) {
    case Q4_0: return launch_fmt<Q4_0, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case Q8_0: return launch_fmt<Q8_0, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case Q4_K: return launch_fmt<Q4_K, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case Q5_K: return launch_fmt<Q5_K, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case Q6_K: return launch_fmt<Q6_K, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case IQ4_XS: return launch_fmt<IQ4_XS, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    }
    return RC_ERR_BAD_TYPE;
}

} // namespace

namespace {

constexpr int kMaxStageBytes = 200 * 1024;

template <int FMT, int NB, int ROWS, bool DUMP> int set_attr_one()
{
    return (int)cudaFuncSetAttribute(matvec_kernel<FMT, NB, ROWS, DUMP>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxStageBytes);
}

template <int FMT> int set_attr_fmt()
{
    int rc = 0;
    rc |= set_attr_one<FMT, 1, 1, false>();
    rc |= set_attr_one<FMT, 1, 2, false>();
    rc |= set_attr_one<FMT, 1, 4, false>();
    rc |= set_attr_one<FMT, 2, 1, false>();
    rc |= set_attr_one<FMT, 2, 2, false>();
    rc |= set_attr_one<FMT, 4, 1, false>();
    rc |= set_attr_one<FMT, 4, 2, false>();
    rc |= set_attr_one<FMT, 8, 1, false>();
    rc |= set_attr_one<FMT, 16, 1, false>();
    rc |= set_attr_one<FMT, 1, 1, true>();
    rc |= set_attr_one<FMT, 2, 1, true>();
    rc |= set_attr_one<FMT, 4, 1, true>();
    rc |= set_attr_one<FMT, 8, 1, true>();
    rc |= set_attr_one<FMT, 16, 1, true>();
    return rc;
}

} // namespace

int matvec_set_attributes()
{
    int rc = 0;
    rc |= set_attr_fmt<Q4_0>();
    rc |= set_attr_fmt<Q8_0>();
    rc |= set_attr_fmt<Q4_K>();
    rc |= set_attr_fmt<Q5_K>();
    rc |= set_attr_fmt<Q6_K>();
    rc |= set_attr_fmt<IQ4_XS>();
    rc |= set_attr_pipe<Q4_0>();
    rc |= set_attr_pipe<Q8_0>();
    rc |= set_attr_pipe<Q4_K>();
    rc |= set_attr_pipe<Q5_K>();
    rc |= set_attr_pipe<Q6_K>();
    rc |= set_attr_pipe<IQ4_XS>();
    return rc;
}

void matvec_set_pipe_tuning(int rows_per_stage, int stages, int cwarps, int ctas_per_sm, int disable)
{
    g_pipe.rows_per_stage = rows_per_stage;
    g_pipe.stages = stages;
    g_pipe.cwarps = cwarps;
    g_pipe.ctas_per_sm = ctas_per_sm;
    g_pipe.disable = disable;
}

int matvec_device_error(unsigned int *out)
{
    return (int)cudaMemcpyFromSymbol(out, g_pipe_error, sizeof(unsigned int));
}

namespace {
template <int FMT>
int launch_grouped_fmt(cudaStream_t s, const void *slab, size_t bpe, const int32_t *expert_off,
                       const int32_t *tile_off, uint32_t n_expert, const void *xq, float *y,
                       uint32_t in_dim, uint32_t out_dim, uint32_t n_entries)
{
    constexpr int BN = 16;
    const uint32_t n_sub = in_dim >> 5;
    const size_t smem = (size_t)BN * n_sub * kStageBytesPerBlock;
    if (smem > kMaxStageBytesHost) return RC_ERR_BAD_SHAPE;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(matvec_grouped_kernel<FMT, BN>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kMaxStageBytesHost);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    const uint32_t threads = 256;
    const uint32_t n_groups = (out_dim + 7) / 8;
    const uint32_t gx = min(n_groups, 8u);
    const uint32_t tiles_ub = (n_entries + BN - 1) / BN + n_expert;
    if (tiles_ub > 65535u) return RC_ERR_BAD_ARGUMENT;
    matvec_grouped_kernel<FMT, BN><<<dim3(gx, tiles_ub), threads, smem, s>>>(
        (const uint8_t *)slab, bpe, expert_off, tile_off, n_expert, (const uint8_t *)xq, y, in_dim,
        out_dim);
    return (int)cudaGetLastError();
}
} // namespace

// dp4a grouped GEMM with a 16-token tile: every tile streams its expert's weights once.
int launch_matvec_grouped(cudaStream_t s, int type, const void *slab, size_t bpe,
                          const int32_t *expert_off, const int32_t *tile_off, uint32_t n_expert,
                          const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
                          uint32_t n_entries)
{
#define RC_G(F) return launch_grouped_fmt<F>(s, slab, bpe, expert_off, tile_off, n_expert, xq, y, in_dim, out_dim, n_entries)
    switch (type) {
    case Q4_0: RC_G(Q4_0);
    case Q8_0: RC_G(Q8_0);
    case Q4_K: RC_G(Q4_K);
    case Q5_K: RC_G(Q5_K);
    case Q6_K: RC_G(Q6_K);
    case IQ4_XS: RC_G(IQ4_XS);
    }
#undef RC_G
    return RC_ERR_BAD_TYPE;
}

void matvec_set_tuning(int rows, int threads, int ctas_per_sm)
{
    g_tune.rows = rows;
    g_tune.threads = threads;
    g_tune.ctas_per_sm = ctas_per_sm;
}

int launch_matvec(cudaStream_t s, int type, const void *w, const void *xq, float *y,
                  uint32_t in_dim, uint32_t out_dim, uint32_t n_rows, int32_t *idots)
{
    // Split the batch when the staged activations of all rows do not fit in shared memory;
    // each part reads the weights once more, which only very long rows ever need.
    uint32_t part = n_rows;
    const uint32_t n_sub = in_dim >> 5;
    while (part > 1 && (size_t)part * n_sub * kStageBytesPerBlock > kMaxStageBytesHost) part = (part + 1) / 2;
    if ((size_t)part * n_sub * kStageBytesPerBlock > kMaxStageBytesHost) return RC_ERR_BAD_SHAPE;
    for (uint32_t b0 = 0; b0 < n_rows; b0 += part) {
        const uint32_t nb = min(part, n_rows - b0);
        const uint8_t *xp = (const uint8_t *)xq + (size_t)b0 * n_sub * RC_BLOCKQ8_BYTES;
        float *yp = y ? y + (size_t)b0 * out_dim : nullptr;
        int rc;
        if (idots)
            rc = launch_any<true>(s, type, w, xp, yp, idots + (size_t)b0 * out_dim * n_sub * 2,
                                  in_dim, out_dim, nb);
        else
            rc = launch_any<false>(s, type, w, xp, yp, nullptr, in_dim, out_dim, nb);
        if (rc) return rc;
    }
    return RC_OK;
}

} // namespace rc
