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
// and of their _batched forms (kernels/matvec_q4k_repacked_batched.cpp:107-126).  The
// per-block integers are formed exactly as there; the f32 factors are associated slightly
// differently (one rounding of d*dx, one of (float)(sc*idot)), far inside the 1e-3 bound.
//
// How it runs on B200 is not the reference's Wave64 scheme.  The kernel is HBM-bound and
// lasts a few microseconds, so the design is about bytes in flight and about starting early:
//   - a CTA is 8 warps arranged as RB weight rows x KS splits of the row ("split-K" across
//     warps, chosen on the host so that short-and-wide and long-and-narrow matrices both give
//     every SM several waves of work); CTAs are persistent over row blocks;
//   - lane l owns sub-blocks l, l+32, ... so one warp instruction reads 512 contiguous bytes
//     of the nibble plane with 128-bit non-allocating loads; a warp issues the plane loads of
//     a whole group of G such iterations into registers (2.5 KB and more in flight per warp, 32
//     warps per SM) before the first dot, and issues the next group's loads before it reduces
//     the finished one;
//   - the first group's weight loads are issued before the activations are staged: weights
//     never depend on the preceding kernel, activations do;
//   - the BlockQ8 activations are staged once per CTA in shared memory in planar form (two
//     16-byte halves, pre-scaled scale/sum pair, integer half sums), so the inner loop reads
//     them with conflict-free 128-bit loads.
// A shared-memory ring filled by cp.async.bulk with a producer warp was built and measured
// first: 12.3 us on the 5120->17408 Q4_K matrix against 9.9 us for this form (a plain read of
// the same bytes takes 8.7 us), so the ring is not used.
#include <algorithm>
#include <cstring>
#include <type_traits>

#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {

namespace {

constexpr size_t kMaxStageBytesHost = 200 * 1024;
constexpr int kWarpsPerCta = 8;

template <int FMT> struct FmtTraits {
    // integer half sums of the activation block are needed for the "-32" / "-8" offsets
    static constexpr bool needs_is = (FMT == Q6_K || FMT == Q4_0);
    static constexpr uint32_t x_bytes = needs_is ? 48 : 40; // staged bytes per activation block
    // iterations (32 sub-blocks each) whose raw weight registers a warp holds at once
    static constexpr int G = (FMT == Q8_0) ? 3 : (FMT == Q5_K || FMT == Q5_1 || FMT == Q6_K || kCodebook<FMT>) ? 4 : 5;
    // group lengths the plain row kernel is built for (longer groups of the wide formats spill)
    static constexpr int rows_max_len = (FMT == Q6_K) ? 3 : (FMT == Q8_0 || FMT == Q5_K || FMT == Q5_1) ? 4 : 5;
};

// Staged activations: [n_rows][n_sub] arrays, sub-block index fastest, so a warp's reads are
// conflict-free 16-byte (or 8-byte) rows.
struct XStage {
    int4 *lo, *hi;
    float2 *ds;
    int2 *is;
};

template <int FMT>
__device__ __forceinline__ XStage carve_stage(uint8_t *smem, uint32_t n_blocks)
{
    XStage s;
    s.lo = reinterpret_cast<int4 *>(smem);
    s.hi = s.lo + n_blocks;
    s.ds = reinterpret_cast<float2 *>(s.hi + n_blocks);
    s.is = reinterpret_cast<int2 *>(s.ds + n_blocks);
    return s;
}

// Stages n_blocks BlockQ8 blocks.  What is stored is arranged for the consumer math below:
//   Q4_K, Q4_0  ds.x = d/16 (their dots are formed 16x too large, see dot_nibbles16)
//   Q4_K, Q5_K  ds.y = -xsum (the min term is added with one FMA; Q5_1 adds +m * xsum, ds.y = xsum)
//   Q6_K        is = (32*sum(lo half), 32*sum(hi half));   Q4_0  is.x = 128*sum(all)
//   IQ4_XS, IQ3_S  quants permuted into iq4_lookup8 order
template <int FMT>
__device__ __forceinline__ void stage_block(const XStage &st, uint32_t i, XBlock x)
{
    if (kCodebook<FMT>) {
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
    const float dscale = (FMT == Q4_K || FMT == Q4_0) ? 0.0625f : 1.0f;
    const float ssign = (FMT == Q4_K || FMT == Q5_K) ? -1.0f : 1.0f;
    st.ds[i] = make_float2(x.d * dscale, x.xsum * ssign);
    if (FMT == Q6_K) st.is[i] = make_int2(32 * x.s_lo, 32 * x.s_hi);
    if (FMT == Q4_0) st.is[i] = make_int2(128 * (x.s_lo + x.s_hi), 0);
}

template <int FMT>
__device__ __forceinline__ void stage_x(const XStage &st, const uint8_t *__restrict__ xq, uint32_t n_blocks)
{
    for (uint32_t i = threadIdx.x; i < n_blocks; i += blockDim.x) stage_block<FMT>(st, i, load_blockq8(xq + (size_t)i * RC_BLOCKQ8_BYTES));
}

// ---- raw weight registers of one (row, sub-block) ---------------------------------------------
// fetch() only loads, so a warp can issue the loads of a whole group before any of them is used.

template <int FMT> struct Raw;
template <> struct Raw<Q4_K> { uint4 q; uint32_t sm, dd; };
template <> struct Raw<Q5_K> { uint4 q; uint32_t qh, sm, dd; };
template <> struct Raw<Q5_1> { uint4 q; uint32_t qh, dm; };
template <> struct Raw<Q6_K> { uint4 q; uint2 h; uint32_t sm, d; };
template <> struct Raw<Q8_0> { uint4 wl, wh; uint32_t d; };
template <> struct Raw<Q4_0> { uint4 q; uint32_t d; };
template <> struct Raw<IQ4_XS> { uint4 q; uint32_t d; };
template <> struct Raw<IQ3_S> { uint4 q; uint32_t d; };

// d|dmin word of a superblock; the plane base may be only 2-byte aligned
__device__ __forceinline__ uint32_t ld_sup32(const uint8_t *p, bool aligned4)
{
    if (aligned4) return __ldg(reinterpret_cast<const uint32_t *>(p));
    return ld_nc_u16(p) | (ld_nc_u16(p + 2) << 16);
}

template <int FMT>
__device__ __forceinline__ void fetch(Raw<FMT> &r, const Planes &p, size_t idx, size_t sup, bool a4)
{
    if constexpr (FMT == Q4_K) {
        r.q = ld_stream_u4(p.nib + idx * 16);
        r.sm = ld_nc_u16(p.sc + idx * 2);
        r.dd = ld_sup32(p.sup + sup * 4, a4);
    } else if constexpr (FMT == Q5_K) {
        r.q = ld_stream_u4(p.nib + idx * 16);
        r.qh = ld_stream_u32(p.aux + idx * 4);
        r.sm = ld_nc_u16(p.sc + idx * 2);
        r.dd = ld_sup32(p.sup + sup * 4, a4);
    } else if constexpr (FMT == Q5_1) {
        r.q = ld_stream_u4(p.nib + idx * 16);
        r.qh = ld_stream_u32(p.aux + idx * 4);
        r.dm = ld_stream_u32(p.sc + idx * 4);
    } else if constexpr (FMT == Q6_K) {
        r.q = ld_stream_u4(p.nib + idx * 16);
        r.h = ld_stream_u2(p.aux + idx * 8);
        r.sm = ld_nc_u16(p.sc + idx * 2);
        r.d = ld_nc_u16(p.sup + sup * 2);
    } else if constexpr (FMT == Q8_0) {
        r.wl = ld_stream_u4(p.nib + idx * 16);
        r.wh = ld_stream_u4(p.aux + idx * 16);
        r.d = ld_nc_u16(p.sc + idx * 2);
    } else {
        r.q = ld_stream_u4(p.nib + idx * 16);
        r.d = ld_nc_u16(p.sc + idx * 2);
    }
}

// The same loads from per-group base pointers (the lane's sub-block of the group's first
// iteration) plus the constant byte offsets of iteration i, so that an unrolled group costs one
// set of 64-bit address computations instead of one per load.  A4: the superblock plane is
// 4-byte aligned.
struct GroupPtrs {
    const uint8_t *nib, *aux, *sc, *sup;
};

template <int FMT, bool A4>
__device__ __forceinline__ void fetch_off(Raw<FMT> &r, const GroupPtrs &g, int i)
{
    if constexpr (FMT == Q4_K) {
        r.q = ld_stream_u4(g.nib + i * 512);
        r.sm = ld_nc_u16(g.sc + i * 64);
        r.dd = ld_sup32(g.sup + i * 16, A4);
    } else if constexpr (FMT == Q5_K) {
        r.q = ld_stream_u4(g.nib + i * 512);
        r.qh = ld_stream_u32(g.aux + i * 128);
        r.sm = ld_nc_u16(g.sc + i * 64);
        r.dd = ld_sup32(g.sup + i * 16, A4);
    } else if constexpr (FMT == Q5_1) {
        r.q = ld_stream_u4(g.nib + i * 512);
        r.qh = ld_stream_u32(g.aux + i * 128);
        r.dm = ld_stream_u32(g.sc + i * 128);
    } else if constexpr (FMT == Q6_K) {
        r.q = ld_stream_u4(g.nib + i * 512);
        r.h = ld_stream_u2(g.aux + i * 256);
        r.sm = ld_nc_u16(g.sc + i * 64);
        r.d = ld_nc_u16(g.sup + i * 8);
    } else if constexpr (FMT == Q8_0) {
        r.wl = ld_stream_u4(g.nib + i * 512);
        r.wh = ld_stream_u4(g.aux + i * 512);
        r.d = ld_nc_u16(g.sc + i * 64);
    } else {
        r.q = ld_stream_u4(g.nib + i * 512);
        r.d = ld_nc_u16(g.sc + i * 64);
    }
}

template <int FMT>
__device__ __forceinline__ GroupPtrs group_ptrs(const Planes &p, uint32_t row, uint32_t sb0)
{
    constexpr uint32_t aux_b = (FMT == Q5_K || FMT == Q5_1) ? 4 : FMT == Q6_K ? 8 : FMT == Q8_0 ? 16 : 0;
    constexpr uint32_t sc_b = FMT == Q5_1 ? 4 : 2;
    constexpr uint32_t sup_b = FMT == Q6_K ? 2 : 4;
    const size_t idx = (size_t)row * p.nsp + sb0;
    GroupPtrs g;
    g.nib = p.nib + idx * 16;
    g.aux = aux_b ? p.aux + idx * aux_b : nullptr;
    g.sc = p.sc + idx * sc_b;
    g.sup = (FMT == Q4_K || FMT == Q5_K || FMT == Q6_K) ? p.sup + ((size_t)row * p.n_super + (sb0 >> 3)) * sup_b : nullptr;
    return g;
}

// unsigned bytes x signed bytes
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// 16 x the dot of 32 unsigned nibbles with the activation quants: the high nibbles are used in
// place as unsigned bytes 16*nibble (one AND instead of shift + AND), the low-nibble dot is
// scaled by 16 once at the end.  Exact: |result| <= 16*32*15*127 < 2^20.
__device__ __forceinline__ int dot_nibbles16(const uint4 &q, const int4 &xl, const int4 &xh)
{
    const uint32_t M = 0x0F0F0F0Fu, H = 0xF0F0F0F0u;
    int lo = 0, hi = 0;
    lo = __dp4a((int)(q.x & M), xl.x, lo);
    hi = dp4a_us(q.x & H, xh.x, hi);
    lo = __dp4a((int)(q.y & M), xl.y, lo);
    hi = dp4a_us(q.y & H, xh.y, hi);
    lo = __dp4a((int)(q.z & M), xl.z, lo);
    hi = dp4a_us(q.z & H, xh.z, hi);
    lo = __dp4a((int)(q.w & M), xl.w, lo);
    hi = dp4a_us(q.w & H, xh.w, hi);
    return lo * 16 + hi;
}

// Exact float of an integer 0..255 without the conversion unit.
__device__ __forceinline__ float small_uint_to_float(uint32_t v)
{
    return __uint_as_float(0x4B000000u | v) - 8388608.0f;
}

// One (weight row, sub-block) against one activation block: the f32 term, and the block
// integers i0/i1 (i1 is the second 16-weight half, Q6_K only).
template <int FMT>
__device__ __forceinline__ float term(const Raw<FMT> &r, const int4 &xl, const int4 &xh, float2 ds,
                                      int2 is, int &i0, int &i1)
{
    const uint32_t M = 0x0F0F0F0Fu;
    i1 = 0;
    if constexpr (FMT == Q4_K) {
        const int idot16 = dot_nibbles16(r.q, xl, xh);
        i0 = idot16 >> 4;
        const float d = f16_bits_to_f32(r.dd), dmin = f16_bits_to_f32(r.dd >> 16);
        const int sc = (int)(r.sm & 0xFFu);
        float t = (d * ds.x) * (float)(sc * idot16);
        return fmaf(dmin * ds.y, small_uint_to_float(r.sm >> 8), t);
    } else if constexpr (FMT == Q5_K || FMT == Q5_1) {
        // bit 4g+c of qh is the 5th bit of weight c of group g; group 2j pairs with the low
        // nibbles of word j, group 2j+1 with the high nibbles (src/quant/q5_k.rs:134-137)
        const uint4 q = r.q;
        const uint32_t qh = r.qh;
        int s = 0, t = 0;
        s = __dp4a((int)((q.x & M) | bits4_to_bit4(qh)), xl.x, s);
        t = __dp4a((int)(((q.x >> 4) & M) | bits4_to_bit4(qh >> 4)), xh.x, t);
        s = __dp4a((int)((q.y & M) | bits4_to_bit4(qh >> 8)), xl.y, s);
        t = __dp4a((int)(((q.y >> 4) & M) | bits4_to_bit4(qh >> 12)), xh.y, t);
        s = __dp4a((int)((q.z & M) | bits4_to_bit4(qh >> 16)), xl.z, s);
        t = __dp4a((int)(((q.z >> 4) & M) | bits4_to_bit4(qh >> 20)), xh.z, t);
        s = __dp4a((int)((q.w & M) | bits4_to_bit4(qh >> 24)), xl.w, s);
        t = __dp4a((int)(((q.w >> 4) & M) | bits4_to_bit4(qh >> 28)), xh.w, t);
        i0 = s + t;
        if constexpr (FMT == Q5_1) {
            // dsc = d, deff = -m (kernels/moe_matvec_q5k_repacked.cpp:86-91): dsc*dx*idot - deff*xsum
            const float v = (f16_bits_to_f32(r.dm) * ds.x) * (float)i0;
            return fmaf(f16_bits_to_f32(r.dm >> 16), ds.y, v);
        } else {
            const float d = f16_bits_to_f32(r.dd), dmin = f16_bits_to_f32(r.dd >> 16);
            const int sc = (int)(r.sm & 0xFFu);
            float v = (d * ds.x) * (float)(sc * i0);
            return fmaf(dmin * ds.y, small_uint_to_float(r.sm >> 8), v);
        }
    } else if constexpr (FMT == Q6_K) {
        // byte g of the high-2 plane belongs to group g (src/quant/q6_k.rs:128-133)
        const uint4 q = r.q;
        uint32_t g0, g1, g2, g3, g4, g5, g6, g7;
        spread_fields4(r.h.x, g0, g1, g2, g3);
        spread_fields4(r.h.y, g4, g5, g6, g7);
        int s = 0, t = 0;
        s = __dp4a((int)((q.x & M) | g0), xl.x, s);
        t = __dp4a((int)(((q.x >> 4) & M) | g1), xh.x, t);
        s = __dp4a((int)((q.y & M) | g2), xl.y, s);
        t = __dp4a((int)(((q.y >> 4) & M) | g3), xh.y, t);
        s = __dp4a((int)((q.z & M) | g4), xl.z, s);
        t = __dp4a((int)(((q.z >> 4) & M) | g5), xh.z, t);
        s = __dp4a((int)((q.w & M) | g6), xl.w, s);
        t = __dp4a((int)(((q.w >> 4) & M) | g7), xh.w, t);
        i0 = s - is.x;
        i1 = t - is.y;
        const int slo = (int)(int8_t)(r.sm & 0xFFu), shi = (int)(int8_t)(r.sm >> 8);
        return (f16_bits_to_f32(r.d) * ds.x) * (float)(slo * i0 + shi * i1);
    } else if constexpr (FMT == Q8_0) {
        int s = 0, t = 0;
        s = __dp4a((int)r.wl.x, xl.x, s);
        t = __dp4a((int)r.wh.x, xh.x, t);
        s = __dp4a((int)r.wl.y, xl.y, s);
        t = __dp4a((int)r.wh.y, xh.y, t);
        s = __dp4a((int)r.wl.z, xl.z, s);
        t = __dp4a((int)r.wh.z, xh.z, t);
        s = __dp4a((int)r.wl.w, xl.w, s);
        t = __dp4a((int)r.wh.w, xh.w, t);
        i0 = s + t;
        return (f16_bits_to_f32(r.d) * ds.x) * (float)i0;
    } else if constexpr (FMT == Q4_0) {
        const int idot16 = dot_nibbles16(r.q, xl, xh) - is.x; // 16 * sum((q-8)*xq)
        i0 = idot16 >> 4;
        return (f16_bits_to_f32(r.d) * ds.x) * (float)idot16;
    } else { // IQ4_XS and IQ3_S, activations staged in iq4_lookup8 order
        int c0, c1, c2, c3, c4, c5, c6, c7;
        iq4_lookup8<FMT>(r.q.x, c0, c1);
        iq4_lookup8<FMT>(r.q.y, c2, c3);
        iq4_lookup8<FMT>(r.q.z, c4, c5);
        iq4_lookup8<FMT>(r.q.w, c6, c7);
        int s = 0, t = 0;
        s = __dp4a(c0, xl.x, s);
        t = __dp4a(c1, xl.y, t);
        s = __dp4a(c2, xl.z, s);
        t = __dp4a(c3, xl.w, t);
        s = __dp4a(c4, xh.x, s);
        t = __dp4a(c5, xh.y, t);
        s = __dp4a(c6, xh.z, s);
        t = __dp4a(c7, xh.w, t);
        i0 = s + t;
        return (f16_bits_to_f32(r.d) * ds.x) * (float)i0;
    }
}

// --------------------------------------------------------------------------------------------
// NB    compile-time bound on activation rows (n_rows <= NB)
// DUMP  write the per-block integers instead of y (debug entry point)
// ks    warps that split one weight row (1, 2, 4 or 8; ks <= iterations per row)
// The CTA walks row blocks block_begin, block_begin + block_stride, ...
// smem: staged activations (n_rows * n_sub * x_bytes), then 2 * warps * NB partial sums.
template <int FMT, int NB, bool DUMP>
__device__ __forceinline__ void
stream_body(uint8_t *smem, const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq,
            float *__restrict__ y, int32_t *__restrict__ idots, uint32_t in_dim, uint32_t out_dim,
            uint32_t n_rows, uint32_t ks, uint32_t block_begin, uint32_t block_stride)
{
    constexpr int G = FmtTraits<FMT>::G;
    if (NB <= 2) n_rows = NB; // the launchers pick NB = n_rows for one and two rows: a compile-time count
    const uint32_t n_sub = in_dim >> 5, n_iters = (n_sub + 31u) >> 5;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const uint32_t rb_rows = n_warps / ks, r_local = warp / ks, chunk = warp - r_local * ks;
    const uint32_t it0 = chunk * n_iters / ks, it1 = (chunk + 1u) * n_iters / ks;
    const uint32_t n_blocks = (out_dim + rb_rows - 1u) / rb_rows;
    // The chunk's iterations are cut into groups of at most G, as evenly as possible (17
    // iterations with G = 4 become 4,4,3,3,3 rather than 4,4,4,4,1).
    const uint32_t chunk_iters = it1 - it0;
    const uint32_t n_groups = (chunk_iters + G - 1u) / G;
    const uint32_t g_base = n_groups ? chunk_iters / n_groups : 0u, g_rem = n_groups ? chunk_iters % n_groups : 0u;
    auto group_len = [&](uint32_t gi) { return g_base + (gi < g_rem ? 1u : 0u); };
    const Planes p = planes_of<FMT>(w, in_dim, out_dim);
    const bool sup_a4 = (reinterpret_cast<uintptr_t>(p.sup) & 3u) == 0;
    const uint32_t n_xblocks = n_rows * n_sub;
    const XStage st = carve_stage<FMT>(smem, n_xblocks);
    float *partial = reinterpret_cast<float *>(smem + (((size_t)n_xblocks * FmtTraits<FMT>::x_bytes + 15u) & ~(size_t)15u));

    Raw<FMT> cur[G];
    // A group of n <= G iterations in which every lane has a sub-block is compiled once per n
    // without guards or clamps (the loads of a group must issue back to back); only the last
    // group of a row whose sub-block count is not a multiple of 32 takes the guarded form.
    auto lanes_full = [&](uint32_t it, uint32_t n) { return (it + n) * 32u <= n_sub; };
    auto with_count = [&](uint32_t n, auto &&f) {
        switch (n) {
        case 1: f(std::integral_constant<int, 1>{}); break;
        case 2: if constexpr (G >= 2) f(std::integral_constant<int, 2>{}); break;
        case 3: if constexpr (G >= 3) f(std::integral_constant<int, 3>{}); break;
        case 4: if constexpr (G >= 4) f(std::integral_constant<int, 4>{}); break;
        default: if constexpr (G >= 5) f(std::integral_constant<int, 5>{}); break;
        }
    };
    auto fetch_group = [&](uint32_t row, uint32_t it, uint32_t n) {
        // rows past the end are clamped: their loads stay legal, their results unused
        row = min(row, out_dim - 1u);
        const size_t rbase = (size_t)row * p.nsp, sbase = (size_t)row * p.n_super;
        if (lanes_full(it, n)) {
            const GroupPtrs g = group_ptrs<FMT>(p, row, it * 32u + lane);
            with_count(n, [&](auto nc) {
                if (sup_a4) {
#pragma unroll
                    for (int i = 0; i < decltype(nc)::value; i++) fetch_off<FMT, true>(cur[i], g, i);
                } else {
#pragma unroll
                    for (int i = 0; i < decltype(nc)::value; i++) fetch_off<FMT, false>(cur[i], g, i);
                }
            });
        } else {
#pragma unroll
            for (int i = 0; i < G; i++) {
                if (i < (int)n) {
                    const uint32_t sb = min((it + i) * 32u + lane, n_sub - 1u);
                    fetch<FMT>(cur[i], p, rbase + sb, sbase + (sb >> 3), sup_a4);
                }
            }
        }
    };

    uint32_t blk = block_begin, it = it0, gi = 0;
    if (blk < n_blocks) fetch_group(blk * rb_rows + r_local, it, group_len(0)); // weights do not wait for x
    pdl_launch_dependents();
    pdl_wait(); // activations (and y) belong to the preceding kernels
    stage_x<FMT>(st, xq, n_xblocks);
    __syncthreads();

    float acc[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) acc[b] = 0.0f;
    uint32_t parity = 0;

    while (blk < n_blocks) {
        const uint32_t row = blk * rb_rows + r_local;
        const uint32_t n_now = group_len(gi);
        if (lanes_full(it, n_now)) {
            with_count(n_now, [&](auto nc) {
#pragma unroll
                for (int i = 0; i < decltype(nc)::value; i++) {
                    const uint32_t sb = (it + i) * 32u + lane;
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        if (b < (int)n_rows) {
                            const uint32_t xi = b * n_sub + sb;
                            const int4 xl = st.lo[xi], xh = st.hi[xi];
                            const float2 ds = st.ds[xi];
                            const int2 is = FmtTraits<FMT>::needs_is ? st.is[xi] : make_int2(0, 0);
                            int i0, i1;
                            acc[b] += term<FMT>(cur[i], xl, xh, ds, is, i0, i1);
                            if (DUMP && row < out_dim) {
                                int32_t *o = idots + (((size_t)b * out_dim + row) * n_sub + sb) * 2;
                                o[0] = i0;
                                o[1] = i1;
                            }
                        }
                    }
                }
            });
        } else {
#pragma unroll
            for (int i = 0; i < G; i++) {
                if (i < (int)n_now) {
                    const uint32_t sb_raw = (it + i) * 32u + lane;
                    const bool valid = sb_raw < n_sub;
                    const uint32_t sb = min(sb_raw, n_sub - 1u);
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        if (b < (int)n_rows) {
                            const uint32_t xi = b * n_sub + sb;
                            const int4 xl = st.lo[xi], xh = st.hi[xi];
                            const float2 ds = st.ds[xi];
                            const int2 is = FmtTraits<FMT>::needs_is ? st.is[xi] : make_int2(0, 0);
                            int i0, i1;
                            const float t = term<FMT>(cur[i], xl, xh, ds, is, i0, i1);
                            acc[b] += valid ? t : 0.0f;
                            if (DUMP && valid && row < out_dim) {
                                int32_t *o = idots + (((size_t)b * out_dim + row) * n_sub + sb) * 2;
                                o[0] = i0;
                                o[1] = i1;
                            }
                        }
                    }
                }
            }
        }
        it += n_now;
        gi++;
        const bool item_done = gi >= n_groups;
        const uint32_t nblk = item_done ? blk + block_stride : blk;
        const uint32_t nit = item_done ? it0 : it;
        const uint32_t ngi = item_done ? 0u : gi;
        if (nblk < n_blocks) fetch_group(nblk * rb_rows + r_local, nit, group_len(ngi)); // in flight during the reduction
        if (item_done) {
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float v = warp_sum(acc[b]);
                acc[b] = 0.0f;
                if (DUMP) continue;
                if (ks == 1) {
                    if (lane == 0 && b < (int)n_rows && row < out_dim) y[(size_t)b * out_dim + row] = v;
                } else if (lane == 0) {
                    partial[(parity * n_warps + warp) * NB + b] = v;
                }
            }
            if (!DUMP && ks > 1) {
                // every warp of the CTA finishes exactly one item per row block
                __syncthreads();
                if (chunk == 0 && lane < n_rows && row < out_dim) {
                    float v = 0.0f;
                    for (uint32_t c = 0; c < ks; c++) v += partial[(parity * n_warps + warp + c) * NB + lane];
                    y[(size_t)lane * out_dim + row] = v;
                }
                parity ^= 1u;
            }
        }
        blk = nblk;
        it = nit;
        gi = ngi;
    }
}

template <int NB> struct MinBlocks { static constexpr int v = NB <= 1 ? 4 : NB <= 4 ? 3 : 2; };
// weight rows a warp of matvec_multi_kernel owns: as many as the accumulators (R * NB) leave registers for
template <int NB> struct MultiRows { static constexpr int v = NB <= 4 ? 4 : 2; };
constexpr int kMultiMinBlocks = 2; // 128 registers: R weight rows in flight twice over, plus R * NB sums

// --------------------------------------------------------------------------------------------
// The common decode shape gets a loop with nothing else in it: one warp per weight row (no row
// split), every lane busy in every iteration (in_dim a multiple of 1024), a row cut into groups of
// LEN iterations plus at most one shorter group.  Same loads, same term(), same order of additions per
// lane as stream_body; it only sheds that kernel's bookkeeping, which is a third of its
// instructions on a 5-iteration row.
// Rows of a last, mostly empty round that the CTAs share (see matvec_rows_kernel): the leftover of the rounds of
// row_stride rows when it is at most a quarter of a round, there is a full round before it and a row has several groups.
__host__ __device__ inline uint32_t rows_shared_tail(uint32_t out_dim, uint32_t row_stride, uint32_t n_units)
{
    const uint32_t full_rounds = out_dim / row_stride, left = out_dim - full_rounds * row_stride;
    return (n_units >= 2u && full_rounds >= 1u && left * 4u <= row_stride) ? left : 0u;
}

template <int FMT, int NB, int LEN, bool TAIL = false>
__global__ void __launch_bounds__(kWarpsPerCta * 32, MinBlocks<NB>::v)
matvec_rows_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, float *__restrict__ y,
                   uint32_t in_dim, uint32_t out_dim, uint32_t n_rows)
{
    extern __shared__ __align__(16) uint8_t smem[];
    if (NB <= 2) n_rows = NB;
    const uint32_t n_sub = in_dim >> 5, n_iters = n_sub >> 5;
    const uint32_t n_groups = n_iters / LEN, tail = n_iters - n_groups * LEN; // a row = n_groups full groups + a shorter one
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const Planes p = planes_of<FMT>(w, in_dim, out_dim);
    const bool sup_a4 = (reinterpret_cast<uintptr_t>(p.sup) & 3u) == 0;
    const XStage st = carve_stage<FMT>(smem, n_rows * n_sub);
    const uint32_t row_stride = gridDim.x * kWarpsPerCta;

    Raw<FMT> cur[LEN];
    // group g of a row; g == n_groups is the short last group (`tail` iterations)
    auto fetch_group = [&](uint32_t row, uint32_t g) {
        const GroupPtrs gp = group_ptrs<FMT>(p, min(row, out_dim - 1u), g * (LEN * 32u) + lane);
        if (g < n_groups) {
            if (sup_a4) {
#pragma unroll
                for (int i = 0; i < LEN; i++) fetch_off<FMT, true>(cur[i], gp, i);
            } else {
#pragma unroll
                for (int i = 0; i < LEN; i++) fetch_off<FMT, false>(cur[i], gp, i);
            }
        } else {
#pragma unroll
            for (int i = 0; i < LEN; i++) {
                if (i < (int)tail) {
                    if (sup_a4) fetch_off<FMT, true>(cur[i], gp, i);
                    else fetch_off<FMT, false>(cur[i], gp, i);
                }
            }
        }
    };
    float acc[NB];
    auto compute = [&](uint32_t g, uint32_t n) {
        const uint32_t sb0 = g * (LEN * 32u) + lane;
#pragma unroll
        for (int i = 0; i < LEN; i++) {
            if (i < (int)n) {
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    if (b < (int)n_rows) {
                        const uint32_t xi = b * n_sub + sb0 + i * 32u;
                        const int4 xl = st.lo[xi], xh = st.hi[xi];
                        const float2 ds = st.ds[xi];
                        const int2 is = FmtTraits<FMT>::needs_is ? st.is[xi] : make_int2(0, 0);
                        int i0, i1;
                        acc[b] += term<FMT>(cur[i], xl, xh, ds, is, i0, i1);
                    }
                }
            }
        }
    };

    uint32_t row = blockIdx.x * kWarpsPerCta + warp;
    const uint32_t first_group = n_groups ? 0u : n_groups; // rows shorter than LEN are one short group
    // A last round that is mostly empty would cost a whole row time for a few rows (5120 rows on 4736 resident warps: 384
    // warps walk a second row while the others idle).  When the leftover is at most a quarter of a round and a row has
    // several groups, those rows are dealt one per CTA instead and the CTA's warps share each: a group per warp, the
    // partial sums added in group order.
    // (TAIL: the instantiation the host picks when that applies; the plain one keeps the original code exactly.)
    const uint32_t n_units = n_groups + (tail ? 1u : 0u);
    const uint32_t shared_rows = TAIL ? rows_shared_tail(out_dim, row_stride, n_units) : 0u;
    const uint32_t main_end = out_dim - shared_rows;
    if (row < main_end) fetch_group(row, first_group);      // weights do not wait for x
    pdl_launch_dependents();
    pdl_wait();
    stage_x<FMT>(st, xq, n_rows * n_sub);
    __syncthreads();

    for (; row < main_end; row += row_stride) {
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.0f;
        for (uint32_t g = 0; g < n_groups; g++) {
            compute(g, LEN);
            // the next group's loads go out before this row is reduced
            if (g + 1 < n_groups || tail) fetch_group(row, g + 1);
            else if (row + row_stride < main_end) fetch_group(row + row_stride, first_group);
        }
        if (tail) {
            compute(n_groups, tail);
            if (row + row_stride < main_end) fetch_group(row + row_stride, first_group);
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const float v = warp_sum(acc[b]);
            if (lane == 0 && b < (int)n_rows) y[(size_t)b * out_dim + row] = v;
        }
    }
    if constexpr (TAIL) {
        __shared__ float s_shared[NB][kWarpsPerCta];
        for (uint32_t t = blockIdx.x; t < shared_rows; t += gridDim.x) {
            const uint32_t r = main_end + t;
#pragma unroll
            for (int b = 0; b < NB; b++) acc[b] = 0.0f;
            for (uint32_t g = warp; g < n_units; g += kWarpsPerCta) {
                fetch_group(r, g);
                compute(g, g < n_groups ? (uint32_t)LEN : tail);
            }
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float v = warp_sum(acc[b]);
                if (lane == 0) s_shared[b][warp] = v;
            }
            __syncthreads();
            if (warp == 0 && lane < n_rows) {
                float v = s_shared[lane][0];
                for (uint32_t w = 1; w < min((uint32_t)kWarpsPerCta, n_units); w++) v += s_shared[lane][w]; // warp order: reproducible
                y[(size_t)lane * out_dim + r] = v;
            }
            __syncthreads();
        }
    }
}

// --------------------------------------------------------------------------------------------
// Several activation rows: the row kernels above read every activation block from shared memory
// once per weight row, and at NB rows that traffic (48 bytes per lane, sub-block and activation
// row) outruns the math.  Here a warp owns R consecutive weight rows: each activation block is
// loaded once and used for all R, so shared-memory reads per weight row drop by R.  Same loads,
// same term(), same order of additions per lane as the other kernels (iterations in turn, then
// the warp reduction), hence the same bits.  The next iteration's weights are requested before
// the current one is used.
template <int FMT, int NB, int R>
__global__ void __launch_bounds__(kWarpsPerCta * 32, kMultiMinBlocks)
matvec_multi_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, float *__restrict__ y,
                    uint32_t in_dim, uint32_t out_dim, uint32_t n_rows)
{
    extern __shared__ __align__(16) uint8_t smem[];
    if (NB <= 2) n_rows = NB;
    const uint32_t n_sub = in_dim >> 5, n_iters = n_sub >> 5;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const Planes p = planes_of<FMT>(w, in_dim, out_dim);
    const bool sup_a4 = (reinterpret_cast<uintptr_t>(p.sup) & 3u) == 0;
    const XStage st = carve_stage<FMT>(smem, n_rows * n_sub);
    const uint32_t row_stride = gridDim.x * kWarpsPerCta * R;

    Raw<FMT> cur[R], nxt[R];
    GroupPtrs gp[R];
    auto set_rows = [&](uint32_t base) {
#pragma unroll
        for (int r = 0; r < R; r++) gp[r] = group_ptrs<FMT>(p, min(base + r, out_dim - 1u), lane);
    };
    auto fetch = [&](Raw<FMT>(&dst)[R], uint32_t it) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (sup_a4) fetch_off<FMT, true>(dst[r], gp[r], (int)it);
            else fetch_off<FMT, false>(dst[r], gp[r], (int)it);
        }
    };

    uint32_t row = (blockIdx.x * kWarpsPerCta + warp) * R;
    if (row < out_dim) { // weights do not wait for x
        set_rows(row);
        fetch(cur, 0);
    }
    pdl_launch_dependents();
    pdl_wait();
    stage_x<FMT>(st, xq, n_rows * n_sub);
    __syncthreads();

    for (; row < out_dim; row += row_stride) {
        float acc[R][NB];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = 0.0f;
        for (uint32_t it = 0; it < n_iters; it++) {
            if (it + 1 < n_iters) {
                fetch(nxt, it + 1);
            } else if (row + row_stride < out_dim) {
                set_rows(row + row_stride);
                fetch(nxt, 0);
            }
            const uint32_t sb = it * 32u + lane;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                if (b < (int)n_rows) {
                    const uint32_t xi = b * n_sub + sb;
                    const int4 xl = st.lo[xi], xh = st.hi[xi];
                    const float2 ds = st.ds[xi];
                    const int2 is = FmtTraits<FMT>::needs_is ? st.is[xi] : make_int2(0, 0);
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        int i0, i1;
                        acc[r][b] += term<FMT>(cur[r], xl, xh, ds, is, i0, i1);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < R; r++) cur[r] = nxt[r];
        }
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float v = warp_sum(acc[r][b]);
                if (lane == 0 && b < (int)n_rows && row + r < out_dim) y[(size_t)b * out_dim + row + r] = v;
            }
    }
}

template <int FMT, int NB, bool DUMP>
__global__ void __launch_bounds__(kWarpsPerCta * 32, MinBlocks<NB>::v)
matvec_stream_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, float *__restrict__ y,
                     int32_t *__restrict__ idots, uint32_t in_dim, uint32_t out_dim, uint32_t n_rows,
                     uint32_t ks)
{
    extern __shared__ __align__(16) uint8_t smem[];
    stream_body<FMT, NB, DUMP>(smem, w, xq, y, idots, in_dim, out_dim, n_rows, ks, blockIdx.x, gridDim.x);
}

// Expert-grouped form: blockIdx.y is a global token tile, mapped to (expert, local tile) by
// binary search over tile_off as in kernels/mmq_gemm_q4k_grouped.cpp:49-60; the tile's rows
// of xq / y are contiguous in expert-sorted order.
// A tile of the sort is kGroupedTile tokens; this kernel takes it as halves of BN = 16 rows
// (blockIdx.y = 2 * tile + half).
constexpr int kGroupedTile = 32;

template <int FMT, int BN>
__global__ void __launch_bounds__(kWarpsPerCta * 32, MinBlocks<BN>::v)
matvec_grouped_kernel(const uint8_t *__restrict__ slab, size_t bytes_per_expert,
                      const int32_t *__restrict__ expert_off, const int32_t *__restrict__ tile_off,
                      uint32_t n_expert, const uint8_t *__restrict__ xq, float *__restrict__ y,
                      uint32_t in_dim, uint32_t out_dim)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t by = blockIdx.y / (kGroupedTile / BN), part = blockIdx.y % (kGroupedTile / BN);
    if (by >= (uint32_t)tile_off[n_expert]) return; // over-launched tile
    uint32_t lo = 0, hi = n_expert;
    while (lo + 1 < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if ((uint32_t)tile_off[mid] <= by) lo = mid; else hi = mid;
    }
    const uint32_t e = lo;
    const uint32_t tok0 = (uint32_t)expert_off[e] + (by - (uint32_t)tile_off[e]) * kGroupedTile + part * BN;
    if (tok0 >= (uint32_t)expert_off[e + 1]) return; // the tile's second half is empty
    const uint32_t n = min((uint32_t)BN, (uint32_t)expert_off[e + 1] - tok0);
    const uint32_t n_sub = in_dim >> 5;
    stream_body<FMT, BN, false>(smem, slab + (size_t)e * bytes_per_expert,
                                xq + (size_t)tok0 * n_sub * RC_BLOCKQ8_BYTES, y + (size_t)tok0 * out_dim,
                                nullptr, in_dim, out_dim, n, 1, blockIdx.x, gridDim.x);
}

// Routed-expert matvec of the decode path (kernels/moe_matvec_q4k_repacked.cpp and siblings, launched by
// src/runtime/qwen35.rs:3066-3103 and, for the down projection, :3105-3139): blockIdx.y is the routing slot,
// blockIdx.z the token; the slot's expert comes from ids on the device, its weights are
// slab + ids * bytes_per_expert, its activation block row tok * xq_tok_stride + slot * xq_slot_stride
// (in BlockQ8 blocks: gate / up share one row per token, down has one per slot).  An id outside the slab
// writes zeros.
template <int FMT>
__global__ void __launch_bounds__(kWarpsPerCta * 32, MinBlocks<1>::v)
moe_expert_matvec_kernel(const uint8_t *__restrict__ slab, size_t bytes_per_expert, const int32_t *__restrict__ ids,
                         uint32_t n_expert, const uint8_t *__restrict__ xq, float *__restrict__ y, uint32_t in_dim,
                         uint32_t out_dim, uint32_t n_used, uint32_t xq_tok_stride, uint32_t xq_slot_stride, uint32_t ks)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t slot = blockIdx.y, tok = blockIdx.z;
    float *yo = y + ((size_t)tok * n_used + slot) * out_dim;
    pdl_wait(); // ids are a predecessor's output
    const int32_t e = ids[(size_t)tok * n_used + slot];
    if (e < 0 || (uint32_t)e >= n_expert) {
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < out_dim; i += gridDim.x * blockDim.x) yo[i] = 0.0f;
        return;
    }
    stream_body<FMT, 1, false>(smem, slab + (size_t)e * bytes_per_expert,
                               xq + ((size_t)tok * xq_tok_stride + (size_t)slot * xq_slot_stride) * RC_BLOCKQ8_BYTES, yo,
                               nullptr, in_dim, out_dim, 1, ks, blockIdx.x, gridDim.x);
}

// Fused gate + up + SwiGLU of the decode-side routed experts (kernels/moe_gate_up_swiglu_q4k_repacked.cpp,
// launched by src/runtime/qwen35.rs:3141-3167): a warp computes row i of the expert's gate tensor and
// row i of its up tensor against the same activation blocks and writes silu(gate) * up: one launch in
// place of two matvecs and the activation.  Whole iterations only (in_dim a multiple of 1024).
template <int FMT>
__global__ void __launch_bounds__(kWarpsPerCta * 32, MinBlocks<1>::v)
moe_gate_up_swiglu_kernel(const uint8_t *__restrict__ gate_slab, const uint8_t *__restrict__ up_slab, size_t bytes_per_expert,
                          const int32_t *__restrict__ ids, uint32_t n_expert, const uint8_t *__restrict__ xq,
                          float *__restrict__ y, uint32_t in_dim, uint32_t out_dim, uint32_t n_used, uint32_t xq_tok_stride,
                          uint32_t xq_slot_stride)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t n_sub = in_dim >> 5, n_iters = n_sub >> 5;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t slot = blockIdx.y, tok = blockIdx.z;
    float *yo = y + ((size_t)tok * n_used + slot) * out_dim;
    pdl_launch_dependents();
    pdl_wait(); // ids and activations are predecessors' outputs
    const int32_t e = ids[(size_t)tok * n_used + slot];
    if (e < 0 || (uint32_t)e >= n_expert) {
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < out_dim; i += gridDim.x * blockDim.x) yo[i] = 0.0f;
        return;
    }
    const Planes pg = planes_of<FMT>(gate_slab + (size_t)e * bytes_per_expert, in_dim, out_dim);
    const Planes pu = planes_of<FMT>(up_slab + (size_t)e * bytes_per_expert, in_dim, out_dim);
    const bool a4 = ((reinterpret_cast<uintptr_t>(pg.sup) | reinterpret_cast<uintptr_t>(pu.sup)) & 3u) == 0;
    const XStage st = carve_stage<FMT>(smem, n_sub);
    stage_x<FMT>(st, xq + ((size_t)tok * xq_tok_stride + (size_t)slot * xq_slot_stride) * RC_BLOCKQ8_BYTES, n_sub);
    __syncthreads();
    for (uint32_t row = blockIdx.x * kWarpsPerCta + warp; row < out_dim; row += gridDim.x * kWarpsPerCta) {
        const GroupPtrs gg = group_ptrs<FMT>(pg, row, lane), gu = group_ptrs<FMT>(pu, row, lane);
        float ag = 0.0f, au = 0.0f;
        Raw<FMT> rg, ru;
        if (a4) { fetch_off<FMT, true>(rg, gg, 0); fetch_off<FMT, true>(ru, gu, 0); }
        else { fetch_off<FMT, false>(rg, gg, 0); fetch_off<FMT, false>(ru, gu, 0); }
        for (uint32_t it = 0; it < n_iters; it++) {
            Raw<FMT> ng = rg, nu = ru;
            if (it + 1 < n_iters) {
                if (a4) { fetch_off<FMT, true>(ng, gg, (int)it + 1); fetch_off<FMT, true>(nu, gu, (int)it + 1); }
                else { fetch_off<FMT, false>(ng, gg, (int)it + 1); fetch_off<FMT, false>(nu, gu, (int)it + 1); }
            }
            const uint32_t xi = it * 32u + lane;
            const int4 xl = st.lo[xi], xh = st.hi[xi];
            const float2 ds = st.ds[xi];
            const int2 is = FmtTraits<FMT>::needs_is ? st.is[xi] : make_int2(0, 0);
            int i0, i1;
            ag += term<FMT>(rg, xl, xh, ds, is, i0, i1);
            au += term<FMT>(ru, xl, xh, ds, is, i0, i1);
            rg = ng;
            ru = nu;
        }
        const float g = warp_sum(ag), u = warp_sum(au);
        if (lane == 0) yo[row] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
    }
}

// --------------------------------------------------------------------------------------------
// The whole decode FFN of one GPU in ONE cooperative launch (step_swiglu_ffn, src/runtime/qwen35.rs:2694-2707:
// quantize x -> gate, up -> silu(gate) * up -> quantize -> down), row-sharded over `world` GPUs; the phases are listed
// at ffn_decode_kernel.  Seven launches of 3 to 9 us each become one, with no barrier inside the grid: a gate row and its
// up row are walked by warps of one CTA.  A wait that runs out records a code (rc_device_status) and the launch ends.
constexpr unsigned long long kFfnWaitNs = 200ull * 1000 * 1000;
constexpr uint32_t kFfnEmpty = 0xFFFFFFFFu; // "not arrived yet" in the intermediate and output vectors
__device__ unsigned int g_ffn_error;
// measurement aid, off until the first ffn_read_trace(): phase timestamps (globaltimer ns) of CTA 0, and the latest time any
// CTA passed each mark
__device__ unsigned long long g_ffn_trace[16];
__device__ unsigned long long g_ffn_trace_max[16];
__device__ unsigned long long g_ffn_cta[8][160];
static uint32_t g_ffn_trace_on = 0;

struct FfnPeers {
    float *h[RC_MAX_PEERS];  // rank r's intermediate vector, three copies: f32 [3][ffn_total]
    float *y[RC_MAX_PEERS];  // rank r's arriving output rows, three copies: f32 [3][out_total]
};
struct FfnParams {
    const uint8_t *gate, *up, *down;
    const float *x;
    float *y;                  // f32 [out_total]: the finished output of this call (device or pinned host memory)
    unsigned long long *sync;  // work: [0] calls done, [1] CTAs past their gate and up rows, [2] gate/up rows drawn, over all calls
    uint32_t in_dim, ffn_local, ffn_total, ffn_begin, out_local, out_total, out_begin, world, rank;
    uint32_t ks, ks_gu;        // warps that share a down row / a gate or up row
    uint32_t trace;            // record phase times (debug)
};

__device__ __forceinline__ unsigned long long ffn_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ float ffn_ld_cg(const float *p)
{
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
// a 40-byte record written during this launch (by this or another GPU): read through L2, never through the
// non-coherent path
__device__ __forceinline__ XBlock load_blockq8_cg(const uint8_t *p)
{
    uint2 w[5];
#pragma unroll
    for (int i = 0; i < 5; i++)
        asm volatile("ld.global.cg.v2.u32 {%0, %1}, [%2];" : "=r"(w[i].x), "=r"(w[i].y) : "l"(p + 8 * i));
    XBlock x;
    x.d = __uint_as_float(w[0].x);
    x.xsum = __uint_as_float(w[0].y);
    x.lo = make_int4((int)w[1].x, (int)w[1].y, (int)w[2].x, (int)w[2].y);
    x.hi = make_int4((int)w[3].x, (int)w[3].y, (int)w[4].x, (int)w[4].y);
    const int ones = 0x01010101;
    x.s_lo = __dp4a(x.lo.x, ones, __dp4a(x.lo.y, ones, __dp4a(x.lo.z, ones, __dp4a(x.lo.w, ones, 0))));
    x.s_hi = __dp4a(x.hi.x, ones, __dp4a(x.hi.y, ones, __dp4a(x.hi.z, ones, __dp4a(x.hi.w, ones, 0))));
    return x;
}

// The BlockQ8 of 32 values held one per lane, as ten words: every lane returns word (lane < 10 ? lane : 0).
__device__ __forceinline__ uint32_t q8_words(float v, uint32_t lane)
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
    return lane == 0 ? __float_as_uint(d) : lane == 1 ? __float_as_uint(sum) : word;
}

// One warp's walk over rows of one tensor against staged activations.  A CTA's warps are split into teams of `vwarps`
// (the caller gives each warp its place `vwarp` in its team and the team's tensor); `ks` warps of a team share a row, each
// with a balanced slice of the row's 1024-wide iterations, loaded LEN iterations at a time.  prime() sends the first
// loads, which depend on no activation, so that they can fly while the activations are still being produced; run() keeps
// the next chunk (of this row, else of the warp's next row) in flight while the current one is multiplied.
template <int FMT> struct RowWalk {
    static constexpr int LEN = FmtTraits<FMT>::rows_max_len;
    Planes p;
    uint32_t lane, n_rows, n_sub, i0, i1, row, row_base, row_stride, rows_per_cta; // n_rows: one past the walk's last row
    bool a4;
    Raw<FMT> cur[LEN];

    // n_sub_ need not be a multiple of 32: the last iteration's lanes beyond the row read its last sub-block again, against
    // staged activations that are zero there (the caller stages zero blocks up to the next multiple of 32).
    // The walk covers rows [first, first + rows) of the tensor.
    __device__ __forceinline__ void init(const Planes &planes, uint32_t n_sub_, uint32_t rows, uint32_t ks, uint32_t vwarp, uint32_t vwarps,
                                         uint32_t first = 0)
    {
        p = planes;
        lane = threadIdx.x & 31u;
        n_rows = first + rows;
        n_sub = n_sub_;
        const uint32_t slice = vwarp % ks, n_iters = (n_sub + 31u) >> 5;
        i0 = slice * n_iters / ks;
        i1 = (slice + 1u) * n_iters / ks;
        rows_per_cta = vwarps / ks;
        row_base = first + blockIdx.x * rows_per_cta;
        row = row_base + vwarp / ks;
        row_stride = gridDim.x * rows_per_cta;
        a4 = (reinterpret_cast<uintptr_t>(p.sup) & 3u) == 0;
    }
    __device__ __forceinline__ void fetch(uint32_t r, uint32_t it)
    {
        if (it + LEN <= i1 && (it + LEN) * 32u <= n_sub) { // the common, unguarded chunk: its loads issue back to back
            const GroupPtrs gp = group_ptrs<FMT>(p, r, it * 32u + lane);
#pragma unroll
            for (int i = 0; i < LEN; i++) {
                if (a4) fetch_off<FMT, true>(cur[i], gp, i);
                else fetch_off<FMT, false>(cur[i], gp, i);
            }
        } else {
#pragma unroll
            for (int i = 0; i < LEN; i++) {
                if (it + i < i1) {
                    const GroupPtrs gp = group_ptrs<FMT>(p, r, min((it + i) * 32u + lane, n_sub - 1u));
                    if (a4) fetch_off<FMT, true>(cur[i], gp, 0);
                    else fetch_off<FMT, false>(cur[i], gp, 0);
                }
            }
        }
    }
    __device__ __forceinline__ void prime()
    {
        if (row < n_rows && i0 < i1) fetch(row, i0);
    }
    // Asks L2 for the 4-bit and high-bit planes of the rows that this CTA walks (whole rows: all their slices are this CTA's;
    // the rows of one round are consecutive), round by round, up to `budget` bytes, shared by n_pf warps.
    __device__ __forceinline__ void prefetch_cta_rows(uint32_t pf, uint32_t n_pf, uint32_t budget) const
    {
        constexpr uint32_t aux_w = (FMT == Q8_0) ? 16u : (FMT == Q6_K) ? 8u : (FMT == Q5_K || FMT == Q5_1) ? 4u : 0u;
        uint32_t spent = 0;
        for (uint32_t r0 = row_base; r0 < n_rows && spent < budget; r0 += row_stride) {
            const uint32_t n = min(rows_per_cta, n_rows - r0);
            const uint32_t len = n * p.nsp * 16u, len1 = n * p.nsp * aux_w;
            const uint8_t *b0 = p.nib + (size_t)r0 * p.nsp * 16u;
            for (uint32_t o = (pf * 32u + lane) * 128u; o < len; o += n_pf * 32u * 128u) asm volatile("prefetch.global.L2 [%0];" ::"l"(b0 + o));
            if (aux_w) {
                const uint8_t *b1 = p.aux + (size_t)r0 * p.nsp * aux_w;
                for (uint32_t o = (pf * 32u + lane) * 128u; o < len1; o += n_pf * 32u * 128u) asm volatile("prefetch.global.L2 [%0];" ::"l"(b1 + o));
            }
            spent += len + len1;
        }
    }
    // This warp's slice of row r (its first chunk in flight already) against the staged activations; while the last chunk is
    // multiplied, the first chunk of row r_next (if r_next < n_rows) goes out.  The same sum in all lanes.
    __device__ __forceinline__ float walk_row(const XStage &st, uint32_t r, uint32_t r_next)
    {
        float acc = 0.0f;
        for (uint32_t it = i0; it < i1; it += LEN) {
            if (it + LEN <= i1) {
#pragma unroll
                for (int i = 0; i < LEN; i++) {
                    const uint32_t xi = (it + i) * 32u + lane;
                    const int4 xl = st.lo[xi], xh = st.hi[xi];
                    const float2 ds = st.ds[xi];
                    const int2 is = FmtTraits<FMT>::needs_is ? st.is[xi] : make_int2(0, 0);
                    int d0, d1;
                    acc += term<FMT>(cur[i], xl, xh, ds, is, d0, d1);
                }
            } else {
#pragma unroll
                for (int i = 0; i < LEN; i++) {
                    if (it + i < i1) {
                        const uint32_t xi = (it + i) * 32u + lane;
                        const int4 xl = st.lo[xi], xh = st.hi[xi];
                        const float2 ds = st.ds[xi];
                        const int2 is = FmtTraits<FMT>::needs_is ? st.is[xi] : make_int2(0, 0);
                        int d0, d1;
                        acc += term<FMT>(cur[i], xl, xh, ds, is, d0, d1);
                    }
                }
            }
            if (it + LEN < i1) fetch(r, it + LEN);
            else if (r_next < n_rows) fetch(r_next, i0);
        }
        return warp_sum(acc);
    }
    // Rows dealt out in fixed order (row, row + row_stride, ...).  finish(row, live, sum) runs on every lane of every warp
    // once per round of the CTA; a round is uniform over the CTA, so finish may synchronize warps.
    template <typename Finish> __device__ __forceinline__ void run(const XStage &st, Finish finish)
    {
        for (uint32_t r0 = row_base; r0 < n_rows; r0 += row_stride, row += row_stride) {
            const bool live = row < n_rows && i0 < i1;
            finish(row, live, live ? walk_row(st, row, row + row_stride) : 0.0f);
        }
    }
};

// Quantizes n_blocks blocks of 32 f32 values (16-byte aligned) into staged activations for format FMT, the whole CTA at
// work: a warp loads four blocks per instruction (one float4 per lane, eight lanes per block) and all of a warp's loads go
// out before the first is used.  The sum follows the warp quantizer's butterfly (element i adds v[i] + v[i ^ 16], then
// ^ 8, 4, 2, 1: lanes ^ 4, 2, 1 of the block's eight, then the lane's own elements ^ 2, ^ 1), so a record equals
// quantize_q8's bit for bit.  through_l2: the values are written during this launch (by this or another GPU): they are read
// with relaxed system-scope loads, which observe them (a polling loop of ld.global.cg was seen to spin on a stale line).
__device__ __forceinline__ bool ffn_any_empty(const float4 &v)
{
    return __float_as_uint(v.x) == kFfnEmpty || __float_as_uint(v.y) == kFfnEmpty || __float_as_uint(v.z) == kFfnEmpty ||
           __float_as_uint(v.w) == kFfnEmpty;
}
// The slow path of a polled read, kept out of line so that the callers' unrolled loops stay in registers.
__device__ __noinline__ float4 ffn_wait_quad(const float *p, volatile int *ok)
{
    const unsigned long long t0 = ffn_ns();
    uint32_t spins = 0;
    float4 v;
    do {
        __nanosleep(100);
        asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
        if ((++spins & 15u) == 0 && (!*ok || ffn_ns() - t0 > kFfnWaitNs)) {
            if (*ok) {
                atomicExch(&g_ffn_error, 2u);
                *ok = 0;
            }
            break;
        }
    } while (ffn_any_empty(v));
    return v;
}
//   warp, n_warps: the calling warp's place among the warps that share the work.
//   poll: a value that still reads as kFfnEmpty has not arrived: it is read again, until *ok drops or the limit runs out
//   (then the code is recorded, *ok cleared and whatever is there is used: the caller discards the result).
template <int FMT, int kAhead = 6>
__device__ __forceinline__ void quantize_stage(const XStage &st, uint32_t n_blocks, const float *src, bool through_l2, uint32_t warp,
                                               uint32_t n_warps, bool poll = false, volatile int *ok = nullptr)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n_quads = (n_blocks + 3u) >> 2;
    for (uint32_t q0 = warp; q0 < n_quads; q0 += n_warps * kAhead) {
        float4 f[kAhead];
#pragma unroll
        for (int a = 0; a < kAhead; a++) {
            const uint32_t q = q0 + a * n_warps, b = q * 4u + (lane >> 3);
            f[a] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (q < n_quads && b < n_blocks) {
                const float *p = src + (size_t)b * 32u + (lane & 7u) * 4u;
                if (through_l2)
                    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(f[a].x), "=f"(f[a].y), "=f"(f[a].z), "=f"(f[a].w) : "l"(p));
                else
                    f[a] = *reinterpret_cast<const float4 *>(p);
            }
        }
#pragma unroll
        for (int a = 0; a < kAhead; a++) {
            const uint32_t q = q0 + a * n_warps, b = q * 4u + (lane >> 3);
            if (q >= n_quads) continue; // uniform over the warp
            float4 v = f[a];
            if (poll && b < n_blocks && ffn_any_empty(v)) v = ffn_wait_quad(src + (size_t)b * 32u + (lane & 7u) * 4u, ok);
            float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
            float s0 = v.x, s1 = v.y, s2 = v.z, s3 = v.w;
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) {
                amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
                s0 = __fadd_rn(s0, __shfl_xor_sync(0xFFFFFFFFu, s0, o));
                s1 = __fadd_rn(s1, __shfl_xor_sync(0xFFFFFFFFu, s1, o));
                s2 = __fadd_rn(s2, __shfl_xor_sync(0xFFFFFFFFu, s2, o));
                s3 = __fadd_rn(s3, __shfl_xor_sync(0xFFFFFFFFu, s3, o));
            }
            XBlock xb;
            xb.xsum = __fadd_rn(__fadd_rn(s0, s2), __fadd_rn(s1, s3));
            xb.d = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
            const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
            const int q0i = max(-127, min(127, __float2int_rn(__fmul_rn(v.x, inv))));
            const int q1i = max(-127, min(127, __float2int_rn(__fmul_rn(v.y, inv))));
            const int q2i = max(-127, min(127, __float2int_rn(__fmul_rn(v.z, inv))));
            const int q3i = max(-127, min(127, __float2int_rn(__fmul_rn(v.w, inv))));
            const int word = (q0i & 0xFF) | ((q1i & 0xFF) << 8) | ((q2i & 0xFF) << 16) | ((q3i & 0xFF) << 24);
            const uint32_t base = lane & 24u;
            xb.lo.x = __shfl_sync(0xFFFFFFFFu, word, base + 0);
            xb.lo.y = __shfl_sync(0xFFFFFFFFu, word, base + 1);
            xb.lo.z = __shfl_sync(0xFFFFFFFFu, word, base + 2);
            xb.lo.w = __shfl_sync(0xFFFFFFFFu, word, base + 3);
            xb.hi.x = __shfl_sync(0xFFFFFFFFu, word, base + 4);
            xb.hi.y = __shfl_sync(0xFFFFFFFFu, word, base + 5);
            xb.hi.z = __shfl_sync(0xFFFFFFFFu, word, base + 6);
            xb.hi.w = __shfl_sync(0xFFFFFFFFu, word, base + 7);
            if ((lane & 7u) == 0 && b < n_blocks) {
                const int ones = 0x01010101;
                xb.s_lo = __dp4a(xb.lo.x, ones, __dp4a(xb.lo.y, ones, __dp4a(xb.lo.z, ones, __dp4a(xb.lo.w, ones, 0))));
                xb.s_hi = __dp4a(xb.hi.x, ones, __dp4a(xb.hi.y, ones, __dp4a(xb.hi.z, ones, __dp4a(xb.hi.w, ones, 0))));
                stage_block<FMT>(st, b, xb);
            }
        }
    }
}

// Zero blocks [n_blocks, next multiple of 32) of staged activations: what RowWalk's lanes beyond a ragged row multiply by.
template <int FMT> __device__ __forceinline__ void stage_zero_tail(const XStage &st, uint32_t n_blocks)
{
    const uint32_t padded = (n_blocks + 31u) & ~31u;
    XBlock z;
    z.d = 0.0f;
    z.xsum = 0.0f;
    z.lo = z.hi = make_int4(0, 0, 0, 0);
    z.s_lo = z.s_hi = 0;
    for (uint32_t b = n_blocks + threadIdx.x; b < padded; b += blockDim.x) stage_block<FMT>(st, b, z);
}

__device__ __forceinline__ void ffn_group_sync(uint32_t id, uint32_t n_threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n_threads) : "memory");
}

// The decode feed-forward of one shard in one launch, one CTA of 24 warps per SM (a cooperative launch: every CTA is
// resident, so CTAs may wait for data that other CTAs and other GPUs produce):
//   1. every CTA quantizes x into shared memory while its first weights are in flight; warps 0-11 walk gate rows and warps
//      12-23 the same up rows, so silu(g) * u of a row is formed inside the CTA and stored, as f32, into every rank's
//      intermediate vector;
//   2. every CTA reads this rank's whole intermediate vector, reading again what has not arrived, quantizes it into shared
//      memory (records equal to quantize_q8's), and walks its down rows, storing each into every rank's output vector;
//   3. CTA 0 reads this rank's whole output vector the same way, copies it to y and publishes the call number.
// Arrival needs no flag, fence or counter: a vector is filled with kFfnEmpty (a NaN pattern that arithmetic never
// produces; a producer that meets it stores the canonical NaN) before its values are stored, and a 4-byte store arrives
// whole.  Each vector exists three times; call c uses copy c % 3 and refills copy (c + 2) % 3, which this rank's CTAs
// finished reading in call c - 1 and which a peer stores into in its call c + 2, i.e. after it has seen all of this rank's
// output rows of call c + 1: the end of this launch lies between the refill and those rows, so no fence is needed (with two
// copies the refill would have to be fenced against this launch's own output rows: a system-scope fence here costs 8 us).
// Every wait gives up after kFfnWaitNs, records a code and lets the kernel run out.
constexpr int kFfnWarps = 24;
constexpr uint32_t kFfnTeam = kFfnWarps / 2;

__device__ __forceinline__ float ffn_boxed(float v)
{
    return __float_as_uint(v) == kFfnEmpty ? __uint_as_float(0x7FFFFFFFu) : v;
}

template <int FG, int FD>
__global__ void __launch_bounds__(kFfnWarps * 32, 1) ffn_decode_kernel(const FfnParams P, const FfnPeers peers)
{
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ float s_part[2][kFfnWarps];
    __shared__ uint32_t s_next[2][kFfnTeam];
    __shared__ unsigned long long s_call;
    __shared__ int s_ok;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t n_sub_x = P.in_dim >> 5, n_sub_h = P.ffn_total >> 5;
    auto mark = [&](int k) {
        if (P.trace && threadIdx.x == 0) {
            const unsigned long long t = ffn_ns();
            if (blockIdx.x == 0) g_ffn_trace[k] = t;
            atomicMax(&g_ffn_trace_max[k], t);
            if (k < 8 && blockIdx.x < 160) g_ffn_cta[k][blockIdx.x] = t;
        }
    };
    mark(0);
    const unsigned long long call = *reinterpret_cast<volatile unsigned long long *>(P.sync) + 1ull; // written only by the previous launch
    const uint32_t cur = (uint32_t)(call % 3ull);
    if (threadIdx.x == 0) {
        s_call = call;
        s_ok = 1;
    }
    // ---- phase 1
    const XStage stx = carve_stage<FG>(smem, n_sub_x);
    {
        RowWalk<FG> w1;
        const bool is_up = warp >= kFfnTeam;
        const uint32_t vwarp = warp % kFfnTeam, ks = P.ks_gu;
        w1.init(planes_of<FG>(is_up ? P.up : P.gate, P.in_dim, P.ffn_local), n_sub_x, P.ffn_local, ks, vwarp, kFfnTeam);
        w1.prime();
        {
            // refill the copies that the call after the next will use (this rank's CTAs read them last in the previous call)
            float *const h_fill = peers.h[P.rank] + (size_t)((cur + 2u) % 3u) * P.ffn_total;
            float *const y_fill = peers.y[P.rank] + (size_t)((cur + 2u) % 3u) * P.out_total;
            for (uint32_t k = blockIdx.x * blockDim.x + threadIdx.x; k < P.ffn_total; k += gridDim.x * blockDim.x) h_fill[k] = __uint_as_float(kFfnEmpty);
            for (uint32_t k = blockIdx.x * blockDim.x + threadIdx.x; k < P.out_total; k += gridDim.x * blockDim.x) y_fill[k] = __uint_as_float(kFfnEmpty);
        }
        quantize_stage<FG>(stx, n_sub_x, P.x, false, warp, kFfnWarps);
        __syncthreads();
        mark(1);
        // The 2 * ks warps that hold slices of gate row i and up row i meet at a barrier of their own; the first of them
        // sums the slices in slice order and forms the row's intermediate value.  Rows are dealt out on demand: a group's
        // first two rows are fixed, every further one is the next of a counter that the group's first lane draws from at the
        // start of a round and hands to the group at the round's barrier, one round before its first loads go out (SMs do
        // not all stream equally fast: with fixed shares a tenth of the CTAs ended 5 us after the rest, and every rank
        // waits for the last value).  A call draws exactly ffn_local numbers, so the counter is never reset.
        const uint32_t group = vwarp / ks, slice = vwarp % ks;
        const bool leader = !is_up && slice == 0 && lane == 0;
        const size_t h_off = (size_t)cur * P.ffn_total + P.ffn_begin;
        const unsigned long long base = (call - 1ull) * (unsigned long long)P.ffn_local;
        const uint32_t first_drawn = 2u * w1.row_stride;
        uint32_t buf = 0, r_cur = w1.row, r_next = w1.row + w1.row_stride;
        while (r_cur < P.ffn_local) {
            unsigned long long drawn = 0;
            if (leader) drawn = atomicAdd(P.sync + 2, 1ull);
            const float sum = w1.walk_row(stx, r_cur, r_next);
            if (lane == 0) s_part[buf][warp] = sum;
            if (leader) s_next[buf][group] = first_drawn + (uint32_t)(drawn - base);
            ffn_group_sync(1u + group, 64u * ks);
            if (leader) {
                float g = s_part[buf][warp], u = s_part[buf][warp + kFfnTeam];
                for (uint32_t k = 1; k < ks; k++) {
                    g += s_part[buf][warp + k];
                    u += s_part[buf][warp + kFfnTeam + k];
                }
                const float h = ffn_boxed(__fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u)); // swiglu_q8_kernel's expression
                for (uint32_t k = 0; k < P.world; k++) peers.h[k][h_off + r_cur] = h;
            }
            r_cur = r_next;
            r_next = s_next[buf][group];
            buf ^= 1u;
        }
    }
    mark(2);
    // the down rows' first weights fly across the exchange of the intermediate
    RowWalk<FD> w3;
    w3.init(planes_of<FD>(P.down, P.ffn_total, P.out_local), n_sub_h, P.out_local, P.ks, warp, kFfnWarps);
    w3.prime();
    __syncthreads(); // the shared memory of phase 1 is free
    // This CTA's gate and up rows are done; thread 0 waits until those of every CTA of this GPU are (a monotone count: call x
    // CTAs), which is about when the other ranks' are.  Only then does the CTA poll the intermediate and prefetch: 148 CTAs
    // polling or prefetching crowd the loads of a CTA that still walks its rows, and every rank waits for the last value.
    if (threadIdx.x == 0) {
        atomicAdd(P.sync + 1, 1ull);
        const unsigned long long t0 = ffn_ns(), want = call * (unsigned long long)gridDim.x;
        while (*reinterpret_cast<volatile unsigned long long *>(P.sync + 1) < want) {
            if (ffn_ns() - t0 > kFfnWaitNs) {
                atomicExch(&g_ffn_error, 1u);
                s_ok = 0;
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    mark(3);
    // ---- phase 2: the whole intermediate, quantized per CTA.  Two warps meanwhile call the CTA's down rows into L2 (HBM is
    // idle during the exchange): a prefetch blocks its warp once the request queues are full, hence warps of their own, and
    // no more bytes than the exchange gives time for.
    const XStage sth = carve_stage<FD>(smem, n_sub_h);
    constexpr uint32_t kPfWarps = 2, kStageWarps = kFfnWarps - kPfWarps;
    // (seven quads in flight per warp: the 136 quads of config 2's intermediate are then one batch for each of the 22 warps)
    if (warp < kStageWarps) quantize_stage<FD, 7>(sth, n_sub_h, peers.h[P.rank] + (size_t)cur * P.ffn_total, true, warp, kStageWarps, true, &s_ok);
    else w3.prefetch_cta_rows(warp - kStageWarps, kPfWarps, 224u * 1024u);
    __syncthreads();
    mark(4);
    const bool ok = s_ok != 0;
    if (ok) {
        uint32_t buf = 0;
        const uint32_t ks = P.ks, slice = warp % ks;
        const size_t y_off = (size_t)cur * P.out_total + P.out_begin;
        w3.run(sth, [&](uint32_t r, bool live, float sum) {
            float v = sum;
            if (ks > 1u) {
                if (lane == 0) s_part[buf][warp] = sum;
                ffn_group_sync(1u + warp / ks, 32u * ks);
                if (slice == 0 && lane == 0) {
                    v = s_part[buf][warp];
                    for (uint32_t k = 1; k < ks; k++) v += s_part[buf][warp + k]; // slice order: reproducible
                }
                buf ^= 1u;
            }
            if (slice == 0 && lane == 0 && live) {
                v = ffn_boxed(v);
                for (uint32_t k = 0; k < P.world; k++) peers.y[k][y_off + r] = v;
            }
        });
    }
    mark(5);
    // ---- phase 3
    if (blockIdx.x == 0) {
        __syncthreads();
        if (ok) {
            const float *src = peers.y[P.rank] + (size_t)cur * P.out_total;
            const unsigned long long t0 = ffn_ns();
            for (uint32_t i = threadIdx.x; i < P.out_total; i += blockDim.x) {
                float v = ffn_ld_cg(src + i);
                uint32_t spins = 0;
                while (__float_as_uint(v) == kFfnEmpty) {
                    if ((++spins & 15u) == 0 && (!*(volatile int *)&s_ok || ffn_ns() - t0 > kFfnWaitNs)) {
                        if (*(volatile int *)&s_ok) {
                            atomicExch(&g_ffn_error, 3u);
                            s_ok = 0;
                        }
                        break;
                    }
                    __nanosleep(100);
                    v = ffn_ld_cg(src + i);
                }
                P.y[i] = v;
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            *reinterpret_cast<volatile unsigned long long *>(P.sync) = call; // the next launch's call number follows
            mark(6);
        }
    }
}

// The same step with the down projection sharded along its CONTRACTION (the usual tensor-parallel feed-forward: gate and up
// split by rows, down by the matching columns): a rank's slice of the intermediate never leaves it, and the only exchange
// is the sum of the ranks' partial outputs.  One CTA of 24 warps per SM, cooperative launch:
//   1. as in ffn_decode_kernel, but silu(g) * u goes to this GPU's own h vector (work memory);
//   2. when every CTA of the GPU is past step 1 (a release/acquire count), every CTA quantizes the rank's slice of h into
//      shared memory (ffn_local / 32 blocks: an eighth of the vector at eight GPUs) and walks ALL out_total rows of its
//      down slice [out_total][ffn_local]; the rows of a round are consecutive, so one warp per destination stores the
//      CTA's partial sums of the round into slot (this rank) of that rank's partial buffer in one instruction;
//   3. every CTA takes a share of the output rows, reads the `world` partial sums of each (reading again what has not
//      arrived: the buffers carry the "empty" pattern of ffn_decode_kernel and rotate over three copies the same way),
//      adds them in rank order and writes y.
// The sum over ranks replaces a single row sum, so results differ from the one-GPU step in the last bits and repeat bit
// for bit; the BlockQ8 blocks of the intermediate are the one-GPU step's (shards end on block boundaries).
struct FfnTpPeers {
    float *part[RC_MAX_PEERS]; // rank r's partial sums: f32 [3][world][out_total]
};
struct FfnTpParams {
    const uint8_t *gate, *up, *down;
    const float *x;
    float *y;                  // f32 [out_total]
    float *h;                  // work: f32 [ffn_local]
    unsigned long long *sync;  // work: [0] calls done, [1] CTAs past their gate and up rows, [2] gate/up rows drawn, over all calls
    uint32_t in_dim, ffn_local, out_total, world, rank, ks, ks_gu, trace;
    uint32_t tail_rows, ks_tail; // the down rows of a last, mostly empty round and the warps that share each of them
};

template <int FG, int FD>
__global__ void __launch_bounds__(kFfnWarps * 32, 1) ffn_tp_kernel(const FfnTpParams P, const FfnTpPeers peers)
{
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ float s_part[2][kFfnWarps];
    __shared__ float s_out[2][kFfnWarps];
    __shared__ float s_sum[kFfnWarps * 32];
    __shared__ uint32_t s_next[2][kFfnTeam];
    __shared__ int s_ok;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t n_sub_x = P.in_dim >> 5, n_sub_h = P.ffn_local >> 5;
    auto mark = [&](int k) {
        if (P.trace && threadIdx.x == 0) {
            const unsigned long long t = ffn_ns();
            if (blockIdx.x == 0) g_ffn_trace[k] = t;
            atomicMax(&g_ffn_trace_max[k], t);
            if (k < 8 && blockIdx.x < 160) g_ffn_cta[k][blockIdx.x] = t;
        }
    };
    mark(0);
    const unsigned long long call = *reinterpret_cast<volatile unsigned long long *>(P.sync) + 1ull; // written only by the previous launch
    const uint32_t cur = (uint32_t)(call % 3ull);
    if (threadIdx.x == 0) s_ok = 1;
    // ---- phase 1
    const XStage stx = carve_stage<FG>(smem, n_sub_x);
    {
        RowWalk<FG> w1;
        const bool is_up = warp >= kFfnTeam;
        const uint32_t vwarp = warp % kFfnTeam, ks = P.ks_gu;
        w1.init(planes_of<FG>(is_up ? P.up : P.gate, P.in_dim, P.ffn_local), n_sub_x, P.ffn_local, ks, vwarp, kFfnTeam);
        w1.prime();
        quantize_stage<FG>(stx, n_sub_x, P.x, false, warp, kFfnWarps);
        __syncthreads();
        mark(1);
        {
            // refill the copy of the partial buffer that the call after the next will use (here, not at the top: the call
            // number is the kernel's first load, and nothing before this point has to wait for it)
            float *const fill = peers.part[P.rank] + (size_t)((cur + 2u) % 3u) * P.world * P.out_total;
            const uint32_t n = P.world * P.out_total;
            for (uint32_t k = blockIdx.x * blockDim.x + threadIdx.x; k < n; k += gridDim.x * blockDim.x) fill[k] = __uint_as_float(kFfnEmpty);
        }
        const uint32_t group = vwarp / ks, slice = vwarp % ks;
        const bool leader = !is_up && slice == 0 && lane == 0;
        const unsigned long long base = (call - 1ull) * (unsigned long long)P.ffn_local;
        const uint32_t first_drawn = 2u * w1.row_stride;
        uint32_t buf = 0, r_cur = w1.row, r_next = w1.row + w1.row_stride;
        while (r_cur < P.ffn_local) {
            unsigned long long drawn = 0;
            if (leader) drawn = atomicAdd(P.sync + 2, 1ull);
            const float sum = w1.walk_row(stx, r_cur, r_next);
            if (lane == 0) s_part[buf][warp] = sum;
            if (leader) s_next[buf][group] = first_drawn + (uint32_t)(drawn - base);
            ffn_group_sync(1u + group, 64u * ks);
            if (leader) {
                float g = s_part[buf][warp], u = s_part[buf][warp + kFfnTeam];
                for (uint32_t k = 1; k < ks; k++) {
                    g += s_part[buf][warp + k];
                    u += s_part[buf][warp + kFfnTeam + k];
                }
                P.h[r_cur] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u); // swiglu_q8_kernel's expression
            }
            r_cur = r_next;
            r_next = s_next[buf][group];
            buf ^= 1u;
        }
    }
    mark(2);
    // The down rows in two walks: whole rounds of the grid with P.ks warps per row, then the leftover rows of a last,
    // mostly empty round (P.tail_rows of them, none when that does not pay) with more warps per row, so that the whole GPU
    // works on them instead of a fraction of its warps walking one more full row.
    const uint32_t main_rows = P.out_total - P.tail_rows;
    RowWalk<FD> w3;
    w3.init(planes_of<FD>(P.down, P.ffn_local, P.out_total), n_sub_h, main_rows, P.ks, warp, kFfnWarps);
    w3.prime();
    __syncthreads(); // this CTA's values of h are written; the shared memory of phase 1 is free
    if (threadIdx.x == 0) {
        // release: the CTA's stores to h (ordered before this thread by the barrier) before the count; acquire on the way out
        asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(P.sync + 1), "l"(1ull) : "memory");
        const unsigned long long t0 = ffn_ns(), want = call * (unsigned long long)gridDim.x;
        unsigned long long seen = 0;
        uint32_t spins = 0;
        for (;;) {
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(P.sync + 1) : "memory");
            if (seen >= want) break;
            if ((++spins & 63u) == 0 && ffn_ns() - t0 > kFfnWaitNs) {
                atomicExch(&g_ffn_error, 1u);
                s_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    mark(3);
    // ---- phase 2
    const XStage sth = carve_stage<FD>(smem, (n_sub_h + 31u) & ~31u);
    constexpr uint32_t kPfWarps = 2, kStageWarps = kFfnWarps - kPfWarps;
    if (warp < kStageWarps) quantize_stage<FD, 7>(sth, n_sub_h, P.h, true, warp, kStageWarps);
    else w3.prefetch_cta_rows(warp - kStageWarps, kPfWarps, 224u * 1024u);
    stage_zero_tail<FD>(sth, n_sub_h);
    __syncthreads();
    mark(4);
    const bool ok = s_ok != 0;
    if (ok) {
        uint32_t buf = 0;
        const size_t slot = ((size_t)cur * P.world + P.rank) * P.out_total;
        auto walk = [&](RowWalk<FD> &w, const uint32_t ks) {
            const uint32_t slice = warp % ks, rows_per_cta = kFfnWarps / ks;
            w.run(sth, [&](uint32_t r, bool live, float sum) {
                float v = sum;
                if (ks > 1u) {
                    if (lane == 0) s_part[buf][warp] = sum;
                    ffn_group_sync(1u + warp / ks, 32u * ks);
                    if (slice == 0 && lane == 0) {
                        v = s_part[buf][warp];
                        for (uint32_t k = 1; k < ks; k++) v += s_part[buf][warp + k]; // slice order: reproducible
                    }
                }
                if (slice == 0 && lane == 0) s_out[buf][warp / ks] = ffn_boxed(v);
                __syncthreads(); // the round's partial sums are in shared memory (a round is uniform over the CTA)
                // warp k stores the round's consecutive rows into rank k's buffer: one instruction, one packet on the link
                const uint32_t r0 = r - warp / ks;
                for (uint32_t k = warp; k < P.world; k += kFfnWarps)
                    if (lane < rows_per_cta && r0 + lane < w.n_rows) peers.part[k][slot + r0 + lane] = s_out[buf][lane];
                buf ^= 1u;
            });
        };
        walk(w3, P.ks);
        if (P.tail_rows) {
            RowWalk<FD> w4;
            w4.init(planes_of<FD>(P.down, P.ffn_local, P.out_total), n_sub_h, P.tail_rows, P.ks_tail, warp, kFfnWarps, main_rows);
            w4.prime();
            walk(w4, P.ks_tail);
        }
    }
    mark(5);
    // ---- phase 3: this CTA's share of the output rows, summed over the ranks in rank order
    if (ok) {
        const uint32_t per = (P.out_total + gridDim.x - 1u) / gridDim.x;
        const uint32_t r_begin = min(blockIdx.x * per, P.out_total), r_end = min(r_begin + per, P.out_total);
        const uint32_t chunk = (kFfnWarps * 32u) / P.world; // rows whose partial sums fit the staging array
        const float *src = peers.part[P.rank] + (size_t)cur * P.world * P.out_total;
        const unsigned long long t0 = ffn_ns();
        for (uint32_t c0 = r_begin; c0 < r_end; c0 += chunk) {
            const uint32_t n = min(chunk, r_end - c0);
            __syncthreads();
            for (uint32_t i = threadIdx.x; i < n * P.world; i += blockDim.x) {
                const uint32_t k = i / n, j = i % n;
                const float *a = src + (size_t)k * P.out_total + c0 + j;
                float v = ffn_ld_cg(a);
                uint32_t spins = 0;
                while (__float_as_uint(v) == kFfnEmpty) {
                    if ((++spins & 15u) == 0 && (!*(volatile int *)&s_ok || ffn_ns() - t0 > kFfnWaitNs)) {
                        if (*(volatile int *)&s_ok) {
                            atomicExch(&g_ffn_error, 3u);
                            s_ok = 0;
                        }
                        break;
                    }
                    __nanosleep(100);
                    v = ffn_ld_cg(a);
                }
                s_sum[k * n + j] = v;
            }
            __syncthreads();
            for (uint32_t j = threadIdx.x; j < n; j += blockDim.x) {
                float v = s_sum[j];
                for (uint32_t k = 1; k < P.world; k++) v = __fadd_rn(v, s_sum[k * n + j]);
                P.y[c0 + j] = v;
            }
        }
    }
    if (blockIdx.x == 0) {
        __syncthreads();
        if (threadIdx.x == 0) {
            *reinterpret_cast<volatile unsigned long long *>(P.sync) = call; // the next launch's call number follows
            mark(6);
        }
    }
}

// Warps that share a row: the count, among the powers of two that divide the team size, with the least (rounds of the grid) x
// (dependent load round trips + multiply time per round), the shared-row reduction counted per round.
static uint32_t ffn_pick_ks(uint32_t rows, uint32_t n_iters, uint32_t len, uint32_t grid, uint32_t team)
{
    uint32_t best = 1;
    float best_cost = 1e30f;
    for (uint32_t ks = 1; ks <= team && ks <= n_iters; ks *= 2u) { // (3 and 6 warps per row were measured: never better)
        if (team % ks) continue;
        const uint32_t per_round = grid * (team / ks), rounds = (rows + per_round - 1u) / per_round;
        const uint32_t per = (n_iters + ks - 1u) / ks, trips = (per + len - 1u) / len;
        const float cost = (float)rounds * ((float)trips + 0.15f * (float)per + (ks > 1u ? 0.3f : 0.0f));
        if (cost < best_cost) {
            best_cost = cost;
            best = ks;
        }
    }
    return best;
}

int g_ffn_plain_launch = 0; // measurement: the fused decode FFN as an ordinary launch
int g_ffn_ks_override = 0;   // measurement: warps that share a down row in the tensor-parallel launch (rc_tune_matvec's ks)

template <int FG, int FD>
int launch_ffn(cudaStream_t s, const FfnParams &P, const FfnPeers &peers)
{
    const uint32_t nx = P.in_dim >> 5, nh = P.ffn_total >> 5;
    const size_t smem = (std::max((size_t)nx * FmtTraits<FG>::x_bytes, (size_t)nh * FmtTraits<FD>::x_bytes) + 15u) & ~(size_t)15u;
    if (smem > kMaxStageBytesHost) return RC_ERR_BAD_SHAPE;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(ffn_decode_kernel<FG, FD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    FfnParams Q = P;
    const uint32_t grid = (uint32_t)sm_count(); // one CTA per SM: 24 warps, the whole register file
    Q.ks = ffn_pick_ks(P.out_local, nh >> 5, (uint32_t)FmtTraits<FD>::rows_max_len, grid, (uint32_t)kFfnWarps);
    Q.ks_gu = ffn_pick_ks(P.ffn_local, nx >> 5, (uint32_t)FmtTraits<FG>::rows_max_len, grid, kFfnTeam);
    Q.trace = g_ffn_trace_on;
    FfnPeers pp = peers;
    void *args[] = {&Q, &pp};
    if (g_ffn_plain_launch) {
        ffn_decode_kernel<FG, FD><<<grid, kFfnWarps * 32, smem, s>>>(Q, pp);
        return (int)cudaGetLastError();
    }
    return (int)cudaLaunchCooperativeKernel((const void *)ffn_decode_kernel<FG, FD>, dim3(grid), dim3(kFfnWarps * 32), args, smem, s);
}

template <int FG, int FD>
int launch_ffn_tp(cudaStream_t s, const FfnTpParams &P, const FfnTpPeers &peers)
{
    const uint32_t nx = P.in_dim >> 5, nh = ((P.ffn_local >> 5) + 31u) & ~31u;
    const size_t smem = (std::max((size_t)nx * FmtTraits<FG>::x_bytes, (size_t)nh * FmtTraits<FD>::x_bytes) + 15u) & ~(size_t)15u;
    if (smem > kMaxStageBytesHost) return RC_ERR_BAD_SHAPE;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(ffn_tp_kernel<FG, FD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    FfnTpParams Q = P;
    const uint32_t grid = (uint32_t)sm_count();
    Q.ks = ffn_pick_ks(P.out_total, nh >> 5, (uint32_t)FmtTraits<FD>::rows_max_len, grid, (uint32_t)kFfnWarps);
    if (g_ffn_ks_override > 0 && kFfnWarps % g_ffn_ks_override == 0 && (uint32_t)g_ffn_ks_override <= (nh >> 5)) Q.ks = (uint32_t)g_ffn_ks_override;
    {
        // leftover rows of the last round: their own, larger number of warps per row when the round is at most half full
        const uint32_t per_round = grid * ((uint32_t)kFfnWarps / Q.ks), full = P.out_total / per_round, left = P.out_total - full * per_round;
        Q.tail_rows = 0;
        Q.ks_tail = Q.ks;
        if (full >= 1u && left > 0u && left * 2u <= per_round && g_ffn_ks_override >= 0) {
            const uint32_t kt = ffn_pick_ks(left, nh >> 5, (uint32_t)FmtTraits<FD>::rows_max_len, grid, (uint32_t)kFfnWarps);
            if (kt > Q.ks) {
                Q.tail_rows = left;
                Q.ks_tail = kt;
            }
        }
    }
    Q.ks_gu = ffn_pick_ks(P.ffn_local, nx >> 5, (uint32_t)FmtTraits<FG>::rows_max_len, grid, kFfnTeam);
    Q.trace = g_ffn_trace_on;
    FfnTpPeers pp = peers;
    void *args[] = {&Q, &pp};
    return (int)cudaLaunchCooperativeKernel((const void *)ffn_tp_kernel<FG, FD>, dim3(grid), dim3(kFfnWarps * 32), args, smem, s);
}

struct Tuning {
    int ks = 0;          // 0 = heuristic
    int grid_mult = 0;   // CTAs launched per resident CTA slot; 0 = heuristic
    int no_pdl = 0;      // plain launches (for A/B timing)
    int no_rows_kernel = 0;
};
Tuning g_tune;

template <int FMT> size_t stream_smem_bytes(uint32_t n_rows, uint32_t n_sub, int nb)
{
    const size_t x = (((size_t)n_rows * n_sub * FmtTraits<FMT>::x_bytes) + 15u) & ~(size_t)15u;
    return x + 2u * kWarpsPerCta * (size_t)nb * sizeof(float);
}

template <int FMT, int NB, int LEN>
int launch_rows(cudaStream_t s, const void *w, const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
                uint32_t n_rows, uint32_t grid, size_t smem)
{
    const uint32_t n_iters = in_dim >> 10, n_units = n_iters / LEN + (n_iters % LEN ? 1u : 0u);
    const bool tail = rows_shared_tail(out_dim, grid * kWarpsPerCta, n_units) != 0u;
    auto launch = [&](auto kernel) {
        if (g_tune.no_pdl) {
            kernel<<<grid, kWarpsPerCta * 32, smem, s>>>((const uint8_t *)w, (const uint8_t *)xq, y, in_dim, out_dim, n_rows);
            return (int)cudaGetLastError();
        }
        return (int)launch_pdl(kernel, dim3(grid), dim3(kWarpsPerCta * 32), smem, s, (const uint8_t *)w, (const uint8_t *)xq, y, in_dim,
                               out_dim, n_rows);
    };
    return tail ? launch(matvec_rows_kernel<FMT, NB, LEN, true>) : launch(matvec_rows_kernel<FMT, NB, LEN, false>);
}

template <int FMT, int NB, bool DUMP>
int launch_one(cudaStream_t s, const void *w, const void *xq, float *y, int32_t *idots,
               uint32_t in_dim, uint32_t out_dim, uint32_t n_rows)
{
    const uint32_t n_sub = in_dim >> 5, n_iters = (n_sub + 31u) >> 5;
    const size_t smem = stream_smem_bytes<FMT>(n_rows, n_sub, NB);
    if (smem > kMaxStageBytesHost) return RC_ERR_TOO_MANY_ROWS; // caller splits the batch
    uint32_t resident = (uint32_t)MinBlocks<NB>::v;
    resident = min(resident, (uint32_t)((227 * 1024) / (smem + 1024)));
    if (resident == 0) resident = 1;
    const uint32_t slots = (uint32_t)sm_count() * resident * kWarpsPerCta;
    // One warp per row is best whenever the rows fill most of the warp slots; only narrower
    // matrices split rows across warps (never leaving a warp without an iteration).
    uint32_t ks = 1;
    while (ks < (uint32_t)kWarpsPerCta && ks * 2u <= n_iters && (uint64_t)out_dim * ks * 4u < 3ull * slots) ks *= 2u;
    if (g_tune.ks > 0) {
        ks = 1;
        while (ks * 2u <= (uint32_t)g_tune.ks && ks * 2u <= (uint32_t)kWarpsPerCta && ks * 2u <= n_iters) ks *= 2u;
    }
    if (DUMP) ks = 1;
    if constexpr (!DUMP && NB >= 2) {
        // Several activation rows: a warp owns R consecutive weight rows (each activation block is read from
        // shared memory once for all R).  R as large as still leaves two CTAs of work per SM: on a 5120-row
        // matrix four rows per warp would leave most warp slots empty (measured: batch 4, 5120 x 5120 Q5_K,
        // 24 us with R = 4).
        constexpr int RMAX = MultiRows<NB>::v;
        if (n_sub % 32u == 0 && !g_tune.no_rows_kernel && (uint64_t)out_dim >= (uint64_t)sm_count() * kWarpsPerCta) {
            const uint32_t capacity = (uint32_t)sm_count() * min(resident, (uint32_t)kMultiMinBlocks);
            int r_pick = RMAX;
            while (r_pick > 1 && (uint64_t)out_dim < 2ull * (uint64_t)sm_count() * kWarpsPerCta * r_pick) r_pick >>= 1;
            if (kCodebook<FMT> && r_pick < RMAX) r_pick = 1; // the codebook lookups hold more registers per row (measured: 11.4 us against 18.4)
            if (g_tune.ks > 0 && g_tune.ks <= RMAX) r_pick = g_tune.ks; // measurement override
            const size_t xsm = (((size_t)n_rows * n_sub * FmtTraits<FMT>::x_bytes) + 15u) & ~(size_t)15u;
            auto go = [&](auto rtag) -> int {
                constexpr int R = decltype(rtag)::value;
                const uint32_t n_cta_rows = (out_dim + kWarpsPerCta * R - 1u) / (kWarpsPerCta * R);
                const uint32_t grid = min(n_cta_rows, capacity * (n_cta_rows >= 3u * capacity ? 2u : 1u));
                if (g_tune.no_pdl) {
                    matvec_multi_kernel<FMT, NB, R><<<grid, kWarpsPerCta * 32, xsm, s>>>((const uint8_t *)w, (const uint8_t *)xq, y, in_dim,
                                                                                        out_dim, n_rows);
                    return (int)cudaGetLastError();
                }
                return (int)launch_pdl(matvec_multi_kernel<FMT, NB, R>, dim3(grid), dim3(kWarpsPerCta * 32), xsm, s, (const uint8_t *)w,
                                       (const uint8_t *)xq, y, in_dim, out_dim, n_rows);
            };
            if constexpr (RMAX >= 4) {
                if (r_pick >= 4) return go(std::integral_constant<int, 4>{});
            }
            if (r_pick >= 2) return go(std::integral_constant<int, 2>{});
            if constexpr (NB <= 4) return go(std::integral_constant<int, 1>{});
            else return go(std::integral_constant<int, 2>{});
        }
    }
    if constexpr (!DUMP && NB <= 4) {
        if (ks == 1 && n_sub % 32u == 0 && !g_tune.no_rows_kernel) {
            // group length: as long as the format's registers allow, the whole row if it is shorter
            uint32_t len = min(n_iters, (uint32_t)FmtTraits<FMT>::rows_max_len);
            if (len < 3) len = 3; // shorter rows run as one short group of the LEN = 3 kernel
            // with several activation rows the math dominates and a ragged last group costs more than
            // the leaner loop saves: those shapes stay on the general kernel
            if (NB > 1 && n_iters % len != 0) len = 0;
            const uint32_t capacity = (uint32_t)sm_count() * resident;
            const uint32_t n_cta_rows = (out_dim + kWarpsPerCta - 1u) / kWarpsPerCta;
            const uint32_t mult = g_tune.grid_mult > 0 ? (uint32_t)g_tune.grid_mult : (n_cta_rows >= 3u * capacity ? 2u : 1u);
            const uint32_t grid = min(n_cta_rows, capacity * mult);
            const size_t xsm = (((size_t)n_rows * n_sub * FmtTraits<FMT>::x_bytes) + 15u) & ~(size_t)15u;
#define RC_ROWS(L) \
    case L: \
        if (L <= FmtTraits<FMT>::rows_max_len) \
            return launch_rows<FMT, NB, L>(s, w, xq, y, in_dim, out_dim, n_rows, grid, xsm); \
        break;
            switch (len) {
                RC_ROWS(3)
                RC_ROWS(4)
                RC_ROWS(5)
            }
#undef RC_ROWS
        }
    }
    const uint32_t rb_rows = kWarpsPerCta / ks;
    const uint32_t n_blocks = (out_dim + rb_rows - 1u) / rb_rows;
    // Two CTAs per resident slot even out the tail once a CTA has three or more row blocks.
    const uint32_t capacity = (uint32_t)sm_count() * resident;
    const uint32_t mult = g_tune.grid_mult > 0 ? (uint32_t)g_tune.grid_mult : (n_blocks >= 3u * capacity ? 2u : 1u);
    const uint32_t grid = min(n_blocks, capacity * mult);
    if (g_tune.no_pdl) {
        matvec_stream_kernel<FMT, NB, DUMP><<<grid, kWarpsPerCta * 32, smem, s>>>(
            (const uint8_t *)w, (const uint8_t *)xq, y, idots, in_dim, out_dim, n_rows, ks);
        return (int)cudaGetLastError();
    }
    return (int)launch_pdl(matvec_stream_kernel<FMT, NB, DUMP>, dim3(grid), dim3(kWarpsPerCta * 32), smem, s,
                           (const uint8_t *)w, (const uint8_t *)xq, y, idots, in_dim, out_dim, n_rows, ks);
}

template <int FMT, bool DUMP>
int launch_fmt(cudaStream_t s, const void *w, const void *xq, float *y, int32_t *idots,
               uint32_t in_dim, uint32_t out_dim, uint32_t n_rows)
{
    if (n_rows == 1) return launch_one<FMT, 1, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    if (n_rows == 2) return launch_one<FMT, 2, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    if (n_rows <= 4) return launch_one<FMT, 4, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    if (n_rows <= 8) return launch_one<FMT, 8, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    return launch_one<FMT, 16, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
}

template <bool DUMP>
int launch_any(cudaStream_t s, int type, const void *w, const void *xq, float *y, int32_t *idots,
               uint32_t in_dim, uint32_t out_dim, uint32_t n_rows)
{
    switch (type) {
    case Q4_0: return launch_fmt<Q4_0, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case Q5_1: return launch_fmt<Q5_1, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case Q8_0: return launch_fmt<Q8_0, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case Q4_K: return launch_fmt<Q4_K, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case Q5_K: return launch_fmt<Q5_K, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case Q6_K: return launch_fmt<Q6_K, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case IQ4_XS: return launch_fmt<IQ4_XS, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    case IQ3_S: return launch_fmt<IQ3_S, DUMP>(s, w, xq, y, idots, in_dim, out_dim, n_rows);
    }
    return RC_ERR_BAD_TYPE;
}

template <int FMT, int NB, bool DUMP> int set_attr_one()
{
    return (int)cudaFuncSetAttribute(matvec_stream_kernel<FMT, NB, DUMP>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
}

constexpr int kGroupedBN = 16;

template <int FMT, int NB> int set_attr_rows()
{
    int rc = 0;
    if constexpr (NB >= 2) {
        rc |= (int)cudaFuncSetAttribute(matvec_multi_kernel<FMT, NB, MultiRows<NB>::v>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kMaxStageBytesHost);
        rc |= (int)cudaFuncSetAttribute(matvec_multi_kernel<FMT, NB, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
        rc |= (int)cudaFuncSetAttribute(matvec_multi_kernel<FMT, NB, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
    }
    rc |= (int)cudaFuncSetAttribute(matvec_rows_kernel<FMT, NB, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
    rc |= (int)cudaFuncSetAttribute(matvec_rows_kernel<FMT, NB, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
    rc |= (int)cudaFuncSetAttribute(matvec_rows_kernel<FMT, NB, 5>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
    rc |= (int)cudaFuncSetAttribute(matvec_rows_kernel<FMT, NB, 3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
    rc |= (int)cudaFuncSetAttribute(matvec_rows_kernel<FMT, NB, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
    rc |= (int)cudaFuncSetAttribute(matvec_rows_kernel<FMT, NB, 5, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
    return rc;
}

template <int FMT> int set_attr_fmt()
{
    int rc = 0;
    rc |= set_attr_one<FMT, 1, false>();
    rc |= set_attr_one<FMT, 2, false>();
    rc |= set_attr_one<FMT, 4, false>();
    rc |= set_attr_one<FMT, 8, false>();
    rc |= set_attr_one<FMT, 16, false>();
    rc |= set_attr_one<FMT, 1, true>();
    rc |= set_attr_one<FMT, 2, true>();
    rc |= set_attr_one<FMT, 4, true>();
    rc |= set_attr_one<FMT, 8, true>();
    rc |= set_attr_one<FMT, 16, true>();
    rc |= set_attr_rows<FMT, 1>() | set_attr_rows<FMT, 2>() | set_attr_rows<FMT, 4>();
    rc |= (int)cudaFuncSetAttribute(matvec_multi_kernel<FMT, 8, MultiRows<8>::v>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
    rc |= (int)cudaFuncSetAttribute(matvec_multi_kernel<FMT, 16, MultiRows<16>::v>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
    rc |= (int)cudaFuncSetAttribute(matvec_grouped_kernel<FMT, kGroupedBN>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
    return rc;
}

template <int FMT>
int launch_grouped_fmt(cudaStream_t s, const void *slab, size_t bpe, const int32_t *expert_off,
                       const int32_t *tile_off, uint32_t n_expert, const void *xq, float *y,
                       uint32_t in_dim, uint32_t out_dim, uint32_t n_entries)
{
    constexpr int BN = kGroupedBN;
    const uint32_t n_sub = in_dim >> 5;
    const size_t smem = stream_smem_bytes<FMT>(BN, n_sub, BN);
    if (smem > kMaxStageBytesHost) return RC_ERR_BAD_SHAPE;
    const uint32_t n_blocks = (out_dim + kWarpsPerCta - 1) / kWarpsPerCta;
    const uint32_t gx = min(n_blocks, 8u);
    const uint32_t tiles_ub = ((n_entries + kGroupedTile - 1) / kGroupedTile + n_expert) * (kGroupedTile / BN);
    if (tiles_ub > 65535u) return RC_ERR_BAD_ARGUMENT;
    matvec_grouped_kernel<FMT, BN><<<dim3(gx, tiles_ub), kWarpsPerCta * 32, smem, s>>>(
        (const uint8_t *)slab, bpe, expert_off, tile_off, n_expert, (const uint8_t *)xq, y, in_dim,
        out_dim);
    return (int)cudaGetLastError();
}

template <int FMT>
int launch_expert_fmt(cudaStream_t s, const void *slab, size_t bpe, const int32_t *ids, uint32_t n_expert, const void *xq,
                      float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_used, uint32_t n_tok, uint32_t tok_stride,
                      uint32_t slot_stride)
{
    const uint32_t n_sub = in_dim >> 5, n_iters = (n_sub + 31u) >> 5;
    const size_t smem = stream_smem_bytes<FMT>(1, n_sub, 1);
    if (smem > kMaxStageBytesHost) return RC_ERR_BAD_SHAPE;
    // all slots of all tokens run at once: split rows across warps only while they leave warp slots idle
    const uint32_t slots = (uint32_t)sm_count() * (uint32_t)MinBlocks<1>::v * kWarpsPerCta;
    const uint64_t rows_total = (uint64_t)out_dim * n_used * n_tok;
    uint32_t ks = 1;
    while (ks < (uint32_t)kWarpsPerCta && ks * 2u <= n_iters && rows_total * ks * 4u < 3ull * slots) ks *= 2u;
    const uint32_t rb_rows = kWarpsPerCta / ks;
    const uint32_t gx = (out_dim + rb_rows - 1u) / rb_rows;
    for (uint32_t t0 = 0; t0 < n_tok; t0 += 65535u) {
        const uint32_t nt = min(65535u, n_tok - t0);
        cudaError_t e = launch_pdl(moe_expert_matvec_kernel<FMT>, dim3(gx, n_used, nt), dim3(kWarpsPerCta * 32), smem, s,
                                   (const uint8_t *)slab, bpe, ids + (size_t)t0 * n_used, n_expert,
                                   (const uint8_t *)xq + (size_t)t0 * tok_stride * RC_BLOCKQ8_BYTES,
                                   y + (size_t)t0 * n_used * out_dim, in_dim, out_dim, n_used, tok_stride, slot_stride, ks);
        if (e != cudaSuccess) return (int)e;
    }
    return RC_OK;
}

template <int FMT>
int launch_gate_up_swiglu_fmt(cudaStream_t s, const void *gate_slab, const void *up_slab, size_t bpe, const int32_t *ids,
                              uint32_t n_expert, const void *xq, float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_used,
                              uint32_t n_tok, uint32_t tok_stride, uint32_t slot_stride)
{
    const uint32_t n_sub = in_dim >> 5;
    if (n_sub % 32u) return RC_ERR_BAD_SHAPE; // whole iterations only
    const size_t smem = stream_smem_bytes<FMT>(1, n_sub, 1);
    if (smem > kMaxStageBytesHost) return RC_ERR_BAD_SHAPE;
    const uint32_t gx = (out_dim + kWarpsPerCta - 1u) / kWarpsPerCta;
    for (uint32_t t0 = 0; t0 < n_tok; t0 += 65535u) {
        const uint32_t nt = min(65535u, n_tok - t0);
        cudaError_t e = launch_pdl(moe_gate_up_swiglu_kernel<FMT>, dim3(gx, n_used, nt), dim3(kWarpsPerCta * 32), smem, s,
                                   (const uint8_t *)gate_slab, (const uint8_t *)up_slab, bpe, ids + (size_t)t0 * n_used, n_expert,
                                   (const uint8_t *)xq + (size_t)t0 * tok_stride * RC_BLOCKQ8_BYTES,
                                   y + (size_t)t0 * n_used * out_dim, in_dim, out_dim, n_used, tok_stride, slot_stride);
        if (e != cudaSuccess) return (int)e;
    }
    return RC_OK;
}

template <int FMT> int set_attr_expert()
{
    if ((int)cudaFuncSetAttribute(moe_gate_up_swiglu_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost))
        return 1;
    return (int)cudaFuncSetAttribute(moe_expert_matvec_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStageBytesHost);
}

} // namespace

int launch_moe_expert_matvec(cudaStream_t s, int type, const void *slab, size_t bpe, const int32_t *ids, uint32_t n_expert,
                             const void *xq, float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_used, uint32_t n_tok,
                             uint32_t tok_stride, uint32_t slot_stride)
{
#define RC_E(F) return launch_expert_fmt<F>(s, slab, bpe, ids, n_expert, xq, y, in_dim, out_dim, n_used, n_tok, tok_stride, slot_stride)
    switch (type) {
    case Q4_0: RC_E(Q4_0);
    case Q5_1: RC_E(Q5_1);
    case Q8_0: RC_E(Q8_0);
    case Q4_K: RC_E(Q4_K);
    case Q5_K: RC_E(Q5_K);
    case Q6_K: RC_E(Q6_K);
    case IQ4_XS: RC_E(IQ4_XS);
    case IQ3_S: RC_E(IQ3_S);
    }
#undef RC_E
    return RC_ERR_BAD_TYPE;
}

int launch_moe_gate_up_swiglu(cudaStream_t s, int type, const void *gate_slab, const void *up_slab, size_t bpe, const int32_t *ids,
                              uint32_t n_expert, const void *xq, float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_used,
                              uint32_t n_tok, uint32_t tok_stride, uint32_t slot_stride)
{
#define RC_S(F) return launch_gate_up_swiglu_fmt<F>(s, gate_slab, up_slab, bpe, ids, n_expert, xq, y, in_dim, out_dim, n_used, n_tok, tok_stride, slot_stride)
    switch (type) {
    case Q4_0: RC_S(Q4_0);
    case Q5_1: RC_S(Q5_1);
    case Q8_0: RC_S(Q8_0);
    case Q4_K: RC_S(Q4_K);
    case Q5_K: RC_S(Q5_K);
    case Q6_K: RC_S(Q6_K);
    case IQ4_XS: RC_S(IQ4_XS);
    case IQ3_S: RC_S(IQ3_S);
    }
#undef RC_S
    return RC_ERR_BAD_TYPE;
}

int matvec_set_attributes()
{
    int rc = 0;
    rc |= set_attr_fmt<Q4_0>();
    rc |= set_attr_fmt<Q5_1>();
    rc |= set_attr_fmt<Q8_0>();
    rc |= set_attr_fmt<Q4_K>();
    rc |= set_attr_fmt<Q5_K>();
    rc |= set_attr_fmt<Q6_K>();
    rc |= set_attr_fmt<IQ4_XS>();
    rc |= set_attr_fmt<IQ3_S>();
    rc |= set_attr_expert<Q4_0>() | set_attr_expert<Q5_1>() | set_attr_expert<Q8_0>() | set_attr_expert<Q4_K>() | set_attr_expert<Q5_K>() |
          set_attr_expert<Q6_K>() | set_attr_expert<IQ4_XS>() | set_attr_expert<IQ3_S>();
    return rc;
}

// dp4a grouped GEMM: every 16-token half tile streams its expert's weights once.
int launch_matvec_grouped(cudaStream_t s, int type, const void *slab, size_t bpe,
                          const int32_t *expert_off, const int32_t *tile_off, uint32_t n_expert,
                          const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
                          uint32_t n_entries)
{
#define RC_G(F) return launch_grouped_fmt<F>(s, slab, bpe, expert_off, tile_off, n_expert, xq, y, in_dim, out_dim, n_entries)
    switch (type) {
    case Q4_0: RC_G(Q4_0);
    case Q5_1: RC_G(Q5_1);
    case Q8_0: RC_G(Q8_0);
    case Q4_K: RC_G(Q4_K);
    case Q5_K: RC_G(Q5_K);
    case Q6_K: RC_G(Q6_K);
    case IQ4_XS: RC_G(IQ4_XS);
    case IQ3_S: RC_G(IQ3_S);
    }
#undef RC_G
    return RC_ERR_BAD_TYPE;
}

uint32_t matvec_grouped_bn() { return kGroupedTile; }

void matvec_set_tuning(int ks, int grid_mult, int no_pdl)
{
    g_tune.ks = ks;
    g_tune.grid_mult = grid_mult;
    g_tune.no_pdl = no_pdl & 1;
    g_tune.no_rows_kernel = (no_pdl >> 1) & 1;
    g_ffn_plain_launch = (no_pdl >> 2) & 1;
    g_ffn_ks_override = ks;
}
bool matvec_pdl_enabled() { return !g_tune.no_pdl; }

int launch_matvec(cudaStream_t s, int type, const void *w, const void *xq, float *y,
                  uint32_t in_dim, uint32_t out_dim, uint32_t n_rows, int32_t *idots)
{
    // Split the batch when the staged activations of all rows do not fit in shared memory;
    // each part reads the weights once more, which only very long rows ever need.
    uint32_t part = n_rows;
    const uint32_t n_sub = in_dim >> 5;
    const size_t per_row = (size_t)n_sub * 48 + 2u * kWarpsPerCta * sizeof(float);
    while (part > 1 && (size_t)part * per_row + 64 > kMaxStageBytesHost) part = (part + 1) / 2;
    if ((size_t)part * per_row + 64 > kMaxStageBytesHost) return RC_ERR_BAD_SHAPE;
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

size_t ffn_decode_work_bytes(uint32_t) { return 64; }

// Copies out CTA 0's marks [0, 16) and the per-mark maxima over CTAs [16, 32), clears the maxima and switches the marks on.
int ffn_read_trace(void *out, size_t bytes)
{
    unsigned long long buf[32] = {0};
    cudaError_t e = cudaMemcpyFromSymbol(buf, g_ffn_trace, sizeof(g_ffn_trace));
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(buf + 16, g_ffn_trace_max, sizeof(g_ffn_trace_max));
    if (e != cudaSuccess) return (int)e;
    const unsigned long long zeros[16] = {0};
    e = cudaMemcpyToSymbol(g_ffn_trace_max, zeros, sizeof(zeros));
    if (bytes >= sizeof(buf) + sizeof(g_ffn_cta)) cudaMemcpyFromSymbol((char *)out + sizeof(buf), g_ffn_cta, sizeof(g_ffn_cta));
    g_ffn_trace_on = 1;
    memcpy(out, buf, bytes < sizeof(buf) ? bytes : sizeof(buf));
    return (int)e;
}

int ffn_device_error(unsigned int *out, bool clear)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, g_ffn_error, sizeof(unsigned int));
    if (e == cudaSuccess && clear && *out) {
        const unsigned int zero = 0;
        e = cudaMemcpyToSymbol(g_ffn_error, &zero, sizeof(unsigned int));
    }
    return (int)e;
}

int launch_ffn_decode(cudaStream_t s, int gate_type, int down_type, const void *gate, const void *up, const void *down, const float *x,
                      uint32_t in_dim, uint32_t ffn_local, uint32_t ffn_total, uint32_t ffn_begin, uint32_t out_local,
                      uint32_t out_total, uint32_t out_begin, uint32_t world, uint32_t rank, void *const *h_peers,
                      void *const *y_peers, float *y, void *work)
{
    FfnParams P;
    P.gate = (const uint8_t *)gate;
    P.up = (const uint8_t *)up;
    P.down = (const uint8_t *)down;
    P.x = x;
    P.y = y;
    P.sync = reinterpret_cast<unsigned long long *>(work);
    P.in_dim = in_dim;
    P.ffn_local = ffn_local;
    P.ffn_total = ffn_total;
    P.ffn_begin = ffn_begin;
    P.out_local = out_local;
    P.out_total = out_total;
    P.out_begin = out_begin;
    P.world = world;
    P.rank = rank;
    P.ks = 1;
    P.ks_gu = 1;
    P.trace = 0;
    FfnPeers peers;
    for (uint32_t r = 0; r < RC_MAX_PEERS; r++) {
        peers.h[r] = r < world ? (float *)h_peers[r] : nullptr;
        peers.y[r] = r < world ? (float *)y_peers[r] : nullptr;
    }
#define RC_FFN(G, D) \
    if (gate_type == G && down_type == D) return launch_ffn<G, D>(s, P, peers);
    RC_FFN(Q4_K, Q6_K)
    RC_FFN(Q4_K, Q4_K)
    RC_FFN(Q5_K, Q6_K)
    RC_FFN(Q6_K, Q6_K)
    RC_FFN(Q8_0, Q8_0)
    RC_FFN(Q4_0, Q4_0)
#undef RC_FFN
    return RC_ERR_BAD_TYPE;
}

int launch_ffn_decode_tp(cudaStream_t s, int gate_type, int down_type, const void *gate, const void *up, const void *down, const float *x,
                         float *y, uint32_t in_dim, uint32_t ffn_local, uint32_t out_total, uint32_t world, uint32_t rank,
                         void *const *part_peers, void *work)
{
    FfnTpParams P;
    P.gate = (const uint8_t *)gate;
    P.up = (const uint8_t *)up;
    P.down = (const uint8_t *)down;
    P.x = x;
    P.y = y;
    P.sync = reinterpret_cast<unsigned long long *>(work);
    P.h = reinterpret_cast<float *>((uint8_t *)work + 64);
    P.in_dim = in_dim;
    P.ffn_local = ffn_local;
    P.out_total = out_total;
    P.world = world;
    P.rank = rank;
    P.ks = 1;
    P.ks_gu = 1;
    P.trace = 0;
    P.tail_rows = 0;
    P.ks_tail = 1;
    FfnTpPeers peers;
    for (uint32_t r = 0; r < RC_MAX_PEERS; r++) peers.part[r] = r < world ? (float *)part_peers[r] : nullptr;
#define RC_FFN(G, D) \
    if (gate_type == G && down_type == D) return launch_ffn_tp<G, D>(s, P, peers);
    RC_FFN(Q4_K, Q6_K)
    RC_FFN(Q4_K, Q4_K)
    RC_FFN(Q5_K, Q6_K)
    RC_FFN(Q6_K, Q6_K)
    RC_FFN(Q8_0, Q8_0)
    RC_FFN(Q4_0, Q4_0)
#undef RC_FFN
    return RC_ERR_BAD_TYPE;
}

size_t ffn_decode_tp_work_bytes(uint32_t ffn_local) { return 64 + (size_t)ffn_local * sizeof(float); }

} // namespace rc
