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

__device__ __forceinline__ uint32_t ld_sup32(const uint8_t *p, bool aligned4)
{
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
    __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t sup, bool a4)
    {
        q = ld_stream_u4(p.nib + idx * 16);
        const uint32_t sm = ld_nc_u16(p.sc + idx * 2);
        const uint32_t dd = ld_sup32(p.sup + sup * 4, a4);
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
    __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t sup, bool a4)
    {
        const uint4 q = ld_stream_u4(p.nib + idx * 16);
        const uint32_t qh = ld_stream_u32(p.aux + idx * 4);
        const uint32_t sm = ld_nc_u16(p.sc + idx * 2);
        const uint32_t dd = ld_sup32(p.sup + sup * 4, a4);
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
    __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t sup, bool)
    {
        const uint4 q = ld_stream_u4(p.nib + idx * 16);
        const uint2 h = ld_stream_u2(p.aux + idx * 8);
        const uint32_t sm = ld_nc_u16(p.sc + idx * 2);
        const float d = f16_bits_to_f32(ld_nc_u16(p.sup + sup * 2));
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
    __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t, bool)
    {
        wl = ld_stream_u4(p.nib + idx * 16);
        wh = ld_stream_u4(p.aux + idx * 16);
        dw = f16_bits_to_f32(ld_nc_u16(p.sc + idx * 2));
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
    __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t, bool)
    {
        q = ld_stream_u4(p.nib + idx * 16);
        dw = f16_bits_to_f32(ld_nc_u16(p.sc + idx * 2));
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
    __device__ __forceinline__ void load(const Planes &p, size_t idx, size_t, bool)
    {
        const uint4 q = ld_stream_u4(p.nib + idx * 16);
        dw = f16_bits_to_f32(ld_nc_u16(p.sc + idx * 2));
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
                wb[r].load(p, (size_t)row * p.nsp + sb, (size_t)row * p.n_super + (sb >> 3), sup_a4);
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
                if (lane == 0 && b < (int)n_rows && row0 + r < out_dim)
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
    return rc;
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
