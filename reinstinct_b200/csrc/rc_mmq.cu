// int8 MMQ GEMM (dense prefill and expert-grouped) on the 5th-generation tensor cores.
//
// What is computed is the block-scaled contraction of the reference's MMQ kernels
// (kernels/mmq_gemm_q4k_repacked.cpp:63-208 and siblings, kernels/mmq_gemm_q4k_grouped.cpp:38-165):
//   Y[tok][row] = sum_sb  dsc[row,sb] * dx[tok,sb] * idot[row,tok,sb]  -  deff[row,sb] * xsum[tok,sb]
// with idot the exact integer dot of one 32-wide sub-block.  Every sub-block carries its own f32
// scale on both sides, so an int32 accumulator cannot run across sub-blocks: each K=32
// tcgen05.mma (kind::i8, int32 accumulator in tensor memory) is one sub-block, and its 128xBN
// int32 tile is drained from tensor memory, converted and scaled on the CUDA cores into f32
// register accumulators.  That drain, not the tensor pipe, bounds the kernel.
//
// One persistent CTA per SM, 12 warps with fixed roles:
//   warp 0        one thread issues TMA tile loads of the raw nibble plane (a 16-byte-wide,
//                 128-row box per sub-block, rows past the end zero-filled by the TMA unit)
//   warp 1        one thread issues the MMAs and their commits
//   warps 2..3    expand raw 4/5/8-bit weights to int8 in the MMA's K-major core-matrix layout,
//                 and copy the int8 quants of the BlockQ8 activations (40-byte records, which
//                 TMA cannot tile) into the same layout, with their scales beside them
//   warps 4..11   epilogue: tcgen05.ld the int32 tile, scale, accumulate; write Y at tile end
// Stages (4 sub-blocks each) flow through mbarrier rings raw -> operands -> tensor memory
// (4 accumulator buffers of BN columns).  Every wait is bounded: when a limit runs out the
// kernel records a code in g_mmq_error, raises a CTA-wide abort flag and every role leaves its
// loop, so that tensor memory is freed and the launch ends.
//
// Operand layout (no swizzle, K-major): a 128x32-byte operand is stored as [half][row][16 B],
// i.e. core matrices of 8 rows x 16 bytes, 128 bytes apart along rows (stride byte offset) and
// rows*16 bytes apart along K (leading byte offset).  A repacked-v2 nibble chunk is exactly one
// row of that: its low nibbles are K 0..15, its high nibbles K 16..31.
#include <cuda.h>

#include "rc_common.cuh"
#include "rc_internal.h"
#include "rc_tc.cuh"

namespace rc {
namespace {

constexpr int kKS = 4;       // sub-blocks (K=32 MMA steps) per pipeline stage
constexpr int kStages = 4;   // operand ring depth
constexpr int kBufs = 4;     // tensor-memory accumulator buffers

__device__ unsigned int g_mmq_error;

struct MmqParams {
    const uint8_t *w;           // dense weight, or the expert slab
    size_t bytes_per_expert;
    const int32_t *expert_off;  // grouped only (nullptr = dense)
    const int32_t *tile_off;
    uint32_t n_expert;
    const uint8_t *xq;
    float *y;
    uint32_t in_dim, out_dim;
    uint32_t n_tok;             // P (dense) or n_entries (grouped)
    uint32_t planar;            // activations come from rc_matmul's planar scratch through TMA (int8 kernel)
    uint32_t b_tma;             // BlockQ8 rows are fetched by TMA (base 16-byte aligned, even sub-block count)
    uint32_t debug;             // measurement aid: bit mask of pipeline parts to skip (results invalid)
};

// Bounded wait: gives up after kWaitLimitCycles SM cycles (about half a second).  False when the limit ran out (records
// `code`, raises the abort flag) or when another role already raised the flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t code)
{
    if (mbar_try(bar, parity)) return true;
    // the limit is kept on the SM's own cycle counter, first read after 64 failed polls: a wait
    // that is about to succeed never pays for a timer read
    long long t0 = 0;
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitCycles) break;
        }
    }
    atomicExch(&g_mmq_error, code);
    *abort_flag = 1u;
    return false;
}

// Instruction descriptor: int32 accumulator, signed 8-bit A and B, both K-major, M = 128.
__host__ __device__ constexpr uint32_t make_idesc_i8(uint32_t n)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

// ---- per-format pieces -----------------------------------------------------------------------------

template <int FMT> struct MmqTraits {
    static constexpr bool has_min = (FMT == Q4_K || FMT == Q5_K);  // "- deff * xsum" term
    static constexpr int raw_planes = (FMT == Q8_0) ? 2 : 1;       // 16-byte planes fetched by TMA
    static constexpr uint32_t raw_bytes = raw_planes * kBM * 16;   // per sub-block
};

// 16 raw bytes (and what else the format needs) of one (row, sub-block) -> the 32 int8 weights
// as the kernels' integer dots define them: lo = weights 0..15, hi = weights 16..31.
template <int FMT>
__device__ __forceinline__ void expand_weights(const uint4 &q, const uint4 &q2, uint32_t extra, uint4 &lo, uint4 &hi)
{
    const uint32_t M = 0x0F0F0F0Fu;
    if constexpr (FMT == Q4_K) {
        lo = make_uint4(q.x & M, q.y & M, q.z & M, q.w & M);
        hi = make_uint4((q.x >> 4) & M, (q.y >> 4) & M, (q.z >> 4) & M, (q.w >> 4) & M);
    } else if constexpr (FMT == Q5_K) {
        const uint32_t qh = extra; // src/quant/q5_k.rs:134-137
        lo = make_uint4((q.x & M) | bits4_to_bit4(qh), (q.y & M) | bits4_to_bit4(qh >> 8),
                        (q.z & M) | bits4_to_bit4(qh >> 16), (q.w & M) | bits4_to_bit4(qh >> 24));
        hi = make_uint4(((q.x >> 4) & M) | bits4_to_bit4(qh >> 4), ((q.y >> 4) & M) | bits4_to_bit4(qh >> 12),
                        ((q.z >> 4) & M) | bits4_to_bit4(qh >> 20), ((q.w >> 4) & M) | bits4_to_bit4(qh >> 28));
    } else if constexpr (FMT == Q8_0) {
        lo = q;
        hi = q2;
    } else if constexpr (FMT == Q4_0) {
        // nibble - 8 as int8: flip bit 3, then sign-extend it (0x08 * 0x1E = 0xF0 stays in its byte)
        auto sub8 = [](uint32_t v) {
            const uint32_t t = v ^ 0x08080808u;
            return t | ((t & 0x08080808u) * 0x1Eu);
        };
        lo = make_uint4(sub8(q.x & M), sub8(q.y & M), sub8(q.z & M), sub8(q.w & M));
        hi = make_uint4(sub8((q.x >> 4) & M), sub8((q.y >> 4) & M), sub8((q.z >> 4) & M), sub8((q.w >> 4) & M));
    } else { // IQ4_XS: codebook lookup, then undo iq4_lookup8's (low, high) interleave
        int a0, a1, b0, b1, c0, c1, d0, d1;
        iq4_lookup8<FMT>(q.x, a0, a1);
        iq4_lookup8<FMT>(q.y, b0, b1);
        iq4_lookup8<FMT>(q.z, c0, c1);
        iq4_lookup8<FMT>(q.w, d0, d1);
        lo = make_uint4(__byte_perm(a0, a1, 0x6420), __byte_perm(b0, b1, 0x6420), __byte_perm(c0, c1, 0x6420),
                        __byte_perm(d0, d1, 0x6420));
        hi = make_uint4(__byte_perm(a0, a1, 0x7531), __byte_perm(b0, b1, 0x7531), __byte_perm(c0, c1, 0x7531),
                        __byte_perm(d0, d1, 0x7531));
    }
}

// Scale words of one weight row for the sub-blocks of one stage.
struct StageScales {
    uint32_t s[kKS]; // K-quants: sc | m << 8;  others: the f16 block scale
    uint32_t dd;     // K-quants: d | dmin << 16 of the stage's superblock (a stage never straddles two)
};

template <int FMT>
__device__ __forceinline__ void load_scales(StageScales &o, const Planes &p, bool sup_a4, uint32_t row, uint32_t k0,
                                            uint32_t nsteps)
{
#pragma unroll
    for (int j = 0; j < kKS; j++)
        if (j < (int)nsteps) o.s[j] = ld_nc_u16(p.sc + ((size_t)row * p.nsp + k0 + j) * 2);
    if constexpr (MmqTraits<FMT>::has_min) {
        const uint8_t *sp = p.sup + ((size_t)row * p.n_super + (k0 >> 3)) * 4;
        o.dd = sup_a4 ? __ldg(reinterpret_cast<const uint32_t *>(sp)) : (ld_nc_u16(sp) | (ld_nc_u16(sp + 2) << 16));
    }
}

struct Tile {
    uint32_t e, m0, tok0, n_valid;
};

template <int BN>
__device__ __forceinline__ uint32_t tile_count(const MmqParams &P, uint32_t tiles_m)
{
    if (P.expert_off) return tiles_m * (uint32_t)P.tile_off[P.n_expert];
    return tiles_m * ((P.n_tok + BN - 1) / BN);
}

// Token tile fastest: CTAs running at the same time share a weight row tile.
template <int BN>
__device__ __forceinline__ Tile decode_tile(const MmqParams &P, uint32_t id)
{
    Tile t;
    if (P.expert_off) {
        const uint32_t T = (uint32_t)P.tile_off[P.n_expert];
        const uint32_t tt = id % T;
        t.m0 = (id / T) * kBM;
        uint32_t lo = 0, hi = P.n_expert;
        while (lo + 1 < hi) {
            const uint32_t mid = (lo + hi) >> 1;
            if ((uint32_t)P.tile_off[mid] <= tt) lo = mid; else hi = mid;
        }
        t.e = lo;
        t.tok0 = (uint32_t)P.expert_off[lo] + (tt - (uint32_t)P.tile_off[lo]) * BN;
        t.n_valid = min((uint32_t)BN, (uint32_t)P.expert_off[lo + 1] - t.tok0);
    } else {
        const uint32_t tiles_n = (P.n_tok + BN - 1) / BN;
        t.e = 0;
        t.m0 = (id / tiles_n) * kBM;
        t.tok0 = (id % tiles_n) * BN;
        t.n_valid = min((uint32_t)BN, P.n_tok - t.tok0);
    }
    return t;
}

// Shared-memory plan (offsets from a 1024-byte aligned base).
template <int FMT, int BN> struct Smem {
    static constexpr uint32_t raw_stage = kKS * MmqTraits<FMT>::raw_bytes;
    static constexpr uint32_t a_sub = kBM * 32, b_sub = BN * 32, sx_sub = BN * 4;
    static constexpr uint32_t rsc_stage = (kKS + 1) * kBM * 4; // row scale words + superblock word
    static constexpr uint32_t raw_off = 0;
    static constexpr uint32_t a_off = raw_off + kStages * raw_stage;
    static constexpr uint32_t b_off = a_off + kStages * kKS * a_sub;
    static constexpr uint32_t dx_off = b_off + kStages * kKS * b_sub;
    static constexpr uint32_t xs_off = dx_off + kStages * kKS * sx_sub;
    static constexpr uint32_t rsc_off = xs_off + kStages * kKS * sx_sub;
    static constexpr uint32_t bar_off = rsc_off + kStages * rsc_stage;
    // barriers: raw_full, raw_empty, op_full, op_empty [kStages each]; tm_full, tm_empty [kBufs each]
    static constexpr uint32_t n_bars = 4 * kStages + 2 * kBufs;
    static constexpr uint32_t misc_off = bar_off + n_bars * 8; // tmem base slot, abort flag
    static constexpr uint32_t total = misc_off + 16 + 1024;    // + alignment slack
};

// Packed pairs of f32 (one instruction, two lanes' worth of results): halves the issue slots of the drain.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi)
{
    return (unsigned long long)__float_as_uint(lo) | ((unsigned long long)__float_as_uint(hi) << 32);
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b)
{
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b)
{
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c)
{
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// EPW epilogue warps (16 for the dense tile: four per scheduler, 32 columns each; 8 for the expert
// tile).  With P.planar the activations come from rc_matmul's planar scratch: the int8 quants land
// by TMA directly in the operand layout and the token scales beside them, so the expanders only
// split nibbles.
template <int FMT, int BN, int EPW, int EXW>
__global__ void __launch_bounds__((2 + EXW + EPW) * 32, 1)
mmq_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_b,
           const __grid_constant__ CUtensorMap tmap_dx, const __grid_constant__ CUtensorMap tmap_xs, const MmqParams P)
{
    using L = Smem<FMT, BN>;
    constexpr int kExpT = EXW * 32; // expander threads (the narrow expert tile is bound by them: four warps)
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bars = sbase + L::bar_off;
    auto raw_full = [&](uint32_t s) { return bars + s * 8u; };
    auto raw_empty = [&](uint32_t s) { return bars + (kStages + s) * 8u; };
    auto op_full = [&](uint32_t s) { return bars + (2 * kStages + s) * 8u; };
    auto op_empty = [&](uint32_t s) { return bars + (3 * kStages + s) * 8u; };
    auto tm_full = [&](uint32_t b) { return bars + (4 * kStages + b) * 8u; };
    auto tm_empty = [&](uint32_t b) { return bars + (4 * kStages + kBufs + b) * 8u; };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::misc_off);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n_sub = P.in_dim >> 5;
    const uint32_t n_iters = (n_sub + kKS - 1) / kKS;
    const uint32_t tiles_m = (P.out_dim + kBM - 1) / kBM;
    const uint32_t n_tiles = tile_count<BN>(P, tiles_m);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; s++) {
            mbar_init(raw_full(s), 1);
            mbar_init(raw_empty(s), kExpT);
            mbar_init(op_full(s), kExpT);
            mbar_init(op_empty(s), EPW); // an epilogue warp arrives after the tm_full of the stage's last MMA
        }
        for (uint32_t b = 0; b < kBufs; b++) {
            mbar_init(tm_full(b), 1);
            mbar_init(tm_empty(b), EPW);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kBufs * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer ---------------------------------------------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
                const Tile t = decode_tile<BN>(P, id);
                for (uint32_t i = 0; i < n_iters; i++, it++) {
                    const uint32_t s = it % kStages;
                    if (it >= kStages) {
                        if (!mbar_wait(raw_empty(s), ((it / kStages) - 1u) & 1u, abort_flag, 1u)) goto tma_done;
                        // planar: this thread also overwrites the operand and scale areas of the slot
                        if (P.planar && !mbar_wait(op_empty(s), ((it / kStages) - 1u) & 1u, abort_flag, 8u)) goto tma_done;
                    }
                    const uint32_t nsteps = min((uint32_t)kKS, n_sub - i * kKS);
                    const uint32_t planar_bytes = P.planar ? kKS * (L::b_sub + 2u * L::sx_sub) : 0u; // whole boxes, zero-filled outside
                    mbar_expect_tx(raw_full(s), nsteps * MmqTraits<FMT>::raw_bytes + planar_bytes);
                    for (uint32_t j = 0; j < nsteps; j++)
                        for (int pl = 0; pl < MmqTraits<FMT>::raw_planes; pl++)
                            tma_load_4d(sbase + L::raw_off + s * L::raw_stage + j * MmqTraits<FMT>::raw_bytes + pl * kBM * 16,
                                        &tmap, raw_full(s), (int)((i * kKS + j) * 16u), (int)t.m0, pl, (int)t.e);
                    if (P.planar) {
                        // (16 bytes, token, 16-byte chunk of K): lands as [chunk][token][16 B] = kKS operands [half][token][16 B]
                        tma_load_3d(sbase + L::b_off + s * kKS * L::b_sub, &tmap_b, raw_full(s), 0, (int)t.tok0, (int)(i * kKS * 2u));
                        tma_load_2d(sbase + L::dx_off + s * kKS * L::sx_sub, &tmap_dx, raw_full(s), (int)t.tok0, (int)(i * kKS));
                        tma_load_2d(sbase + L::xs_off + s * kKS * L::sx_sub, &tmap_xs, raw_full(s), (int)t.tok0, (int)(i * kKS));
                    }
                }
            }
        tma_done:;
        }
    } else if (warp == 1) {
        // ---- MMA issuer -------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_i8(BN);
            uint32_t it = 0, kc = 0;
            for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
                for (uint32_t i = 0; i < n_iters; i++, it++) {
                    const uint32_t s = it % kStages;
                    if (!mbar_wait(op_full(s), (it / kStages) & 1u, abort_flag, 2u)) goto mma_done;
                    tc_fence_after();
                    const uint32_t nsteps = min((uint32_t)kKS, n_sub - i * kKS);
                    for (uint32_t j = 0; j < nsteps; j++, kc++) {
                        const uint32_t b = kc % kBufs;
                        if (kc >= kBufs && !mbar_wait(tm_empty(b), ((kc / kBufs) - 1u) & 1u, abort_flag, 3u)) goto mma_done;
                        tc_fence_after();
                        const uint64_t da = make_desc(sbase + L::a_off + (s * kKS + j) * L::a_sub, kBM * 16, 128);
                        const uint64_t db = make_desc(sbase + L::b_off + (s * kKS + j) * L::b_sub, BN * 16, 128);
                        mma_i8(tmem_base + b * BN, da, db, idesc, 0u);
                        mma_commit(tm_full(b));
                    }
                }
            }
        mma_done:;
        }
    } else if (warp < 2 + EXW) {
        // ---- expanders ------------------------------------------------------------------------------
        const uint32_t tid = threadIdx.x - 64u;
        constexpr int ROWS_PT = kBM / kExpT;                                // weight rows per thread
        constexpr int ITEMS_PT = (BN * kKS + kExpT - 1) / kExpT; // (token, sub-block) items per thread
        uint32_t it = 0;
        for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
            const Tile t = decode_tile<BN>(P, id);
            const Planes pl = planes_of<FMT>(P.w + (size_t)t.e * P.bytes_per_expert, P.in_dim, P.out_dim);
            const bool sup_a4 = (reinterpret_cast<uintptr_t>(pl.sup) & 3u) == 0;
            for (uint32_t i = 0; i < n_iters; i++, it++) {
                const uint32_t s = it % kStages;
                const uint32_t k0 = i * kKS, nsteps = min((uint32_t)kKS, n_sub - k0);
                // global loads first: side planes, row scales, and the first group of BlockQ8 items
                constexpr int GROUP = ITEMS_PT < 4 ? ITEMS_PT : 4;
                uint2 xb[GROUP][5];
                auto load_items = [&](int n0) {
#pragma unroll
                    for (int n = 0; n < GROUP; n++) {
                        const uint32_t q = tid + (n0 + n) * kExpT, tok = q % BN, j = q / BN;
                        if (j < nsteps && tok < t.n_valid) {
                            const uint2 *src = reinterpret_cast<const uint2 *>(
                                P.xq + ((size_t)(t.tok0 + tok) * n_sub + k0 + j) * RC_BLOCKQ8_BYTES);
#pragma unroll
                            for (int w = 0; w < 5; w++) xb[n][w] = __ldg(src + w);
                        } else {
#pragma unroll
                            for (int w = 0; w < 5; w++) xb[n][w] = make_uint2(0u, 0u);
                        }
                    }
                };
                if (!P.planar) load_items(0);
                uint32_t extra[ROWS_PT][kKS];
                StageScales sc[ROWS_PT];
#pragma unroll
                for (int rr = 0; rr < ROWS_PT; rr++) {
                    const uint32_t row = min(t.m0 + tid + rr * kExpT, P.out_dim - 1u);
                    sc[rr].dd = 0;
#pragma unroll
                    for (int j = 0; j < kKS; j++) {
                        sc[rr].s[j] = 0;
                        extra[rr][j] = 0;
                        if constexpr (FMT == Q5_K)
                            if (j < (int)nsteps) extra[rr][j] = ld_stream_u32(pl.aux + ((size_t)row * pl.nsp + k0 + j) * 4);
                    }
                    load_scales<FMT>(sc[rr], pl, sup_a4, row, k0, nsteps);
                }
                if (it >= kStages && !mbar_wait(op_empty(s), ((it / kStages) - 1u) & 1u, abort_flag, 4u)) goto exp_done;
                if (!mbar_wait(raw_full(s), (it / kStages) & 1u, abort_flag, 5u)) goto exp_done;
                // A: whole weight rows of the tile, and their scale words for the epilogue
#pragma unroll
                for (int rr = 0; rr < ROWS_PT; rr++) {
                    const uint32_t r = tid + rr * kExpT;
                    const uint32_t rs = sbase + L::rsc_off + s * L::rsc_stage + r * 4u;
#pragma unroll
                    for (int j = 0; j < kKS; j++) sts_u32(rs + j * kBM * 4u, sc[rr].s[j]);
                    sts_u32(rs + kKS * kBM * 4u, sc[rr].dd);
#pragma unroll
                    for (int j = 0; j < kKS; j++) {
                        if (j < (int)nsteps) {
                            const uint32_t rp = sbase + L::raw_off + s * L::raw_stage + j * MmqTraits<FMT>::raw_bytes + r * 16u;
                            const uint4 q = lds_u4(rp);
                            uint4 q2 = make_uint4(0, 0, 0, 0);
                            if constexpr (FMT == Q8_0) q2 = lds_u4(rp + kBM * 16);
                            uint4 lo, hi;
                            expand_weights<FMT>(q, q2, extra[rr][j], lo, hi);
                            const uint32_t ap = sbase + L::a_off + (s * kKS + j) * L::a_sub + r * 16u;
                            sts_u4(ap, lo);
                            sts_u4(ap + kBM * 16, hi);
                        }
                    }
                }
                // B from BlockQ8 records (rc_mmq_gemm, grouped GEMM): the int8 quants in the same layout, the
                // token scales beside them; a few items at a time to bound the registers in flight
                if (!P.planar) {
#pragma unroll
                    for (int n0 = 0; n0 < ITEMS_PT; n0 += GROUP) {
                        if (n0 > 0) load_items(n0);
#pragma unroll
                        for (int n = 0; n < GROUP; n++) {
                            const uint32_t q = tid + (n0 + n) * kExpT, tok = q % BN, j = q / BN;
                            if (j < nsteps) {
                                const uint32_t bp = sbase + L::b_off + (s * kKS + j) * L::b_sub + tok * 16u;
                                sts_u4(bp, make_uint4(xb[n][1].x, xb[n][1].y, xb[n][2].x, xb[n][2].y));
                                sts_u4(bp + BN * 16, make_uint4(xb[n][3].x, xb[n][3].y, xb[n][4].x, xb[n][4].y));
                                sts_u32(sbase + L::dx_off + (s * kKS + j) * L::sx_sub + tok * 4u, xb[n][0].x);
                                sts_u32(sbase + L::xs_off + (s * kKS + j) * L::sx_sub + tok * 4u, xb[n][0].y);
                            }
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic writes -> MMA reads
                mbar_arrive(op_full(s));
                mbar_arrive(raw_empty(s));
            }
        }
    exp_done:;
    } else {
        // ---- epilogue -----------------------------------------------------------------------------------
        const uint32_t quarter = warp & 3u;        // tensor-memory lanes this warp may read
        const uint32_t half = (warp - (2u + EXW)) >> 2; // which group of COLS columns
        constexpr int COLS = BN / (EPW / 4);       // columns per thread
        constexpr int CHUNKS = COLS / 32 > 0 ? COLS / 32 : 1;
        constexpr int CW = COLS < 32 ? COLS : 32;  // columns per tensor-memory load
        static_assert(COLS == 16 || COLS % 32 == 0, "16 or a multiple of 32 columns per epilogue warp");
        unsigned long long acc[COLS / 2]; // pairs of adjacent tokens
        uint32_t it = 0, kc = 0;
        for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
            const Tile t = decode_tile<BN>(P, id);
            const uint32_t row_raw = t.m0 + quarter * 32u + lane;
#pragma unroll
            for (int c = 0; c < COLS / 2; c++) acc[c] = 0ull;
            for (uint32_t i = 0; i < n_iters; i++, it++) {
                const uint32_t s = it % kStages;
                const uint32_t nsteps = min((uint32_t)kKS, n_sub - i * kKS);
                // the stage's token scales and this row's scale words were staged before op_full completed
                if (!mbar_wait(op_full(s), (it / kStages) & 1u, abort_flag, 6u)) goto epi_done;
                const uint32_t rs = sbase + L::rsc_off + s * L::rsc_stage + (quarter * 32u + lane) * 4u;
                float d_sup = 0.0f, dmin_sup = 0.0f;
                if constexpr (MmqTraits<FMT>::has_min) {
                    const uint32_t dd = lds_u32(rs + kKS * kBM * 4u);
                    d_sup = f16_bits_to_f32(dd);
                    dmin_sup = f16_bits_to_f32(dd >> 16);
                }
                // drain of one sub-block's columns (already in registers) into the accumulators
                auto drain = [&](const uint32_t (&d)[32], int j, int ch) {
                    const uint32_t sw = lds_u32(rs + j * kBM * 4u);
                    float dsc, ndeff = 0.0f;
                    if constexpr (MmqTraits<FMT>::has_min) {
                        dsc = d_sup * (float)(sw & 0xFFu);
                        ndeff = -dmin_sup * (float)(sw >> 8);
                    } else {
                        dsc = f16_bits_to_f32(sw);
                    }
                    const unsigned long long dsc2 = pack2(dsc, dsc), ndeff2 = pack2(ndeff, ndeff);
                    const uint32_t dxp = sbase + L::dx_off + (s * kKS + j) * L::sx_sub + half * COLS * 4u;
                    const uint32_t xsp = sbase + L::xs_off + (s * kKS + j) * L::sx_sub + half * COLS * 4u;
#pragma unroll
                    for (int c = 0; c < CW; c += 4) {
                        const ulonglong2 dx4 = lds_u64x2(dxp + (ch * 32 + c) * 4u);
                        // int -> float is exact here (|idot| < 2^24) and a full-rate conversion on this part
                        const unsigned long long f01 = pack2((float)(int)d[c], (float)(int)d[c + 1]);
                        const unsigned long long f23 = pack2((float)(int)d[c + 2], (float)(int)d[c + 3]);
                        unsigned long long a01 = acc[(ch * 32 + c) / 2], a23 = acc[(ch * 32 + c) / 2 + 1];
                        a01 = fma2(dsc2, mul2(f01, dx4.x), a01);
                        a23 = fma2(dsc2, mul2(f23, dx4.y), a23);
                        if constexpr (MmqTraits<FMT>::has_min) {
                            const ulonglong2 xs4 = lds_u64x2(xsp + (ch * 32 + c) * 4u);
                            a01 = fma2(ndeff2, xs4.x, a01);
                            a23 = fma2(ndeff2, xs4.y, a23);
                        }
                        acc[(ch * 32 + c) / 2] = a01;
                        acc[(ch * 32 + c) / 2 + 1] = a23;
                    }
                };
#pragma unroll
                for (int j = 0; j < kKS; j++) {
                    if (j < (int)nsteps) {
                        const uint32_t b = kc % kBufs;
                        if (!mbar_wait(tm_full(b), (kc / kBufs) & 1u, abort_flag, 7u)) goto epi_done;
                        tc_fence_after();
#pragma unroll
                        for (int ch = 0; ch < CHUNKS; ch++) {
                            uint32_t d[32];
                            if constexpr (CW == 32)
                                tmem_ld32(tmem_base + ((quarter * 32u) << 16) + b * BN + half * COLS + ch * 32, d);
                            else
                                tmem_ld16(tmem_base + ((quarter * 32u) << 16) + b * BN + half * COLS, d);
                            tmem_wait_ld();
                            if (ch == CHUNKS - 1) {
                                // every column of this warp's share is in registers: release the buffer
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(tm_empty(b));
                            }
                            drain(d, j, ch);
                        }
                        kc++;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(op_empty(s)); // done with the stage's operands (its MMAs have completed) and scales
            }
            // tile end: Y[tok][row], a warp writes 32 consecutive rows of one token per store
            if (row_raw < P.out_dim) {
#pragma unroll
                for (int c = 0; c < COLS; c++) {
                    const uint32_t col = half * COLS + c;
                    const float v = __uint_as_float((uint32_t)(acc[c / 2] >> (32 * (c & 1))));
                    if (col < t.n_valid) P.y[(size_t)(t.tok0 + col) * P.out_dim + row_raw] = v;
                }
            }
        }
    epi_done:;
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, kBufs * BN);
    }
}

// =====================================================================================================
// The same GEMM with the operands held as f16 (tcgen05 kind::f16, f32 accumulator).
//
// Every operand value is a small integer that f16 represents exactly (|v| <= 2048), every product
// and every 32-term sum stays below 2^24, so the f32 accumulator in tensor memory holds the exact
// integer the int8 MMA would produce — already as a float, which removes the int->float step of the
// drain.  And because the operand is no longer limited to 8 bits, the integer sub-block scale of the
// K-quants rides inside it: A = sc * q (at most 63 * 31 = 1953), so the drain multiplies by the
// per-superblock f16 d instead of a per-sub-block product.  Q6_K, whose (q - 32) * sc reaches 4096,
// is split exactly as (q - 32) * 2*(sc >> 1) + (q - 32) * (sc & 1): two operands accumulated into the
// same tile, which also gives each 16-weight half its own scale (one K=16 MMA per half).
// Per (row, token, sub-block) the drain is then  acc += d * (dx * D)  [- (dmin * m) * xsum].
//
// Layout: a 128 x 32-element f16 operand is [kc 0..3][row][16 B] (core matrices of 8 rows x 8
// halves); one K=16 MMA reads two adjacent kc blocks.  Roles: warp 0 TMA, warp 1 MMA issue, warps
// 2..5 expanders, warps 6.. epilogue (16 warps of 32 columns for the dense tile: four per scheduler,
// so that one warp's tensor-memory load and barrier latency hides behind the others' math).

constexpr int kKS16 = 2;      // sub-blocks per stage

__device__ unsigned int g_mmq16_error;

__device__ __forceinline__ bool mbar_wait16(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, uint32_t code)
{
    if (mbar_try(bar, parity)) return true;
    // the limit is kept on the SM's own cycle counter, first read after 64 failed polls: a wait
    // that is about to succeed never pays for a timer read
    long long t0 = 0;
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitCycles) break;
        }
    }
    atomicExch(&g_mmq16_error, code);
    *abort_flag = 1u;
    return false;
}

template <int FMT> struct Mmq16Traits {
    static constexpr bool has_min = (FMT == Q4_K || FMT == Q5_K);
    static constexpr bool fold = (FMT == Q4_K || FMT == Q5_K || FMT == Q6_K); // integer scale inside A
    static constexpr int a_parts = (FMT == Q6_K) ? 2 : 1;                     // operands accumulated per sub-block
    static constexpr int raw_planes = (FMT == Q8_0) ? 2 : 1;
    static constexpr uint32_t raw_bytes = raw_planes * kBM * 16;
    static constexpr int stages = (FMT == Q6_K) ? 3 : 4; // Q6_K carries two A operands per sub-block
};

template <int FMT, int BN> struct Smem16 {
    static constexpr uint32_t stages = Mmq16Traits<FMT>::stages;
    static constexpr uint32_t raw_stage = kKS16 * Mmq16Traits<FMT>::raw_bytes;
    static constexpr uint32_t a_part = kBM * 64;                                  // one operand of one sub-block
    static constexpr uint32_t a_sub = a_part * Mmq16Traits<FMT>::a_parts;
    static constexpr uint32_t b_sub = BN * 64, sx_sub = BN * 4;
    static constexpr uint32_t braw_stage = BN * kKS16 * RC_BLOCKQ8_BYTES;         // [token][kKS16 blocks of 40 B]
    static constexpr uint32_t rsc_stage = (kKS16 + 1) * kBM * 4;                  // row scale words + superblock word
    static constexpr uint32_t raw_off = 0;
    static constexpr uint32_t braw_off = raw_off + stages * raw_stage;
    static constexpr uint32_t a_off = braw_off + stages * braw_stage;
    static constexpr uint32_t b_off = a_off + stages * kKS16 * a_sub;
    static constexpr uint32_t dx_off = b_off + stages * kKS16 * b_sub;
    static constexpr uint32_t xs_off = dx_off + stages * kKS16 * sx_sub;
    static constexpr uint32_t rsc_off = xs_off + stages * kKS16 * sx_sub;
    static constexpr uint32_t bar_off = rsc_off + stages * rsc_stage;
    static constexpr uint32_t n_bars = 4 * stages + 2 * kBufs;
    static constexpr uint32_t misc_off = bar_off + n_bars * 8;
    static constexpr uint32_t total = misc_off + 16 + 1024;
};

template <int FMT, int BN, int EPW, int EXW>
__global__ void __launch_bounds__((2 + EXW + EPW) * 32, 1)
mmq16_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_b, const MmqParams P)
{
    using L = Smem16<FMT, BN>;
    using T = Mmq16Traits<FMT>;
    constexpr uint32_t kStages16 = L::stages;
    constexpr int kExpanders16 = EXW * 32;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bars = sbase + L::bar_off;
    auto raw_full = [&](uint32_t s) { return bars + s * 8u; };
    auto raw_empty = [&](uint32_t s) { return bars + (kStages16 + s) * 8u; };
    auto op_full = [&](uint32_t s) { return bars + (2 * kStages16 + s) * 8u; };
    auto op_empty = [&](uint32_t s) { return bars + (3 * kStages16 + s) * 8u; };
    auto tm_full = [&](uint32_t b) { return bars + (4 * kStages16 + b) * 8u; };
    auto tm_empty = [&](uint32_t b) { return bars + (4 * kStages16 + kBufs + b) * 8u; };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::misc_off);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n_sub = P.in_dim >> 5;
    const uint32_t n_iters = (n_sub + kKS16 - 1) / kKS16;
    const uint32_t tiles_m = (P.out_dim + kBM - 1) / kBM;
    const uint32_t n_tiles = tile_count<BN>(P, tiles_m);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages16; s++) {
            mbar_init(raw_full(s), 1);
            mbar_init(raw_empty(s), kExpanders16);
            mbar_init(op_full(s), kExpanders16);
            mbar_init(op_empty(s), EPW); // an epilogue warp arrives after the tm_full of the stage's last MMA
        }
        for (uint32_t b = 0; b < kBufs; b++) {
            mbar_init(tm_full(b), 1);
            mbar_init(tm_empty(b), EPW);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kBufs * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 2) {
      if (warp == 0) {
        // ---- TMA producer: raw 16-byte planes, one box per (sub-block, plane) -----------------
        if (lane == 0) {
            uint32_t it = 0;
            for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
                const Tile t = decode_tile<BN>(P, id);
                for (uint32_t i = 0; i < n_iters; i++, it++) {
                    const uint32_t s = it % kStages16;
                    if (it >= kStages16 && !mbar_wait16(raw_empty(s), ((it / kStages16) - 1u) & 1u, abort_flag, 1u)) break;
                    const uint32_t nsteps = min((uint32_t)kKS16, n_sub - i * kKS16);
                    if (P.debug & 8u) continue;
                    mbar_expect_tx(raw_full(s), nsteps * T::raw_bytes + (P.b_tma ? L::braw_stage : 0u));
                    if (P.b_tma) // BN activation rows x the stage's blocks (a partly outside box is zero-filled)
                        tma_load_2d(sbase + L::braw_off + s * L::braw_stage, &tmap_b, raw_full(s),
                                    (int)(i * kKS16 * RC_BLOCKQ8_BYTES), (int)t.tok0);
                    for (uint32_t j = 0; j < nsteps; j++)
                        for (int pl = 0; pl < T::raw_planes; pl++)
                            tma_load_4d(sbase + L::raw_off + s * L::raw_stage + j * T::raw_bytes + pl * kBM * 16, &tmap,
                                        raw_full(s), (int)((i * kKS16 + j) * 16u), (int)t.m0, pl, (int)t.e);
                }
            }
        }
      } else if (warp == 1) {
        // ---- MMA issuer: two K=16 MMAs per operand part per sub-block ----------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(BN);
            uint32_t it = 0, kc = 0;
            for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
                for (uint32_t i = 0; i < n_iters; i++, it++) {
                    const uint32_t s = it % kStages16;
                    if (!mbar_wait16(op_full(s), (it / kStages16) & 1u, abort_flag, 2u)) goto mma_done;
                    tc_fence_after();
                    const uint32_t nsteps = min((uint32_t)kKS16, n_sub - i * kKS16);
                    for (uint32_t j = 0; j < nsteps; j++, kc++) {
                        const uint32_t b = kc % kBufs;
                        if (kc >= kBufs && !mbar_wait16(tm_empty(b), ((kc / kBufs) - 1u) & 1u, abort_flag, 3u)) goto mma_done;
                        tc_fence_after();
                        const uint32_t a0 = sbase + L::a_off + (s * kKS16 + j) * L::a_sub;
                        const uint32_t b0 = sbase + L::b_off + (s * kKS16 + j) * L::b_sub;
#pragma unroll
                        for (int part = 0; part < T::a_parts; part++) {
#pragma unroll
                            for (int kh = 0; kh < 2; kh++) {
                                const uint64_t da = make_desc(a0 + part * L::a_part + kh * 2 * kBM * 16, kBM * 16, 128);
                                const uint64_t db = make_desc(b0 + kh * 2 * BN * 16, BN * 16, 128);
                                if (!(P.debug & 128u)) mma_f16(tmem_base + b * BN, da, db, idesc, (part | kh) ? 1u : 0u);
                            }
                        }
                        mma_commit(tm_full(b));
                    }
                }
            }
        mma_done:;
        }
      }
    } else if (warp < 2 + EXW) {
        // ---- expanders -----------------------------------------------------------------------------
        const uint32_t tid = threadIdx.x - 64u;
        constexpr int ROWS_PT = kBM / kExpanders16; // weight rows per thread
        constexpr int ITEMS_PT = (BN * kKS16 + kExpanders16 - 1) / kExpanders16; // (token, sub-block) items per thread
        uint32_t it = 0;
        for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
            const Tile t = decode_tile<BN>(P, id);
            const Planes pl = planes_of<FMT>(P.w + (size_t)t.e * P.bytes_per_expert, P.in_dim, P.out_dim);
            for (uint32_t i = 0; i < n_iters; i++, it++) {
                const uint32_t s = it % kStages16;
                const uint32_t k0 = i * kKS16, nsteps = min((uint32_t)kKS16, n_sub - k0);
                // global loads first: activations of this stage and the format's side planes
                uint2 xb[ITEMS_PT][5];
#pragma unroll
                for (int n = 0; n < ITEMS_PT; n++) {
                    const uint32_t q = tid + n * kExpanders16, tok = q % BN, j = q / BN;
                    if (j < nsteps && tok < t.n_valid && !(P.debug & 1u) && !P.b_tma) {
                        const uint2 *src = reinterpret_cast<const uint2 *>(
                            P.xq + ((size_t)(t.tok0 + tok) * n_sub + k0 + j) * RC_BLOCKQ8_BYTES);
#pragma unroll
                        for (int w = 0; w < 5; w++) xb[n][w] = __ldg(src + w);
                    } else {
#pragma unroll
                        for (int w = 0; w < 5; w++) xb[n][w] = make_uint2(0u, 0u);
                    }
                }
                uint32_t e0[ROWS_PT][kKS16], e1[ROWS_PT][kKS16], smw[ROWS_PT][kKS16], ddw[ROWS_PT];
#pragma unroll
                for (int rr = 0; rr < ROWS_PT; rr++) {
                    const uint32_t row = min(t.m0 + tid + rr * kExpanders16, P.out_dim - 1u);
                    ddw[rr] = 0;
#pragma unroll
                    for (int j = 0; j < kKS16; j++) {
                        e0[rr][j] = e1[rr][j] = smw[rr][j] = 0;
                        if (j < (int)nsteps && !(P.debug & 32u)) {
                            const size_t idx = (size_t)row * pl.nsp + k0 + j;
                            if constexpr (FMT == Q5_K) e0[rr][j] = ld_stream_u32(pl.aux + idx * 4);
                            if constexpr (FMT == Q6_K) {
                                const uint2 h = ld_stream_u2(pl.aux + idx * 8);
                                e0[rr][j] = h.x;
                                e1[rr][j] = h.y;
                            }
                            smw[rr][j] = ld_nc_u16(pl.sc + idx * 2);
                        }
                    }
                    // the superblock word of the stage (a stage never straddles two superblocks)
                    if constexpr (T::has_min) {
                        const uint8_t *sp = pl.sup + ((size_t)row * pl.n_super + (k0 >> 3)) * 4;
                        ddw[rr] = ((reinterpret_cast<uintptr_t>(pl.sup) & 3u) == 0)
                                      ? __ldg(reinterpret_cast<const uint32_t *>(sp))
                                      : (ld_nc_u16(sp) | (ld_nc_u16(sp + 2) << 16));
                    } else if constexpr (FMT == Q6_K) {
                        ddw[rr] = ld_nc_u16(pl.sup + ((size_t)row * pl.n_super + (k0 >> 3)) * 2);
                    }
                }
                if (it >= kStages16 && !mbar_wait16(op_empty(s), ((it / kStages16) - 1u) & 1u, abort_flag, 4u)) goto exp_done;
                if (!(P.debug & 8u) && !mbar_wait16(raw_full(s), (it / kStages16) & 1u, abort_flag, 5u)) goto exp_done;
                // A: this thread's weight rows, and their scale words for the epilogue
#pragma unroll
                for (int rr = 0; rr < ROWS_PT; rr++) {
                    const uint32_t r = tid + rr * kExpanders16;
                    const uint32_t rs = sbase + L::rsc_off + s * L::rsc_stage + r * 4u;
#pragma unroll
                    for (int j = 0; j < kKS16; j++) sts_u32(rs + j * kBM * 4u, smw[rr][j]);
                    sts_u32(rs + kKS16 * kBM * 4u, ddw[rr]);
#pragma unroll
                    for (int j = 0; j < kKS16; j++) {
                        if (j < (int)nsteps && !(P.debug & 2u)) {
                            const uint32_t rp = sbase + L::raw_off + s * L::raw_stage + j * T::raw_bytes + r * 16u;
                            const uint4 q = lds_u4(rp);
                            uint4 q2 = make_uint4(0, 0, 0, 0);
                            if constexpr (FMT == Q8_0) q2 = lds_u4(rp + kBM * 16);
                            uint4 o[2][4];
                            expand_f16<FMT>(q, q2, e0[rr][j], e1[rr][j], smw[rr][j], o);
#pragma unroll
                            for (int part = 0; part < T::a_parts; part++) {
                                const uint32_t ap = sbase + L::a_off + (s * kKS16 + j) * L::a_sub + part * L::a_part + r * 16u;
#pragma unroll
                                for (int c = 0; c < 4; c++) sts_u4(ap + c * kBM * 16, o[part][c]);
                            }
                        }
                    }
                }
                // B: int8 quants -> f16 in the same layout; scales beside them
#pragma unroll
                for (int n = 0; n < ITEMS_PT; n++) {
                    const uint32_t q = tid + n * kExpanders16, tok = q % BN, j = q / BN;
                    if (j < nsteps && !(P.debug & 16u)) {
                        const __half2 one = __half2half2(__float2half(1.0f)), off = __half2half2(__float2half(-1152.0f));
                        if (P.b_tma) {
                            const uint32_t src = sbase + L::braw_off + s * L::braw_stage + (tok * kKS16 + j) * RC_BLOCKQ8_BYTES;
                            const bool ok = tok < t.n_valid; // rows past the tile's tokens belong to someone else
#pragma unroll
                            for (int w = 0; w < 5; w++) xb[n][w] = ok ? lds_u2(src + w * 8u) : make_uint2(0u, 0u);
                        }
                        const uint32_t bp = sbase + L::b_off + (s * kKS16 + j) * L::b_sub + tok * 16u;
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            const uint2 w2 = xb[n][1 + c]; // qs[8c .. 8c+7]
                            sts_u4(bp + c * BN * 16, kc_block(w2.x ^ 0x80808080u, w2.y ^ 0x80808080u, one, off));
                        }
                        sts_u32(sbase + L::dx_off + (s * kKS16 + j) * L::sx_sub + tok * 4u, xb[n][0].x);
                        sts_u32(sbase + L::xs_off + (s * kKS16 + j) * L::sx_sub + tok * 4u, xb[n][0].y);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(op_full(s));
                mbar_arrive(raw_empty(s));
            }
        }
    exp_done:;
    } else {
        // ---- epilogue -------------------------------------------------------------------------------------
        const uint32_t quarter = warp & 3u;        // tensor-memory lanes this warp may read
        const uint32_t half = (warp - (2u + EXW)) >> 2;    // which group of COLS columns
        constexpr int COLS = BN / (EPW / 4);
        constexpr int CHUNKS = COLS / 32 > 0 ? COLS / 32 : 1;
        constexpr int CW = COLS < 32 ? COLS : 32;
        static_assert(COLS == 16 || COLS % 32 == 0, "16 or a multiple of 32 columns per epilogue warp");
        float acc[COLS];
        uint32_t it = 0, kc = 0;
        for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
            const Tile t = decode_tile<BN>(P, id);
            const Planes pl = planes_of<FMT>(P.w + (size_t)t.e * P.bytes_per_expert, P.in_dim, P.out_dim);
            const uint32_t row_raw = t.m0 + quarter * 32u + lane;
#pragma unroll
            for (int c = 0; c < COLS; c++) acc[c] = 0.0f;
            for (uint32_t i = 0; i < n_iters; i++, it++) {
                const uint32_t s = it % kStages16;
                const uint32_t k0 = i * kKS16, nsteps = min((uint32_t)kKS16, n_sub - k0);
                if (!mbar_wait16(op_full(s), (it / kStages16) & 1u, abort_flag, 6u)) goto epi_done;
                // this row's scale words, staged by the expanders before op_full completed
                const uint32_t rs = sbase + L::rsc_off + s * L::rsc_stage + (quarter * 32u + lane) * 4u;
                const uint32_t dd_cur = lds_u32(rs + kKS16 * kBM * 4u);
                uint32_t s_cur[kKS16];
#pragma unroll
                for (int j = 0; j < kKS16; j++) s_cur[j] = lds_u32(rs + j * kBM * 4u);
                const float d_sup = T::fold ? f16_bits_to_f32(dd_cur) : 0.0f;
                const float dmin_sup = T::has_min ? f16_bits_to_f32(dd_cur >> 16) : 0.0f;
#pragma unroll
                for (int j = 0; j < kKS16; j++) {
                    if (j < (int)nsteps) {
                        const uint32_t b = kc % kBufs;
                        if (!mbar_wait16(tm_full(b), (kc / kBufs) & 1u, abort_flag, 7u)) goto epi_done;
                        tc_fence_after();
                        const float dsc = T::fold ? d_sup : f16_bits_to_f32(s_cur[j]);
                        const float ndeff = T::has_min ? -dmin_sup * (float)(s_cur[j] >> 8) : 0.0f;
                        const uint32_t dxp = sbase + L::dx_off + (s * kKS16 + j) * L::sx_sub + half * COLS * 4u;
                        const uint32_t xsp = sbase + L::xs_off + (s * kKS16 + j) * L::sx_sub + half * COLS * 4u;
#pragma unroll
                        for (int ch = 0; ch < CHUNKS; ch++) {
                            uint32_t d[32];
                            if (!(P.debug & 256u)) {
                            if constexpr (CW == 32)
                                tmem_ld32(tmem_base + ((quarter * 32u) << 16) + b * BN + half * COLS + ch * 32, d);
                            else
                                tmem_ld16(tmem_base + ((quarter * 32u) << 16) + b * BN + half * COLS, d);
                            tmem_wait_ld();
                            }
                            if (ch == CHUNKS - 1) {
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(tm_empty(b));
                            }
                            if (P.debug & 4u) continue;
#pragma unroll
                            for (int c = 0; c < CW; c += 4) {
                                const uint4 dx4 = lds_u4(dxp + (ch * 32 + c) * 4u);
                                uint4 xs4 = make_uint4(0u, 0u, 0u, 0u);
                                if constexpr (T::has_min) xs4 = lds_u4(xsp + (ch * 32 + c) * 4u);
                                const float dxv[4] = {__uint_as_float(dx4.x), __uint_as_float(dx4.y), __uint_as_float(dx4.z), __uint_as_float(dx4.w)};
                                const float xsv[4] = {__uint_as_float(xs4.x), __uint_as_float(xs4.y), __uint_as_float(xs4.z), __uint_as_float(xs4.w)};
#pragma unroll
                                for (int u = 0; u < 4; u++) {
                                    float a = acc[ch * 32 + c + u];
                                    a = fmaf(dsc, __uint_as_float(d[c + u]) * dxv[u], a);
                                    if constexpr (T::has_min) a = fmaf(ndeff, xsv[u], a);
                                    acc[ch * 32 + c + u] = a;
                                }
                            }
                        }
                        kc++;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(op_empty(s));
            }
            if (row_raw < P.out_dim) {
#pragma unroll
                for (int c = 0; c < COLS; c++) {
                    const uint32_t col = half * COLS + c;
                    if (col < t.n_valid) P.y[(size_t)(t.tok0 + col) * P.out_dim + row_raw] = acc[c];
                }
            }
        }
    epi_done:;
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, kBufs * BN);
    }
}

// ---- host ---------------------------------------------------------------------------------------------

template <int BN> struct Epw8 { static constexpr int v = BN >= 128 ? 16 : 8; };
template <int BN> struct Exw { static constexpr int v = BN >= 128 ? 2 : 4; }; // expander warps

template <int FMT, int BN>
int launch_tc(cudaStream_t s, const MmqParams &P, uint32_t tiles_upper_bound)
{
    CUtensorMap map;
    int rc = make_tmap<FMT>(&map, P.w, P.bytes_per_expert, P.expert_off ? P.n_expert : 1u, P.in_dim, P.out_dim);
    if (rc) return rc;
    CUtensorMap map_b = map, map_dx = map, map_xs = map;
    if (P.planar) {
        // views of rc_matmul's planar scratch (rc_quantize.cu): quants as (16 bytes, token, 16-byte chunk
        // of K), so that one box lands as kKS operands [half][token][16 B]; scales as (token, sub-block)
        EncodeTiledFn fn = encode_fn();
        if (!fn) return RC_ERR_NO_DEVICE;
        const uint32_t n_sub = P.in_dim >> 5;
        const uint64_t ld = ((uint64_t)P.n_tok + 3u) & ~3ull;
        uint8_t *base = const_cast<uint8_t *>(P.xq);
        const cuuint64_t bd[3] = {16, P.n_tok, P.in_dim / 16};
        const cuuint64_t bs[2] = {P.in_dim, 16};
        const cuuint32_t bb[3] = {16, (cuuint32_t)BN, 2 * kKS};
        const cuuint32_t one3[3] = {1, 1, 1};
        CUresult r = fn(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base, bd, bs, bb, one3, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        const cuuint64_t sd[2] = {P.n_tok, n_sub};
        const cuuint64_t ss[1] = {ld * 4};
        const cuuint32_t sb[2] = {(cuuint32_t)BN, kKS};
        const cuuint32_t one2[2] = {1, 1};
        uint8_t *dx = base + (size_t)P.n_tok * P.in_dim;
        if (r == CUDA_SUCCESS)
            r = fn(&map_dx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dx, sd, ss, sb, one2, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r == CUDA_SUCCESS)
            r = fn(&map_xs, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dx + (size_t)n_sub * ld * 4, sd, ss, sb, one2,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return RC_ERR_BAD_ARGUMENT;
    }
    const uint32_t grid = min(tiles_upper_bound, (uint32_t)sm_count());
    constexpr int EPW = Epw8<BN>::v, EXW = Exw<BN>::v;
    mmq_kernel<FMT, BN, EPW, EXW><<<grid, (2 + EXW + EPW) * 32, Smem<FMT, BN>::total, s>>>(map, map_b, map_dx, map_xs, P);
    return (int)cudaGetLastError();
}

// epilogue warps of the f16 kernel: 32 columns per warp for the dense tile, 16 for the expert tile
template <int BN> struct Epw16 { static constexpr int v = BN >= 128 ? 16 : 8; };

template <int FMT, int BN>
int launch_tc16(cudaStream_t s, const MmqParams &P, uint32_t tiles_upper_bound)
{
    CUtensorMap map;
    int rc = make_tmap<FMT>(&map, P.w, P.bytes_per_expert, P.expert_off ? P.n_expert : 1u, P.in_dim, P.out_dim);
    if (rc) return rc;
    const uint32_t grid = min(tiles_upper_bound, (uint32_t)sm_count());
    constexpr int EPW = Epw16<BN>::v;
    // The BlockQ8 rows go through TMA when their layout allows it: 16-byte aligned base and row
    // pitch (an even sub-block count); otherwise the expanders fetch them with plain loads.
    CUtensorMap map_b = map;
    MmqParams Q = P;
    const uint64_t pitch = (uint64_t)(P.in_dim >> 5) * RC_BLOCKQ8_BYTES;
    Q.b_tma = 0;
    if (((uintptr_t)P.xq & 15u) == 0 && pitch % 16 == 0 && !(P.debug & 64u)) {
        EncodeTiledFn fn = encode_fn();
        const cuuint64_t dims[2] = {pitch, P.n_tok};
        const cuuint64_t strides[1] = {pitch};
        const cuuint32_t box[2] = {kKS16 * RC_BLOCKQ8_BYTES, (cuuint32_t)BN};
        const cuuint32_t estr[2] = {1, 1};
        if (fn && fn(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(P.xq), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
            Q.b_tma = 1;
    }
    constexpr int EXW = Exw<BN>::v;
    mmq16_kernel<FMT, BN, EPW, EXW><<<grid, (2 + EXW + EPW) * 32, Smem16<FMT, BN>::total, s>>>(map, map_b, Q);
    return (int)cudaGetLastError();
}

template <int FMT, int BN> int set_attr16()
{
    return (int)cudaFuncSetAttribute(mmq16_kernel<FMT, BN, Epw16<BN>::v, Exw<BN>::v>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)Smem16<FMT, BN>::total);
}

template <int FMT, int BN> int set_attr()
{
    return (int)cudaFuncSetAttribute(mmq_kernel<FMT, BN, Epw8<BN>::v, Exw<BN>::v>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)Smem<FMT, BN>::total);
}

constexpr int kDenseBN = 128;
constexpr int kGroupedBN = 32;

bool g_force_dp4a = false;
int g_mmq_debug = 0;
bool g_no_planar = false;
int g_mmq_kind = 0; // 0: by format (int8 operands, f16 for Q6_K); 16 / 8: force one kernel (8 has no Q6_K)

} // namespace

uint32_t mmq_grouped_bn() { return kGroupedBN; }

int mmq_set_attributes()
{
    int rc = 0;
    rc |= set_attr<Q4_0, kDenseBN>();
    rc |= set_attr<Q8_0, kDenseBN>();
    rc |= set_attr<Q4_K, kDenseBN>();
    rc |= set_attr<Q5_K, kDenseBN>();
    rc |= set_attr<IQ4_XS, kDenseBN>();
    rc |= set_attr<IQ3_S, kDenseBN>();
    rc |= set_attr<Q4_0, kGroupedBN>();
    rc |= set_attr<Q8_0, kGroupedBN>();
    rc |= set_attr<Q4_K, kGroupedBN>();
    rc |= set_attr<Q5_K, kGroupedBN>();
    rc |= set_attr<IQ4_XS, kGroupedBN>();
    rc |= set_attr<IQ3_S, kGroupedBN>();
    rc |= set_attr16<Q4_0, kDenseBN>() | set_attr16<Q8_0, kDenseBN>() | set_attr16<Q4_K, kDenseBN>() |
          set_attr16<Q5_K, kDenseBN>() | set_attr16<Q6_K, kDenseBN>() | set_attr16<IQ4_XS, kDenseBN>() | set_attr16<IQ3_S, kDenseBN>();
    rc |= set_attr16<Q4_0, kGroupedBN>() | set_attr16<Q8_0, kGroupedBN>() | set_attr16<Q4_K, kGroupedBN>() |
          set_attr16<Q5_K, kGroupedBN>() | set_attr16<Q6_K, kGroupedBN>() | set_attr16<IQ4_XS, kGroupedBN>() | set_attr16<IQ3_S, kGroupedBN>();
    return rc;
}

void mmq_force_dp4a(int on) { g_force_dp4a = on != 0; }
void mmq_set_kind(int kind)
{
    g_mmq_kind = (kind & 0xFF) == 8 ? 8 : (kind & 0xFF) == 16 ? 16 : (kind & 0xFF) == 32 ? 32 : 0;
    mmq_x_set_prof(((kind & 0xFF) == 64 || (kind & 0xFF) == 66) ? 1 : 0); // kinds 64, 66: the default route with per-role cycle counters
    mmq_x_set_debug(((kind & 0xFF) == 65 || (kind & 0xFF) == 66) ? kind >> 8 : 0); // kinds 65, 66: the default route with the pipeline parts in kind >> 8 skipped
    mmq_deq_set_bn(g_mmq_kind == 32 ? kind >> 8 : 0); // kind 32: the upper bits force the token-tile width
    g_no_planar = ((kind >> 8) & 512) != 0; // bit 9 of the mask: keep rc_matmul on BlockQ8 records
    g_mmq_debug = kind >> 8; // upper bits: parts of the f16 kernel's pipeline to skip (timing experiments)
}

int mmq_device_error(unsigned int *out, bool clear)
{
    unsigned int a = 0, b = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&a, g_mmq_error, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&b, g_mmq16_error, sizeof(unsigned int));
    *out = (a & 0xFFu) | ((b & 0xFu) << 8);
    if (e == cudaSuccess && clear && (a | b)) {
        const unsigned int zero = 0;
        e = cudaMemcpyToSymbol(g_mmq_error, &zero, sizeof(unsigned int));
        if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_mmq16_error, &zero, sizeof(unsigned int));
    }
    return (int)e;
}

// Formats with one scale per 32-wide sub-block run on the tensor cores.  Q6_K scales each half
// of a sub-block separately (kernels/mmq_gemm_q6k_repacked.cpp), which a K=32 int8 MMA cannot
// keep apart; it goes through the dp4a kernel in slabs of 16 activation rows.
namespace {
int mmq_dense(cudaStream_t s, int type, const void *w, const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
              uint32_t p_rows, bool planar);
}

int launch_mmq_gemm(cudaStream_t s, int type, const void *w, const void *xq, float *y,
                    uint32_t in_dim, uint32_t out_dim, uint32_t p_rows)
{
    return mmq_dense(s, type, w, xq, y, in_dim, out_dim, p_rows, false);
}

// PrefillGemm's quantize + GEMM for more than RC_MATVEC_MAX_ROWS rows.  Every route below keeps the
// integer block dots exact: the default is the integer-operand f16 kernel of rc_mmq_x.cu (the quantizer
// writes its operand image into the scratch), small matrices with few rows go through 16-row passes of
// the batched matvec, Q5_1 through the dp4a passes.  The f16-dequantized GEMM (rc_mmq_deq.cu) is an
// approximation and runs only when asked for by name (rc_matmul_f16, or rc_tune_mmq kind 32).
int launch_mmq_gemm_f32(cudaStream_t s, int type, const void *w, const float *x, float *y, uint32_t in_dim,
                        uint32_t out_dim, uint32_t p_rows, void *scratch, size_t scratch_bytes)
{
    if (g_mmq_kind == 32 && !g_force_dp4a) {
        if (((uintptr_t)scratch & 15u) != 0) return RC_ERR_MISALIGNED;
        if (scratch_bytes < mmq_deq_scratch_bytes(in_dim, p_rows)) return RC_ERR_SCRATCH_TOO_SMALL;
        return launch_mmq_deq_f32(s, type, w, x, y, in_dim, out_dim, p_rows, scratch);
    }
    if (g_mmq_kind == 0 && !g_force_dp4a) {
        const uint32_t n_sub = in_dim >> 5;
        if (mmq_x_supports(type)) {
            // Small matrices and few rows: the GEMM's fixed cost (two launches, ring start-up, the last drain)
            // and its K steps outlast a few 16-row passes of the batched matvec.  Both costs are modelled
            // from measurements on B200: a 16-row matvec pass takes max(8 us, 0.95 us per million weights);
            // the GEMM 8 us + 0.16 us per K=32 step and wave of 128 x 128 tiles.
            const double t16 = fmax(8.0, 0.95e-6 * (double)in_dim * (double)out_dim);
            const double t_mv = (double)((p_rows + 15u) / 16u) * t16;
            const uint64_t tiles = (uint64_t)((out_dim + 127u) / 128u) * ((p_rows + 127u) / 128u);
            const double waves = (double)((tiles + (uint64_t)sm_count() - 1u) / (uint64_t)sm_count());
            const double steps = (double)n_sub + ((type == Q4_K || type == Q5_K) ? (double)((n_sub + 7u) / 8u) : 0.0);
            const double t_gemm = 8.0 + 0.16 * steps * waves;
            if (t_mv >= t_gemm) {
                if (((uintptr_t)scratch & 15u) != 0) return RC_ERR_MISALIGNED;
                if (scratch_bytes < mmq_x_scratch_bytes(in_dim, p_rows)) return RC_ERR_SCRATCH_TOO_SMALL;
                return launch_mmq_x_f32(s, type, w, x, y, in_dim, out_dim, p_rows, scratch, nullptr);
            }
        }
        // batched-matvec passes (also Q5_1, which has no exact tensor-core kernel)
        int rc = launch_quantize_q8(s, x, scratch, in_dim, p_rows);
        if (rc) return rc;
        for (uint32_t p0 = 0; p0 < p_rows; p0 += 16) {
            const uint32_t n = min(16u, p_rows - p0);
            rc = launch_matvec(s, type, w, (const uint8_t *)scratch + (size_t)p0 * n_sub * RC_BLOCKQ8_BYTES,
                               y + (size_t)p0 * out_dim, in_dim, out_dim, n, nullptr);
            if (rc) return rc;
        }
        return RC_OK;
    }
    // rc_tune_mmq kinds 8 / 16 (and the dp4a switch): the per-sub-block kernels of this file, for A/B timing
    const bool i8_kernel = !g_force_dp4a && g_mmq_kind != 16 && type != Q6_K && type != Q5_1;
    const bool planar = i8_kernel && !g_no_planar && ((uintptr_t)scratch & 15u) == 0 && p_rows <= 65535u &&
                        scratch_bytes >= quantize_planar_bytes(in_dim, p_rows);
    int rc = planar ? launch_quantize_q8_planar(s, x, scratch, in_dim, p_rows)
                    : launch_quantize_q8(s, x, scratch, in_dim, p_rows);
    if (rc) return rc;
    return mmq_dense(s, type, w, scratch, y, in_dim, out_dim, p_rows, planar);
}

namespace {
int mmq_dense(cudaStream_t s, int type, const void *w, const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
              uint32_t p_rows, bool planar)
{
    const uint32_t n_sub = in_dim >> 5;
    const bool use16 = g_mmq_kind == 16 || (g_mmq_kind != 8 && type == Q6_K);
    if ((type != Q6_K || use16) && type != Q5_1 && !g_force_dp4a) { // Q5_1 has no exact-integer tensor-core kernel: dp4a passes below
        MmqParams P;
        P.w = (const uint8_t *)w;
        P.bytes_per_expert = 0;
        P.expert_off = nullptr;
        P.tile_off = nullptr;
        P.n_expert = 1;
        P.xq = (const uint8_t *)xq;
        P.y = y;
        P.in_dim = in_dim;
        P.out_dim = out_dim;
        P.n_tok = p_rows;
        P.planar = planar ? 1u : 0u;
        P.b_tma = 0;
        P.debug = (uint32_t)g_mmq_debug;
        const uint32_t tiles = ((out_dim + kBM - 1) / kBM) * ((p_rows + kDenseBN - 1) / kDenseBN);
        if (use16) {
            switch (type) {
            case Q4_0: return launch_tc16<Q4_0, kDenseBN>(s, P, tiles);
            case Q8_0: return launch_tc16<Q8_0, kDenseBN>(s, P, tiles);
            case Q4_K: return launch_tc16<Q4_K, kDenseBN>(s, P, tiles);
            case Q5_K: return launch_tc16<Q5_K, kDenseBN>(s, P, tiles);
            case Q6_K: return launch_tc16<Q6_K, kDenseBN>(s, P, tiles);
            case IQ4_XS: return launch_tc16<IQ4_XS, kDenseBN>(s, P, tiles);
            case IQ3_S: return launch_tc16<IQ3_S, kDenseBN>(s, P, tiles);
            }
            return RC_ERR_BAD_TYPE;
        }
        switch (type) {
        case Q4_0: return launch_tc<Q4_0, kDenseBN>(s, P, tiles);
        case Q8_0: return launch_tc<Q8_0, kDenseBN>(s, P, tiles);
        case Q4_K: return launch_tc<Q4_K, kDenseBN>(s, P, tiles);
        case Q5_K: return launch_tc<Q5_K, kDenseBN>(s, P, tiles);
        case IQ4_XS: return launch_tc<IQ4_XS, kDenseBN>(s, P, tiles);
        case IQ3_S: return launch_tc<IQ3_S, kDenseBN>(s, P, tiles);
        }
        return RC_ERR_BAD_TYPE;
    }
    for (uint32_t p0 = 0; p0 < p_rows; p0 += 16) {
        const uint32_t n = min(16u, p_rows - p0);
        int rc = launch_matvec(s, type, w, (const uint8_t *)xq + (size_t)p0 * n_sub * RC_BLOCKQ8_BYTES,
                               y + (size_t)p0 * out_dim, in_dim, out_dim, n, nullptr);
        if (rc) return rc;
    }
    return RC_OK;
}
} // namespace

// Expert tiles are kGroupedBN tokens wide (the width rc_moe_sort must be given): at a mean of
// 16 tokens per expert a wider tile would be mostly padding, and the kernel is bound by the
// expert weights it streams, not by the MMA shape.
int launch_mmq_grouped(cudaStream_t s, int type, const void *slab, size_t bytes_per_expert,
                       const int32_t *expert_off, const int32_t *tile_off, uint32_t n_expert,
                       const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
                       uint32_t n_entries)
{
    const bool use16 = g_mmq_kind == 16 || (g_mmq_kind != 8 && type == Q6_K);
    if ((type != Q6_K || use16) && type != Q5_1 && !g_force_dp4a) { // Q5_1 has no exact-integer tensor-core kernel: dp4a passes below
        MmqParams P;
        P.w = (const uint8_t *)slab;
        P.bytes_per_expert = bytes_per_expert;
        P.expert_off = expert_off;
        P.tile_off = tile_off;
        P.n_expert = n_expert;
        P.xq = (const uint8_t *)xq;
        P.y = y;
        P.in_dim = in_dim;
        P.out_dim = out_dim;
        P.n_tok = n_entries;
        P.planar = 0;
        P.b_tma = 0;
        P.debug = (uint32_t)g_mmq_debug;
        // the tile count lives on the device (tile_off[n_expert]); this is its upper bound
        const uint32_t tiles = ((out_dim + kBM - 1) / kBM) * ((n_entries + kGroupedBN - 1) / kGroupedBN + n_expert);
        if (use16) {
            switch (type) {
            case Q4_0: return launch_tc16<Q4_0, kGroupedBN>(s, P, tiles);
            case Q8_0: return launch_tc16<Q8_0, kGroupedBN>(s, P, tiles);
            case Q4_K: return launch_tc16<Q4_K, kGroupedBN>(s, P, tiles);
            case Q5_K: return launch_tc16<Q5_K, kGroupedBN>(s, P, tiles);
            case Q6_K: return launch_tc16<Q6_K, kGroupedBN>(s, P, tiles);
            case IQ4_XS: return launch_tc16<IQ4_XS, kGroupedBN>(s, P, tiles);
            case IQ3_S: return launch_tc16<IQ3_S, kGroupedBN>(s, P, tiles);
            }
            return RC_ERR_BAD_TYPE;
        }
        switch (type) {
        case Q4_0: return launch_tc<Q4_0, kGroupedBN>(s, P, tiles);
        case Q8_0: return launch_tc<Q8_0, kGroupedBN>(s, P, tiles);
        case Q4_K: return launch_tc<Q4_K, kGroupedBN>(s, P, tiles);
        case Q5_K: return launch_tc<Q5_K, kGroupedBN>(s, P, tiles);
        case IQ4_XS: return launch_tc<IQ4_XS, kGroupedBN>(s, P, tiles);
        case IQ3_S: return launch_tc<IQ3_S, kGroupedBN>(s, P, tiles);
        }
        return RC_ERR_BAD_TYPE;
    }
    return launch_matvec_grouped(s, type, slab, bytes_per_expert, expert_off, tile_off, n_expert,
                                 xq, y, in_dim, out_dim, n_entries);
}

} // namespace rc
