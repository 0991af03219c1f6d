// Dense prefill GEMM with both operands dequantized to f16 (tcgen05 kind::f16, f32 accumulator in
// tensor memory across the whole K range).
//
// The block-scaled contraction of the reference's MMQ kernels (kernels/mmq_gemm_q4k_repacked.cpp:63-208
// and siblings),
//   Y[tok][row] = sum_sb  dsc[row,sb] * dx[tok,sb] * idot[row,tok,sb]  -  deff[row,sb] * xsum[tok,sb],
// is the plain product  sum_k w[row,k] * a[tok,k]  of the dequantized weights  w = dsc * q  and the
// dequantized BlockQ8 activations  a = dx * qx  (plus, for Q4_K / Q5_K, a second product over the
// sub-blocks:  sum_sb (-deff[row,sb]) * xsum[tok,sb]).  The int8 kernel (rc_mmq.cu) keeps the integer
// dots exact and pays for it with a drain of the accumulator tile after every 32-wide sub-block, on
// the CUDA cores.  Here each operand value is rounded ONCE to f16 (a weight is the product of an exact
// small integer and the format's f16 scale; an activation is dx * qx scaled by a power of two per
// token so that the token's largest value lands in [256, 512)), the accumulator never leaves tensor
// memory until the tile is done, and every weight is expanded once for up to 512 tokens.  The result
// differs from the exact-integer formulation by the two f16 roundings: about 3e-4 in relative L2, a
// third of the 1e-3 that the reference's own GPU-vs-CPU tests allow.
//
// Activations arrive from activations_to_f16_kernel below as the shared-memory image of the B operand:
//   [16-byte chunk of K][token][8 halves]   (main part: in_dim/8 chunks; then the xsum chunks, one half
//   per sub-block; then one f32 per token: the inverse of the token's power-of-two scale)
// so one chunk of a token tile is one contiguous bulk copy.
//
// One persistent CTA per SM, 23 warps: warp 0 one thread issuing the activation bulk copies, warp 1 one
// thread of MMA issue, warp 2 one thread issuing the raw weight TMA loads, warps 3..18 expanders (four
// groups that take the K steps in turn, thread = weight row), warps 19..22 epilogue.  A tile is
// 128 weight rows x BN tokens (BN = 512 fills tensor memory: 128 lanes x 512 f32 columns; 256 and 128
// leave room for two and four accumulator buffers).  Every wait is bounded (see rc_mmq.cu).
#include <cuda.h>

#include <algorithm>

#include "rc_common.cuh"
#include "rc_internal.h"
#include "rc_tc.cuh"

namespace rc {
namespace {

__device__ unsigned int g_mmqd_error;
__device__ unsigned long long g_mmqd_trace[160 * 8]; // measurement aid (debug bit 128): phase timestamps per CTA

__device__ __forceinline__ bool mbar_wait_d(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, uint32_t code)
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
    atomicExch(&g_mmqd_error, code);
    *abort_flag = 1u;
    return false;
}
// The wait of a single-thread role (producers, MMA issuer): a tight spin on the non-blocking probe.
__device__ __forceinline__ bool mbar_spin_d(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, uint32_t code)
{
    long long t0 = 0;
    for (uint32_t spin = 1;; spin++) {
        if (mbar_test(bar, parity)) return true;
        if ((spin & 1023u) == 0u) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitCycles) break;
        }
    }
    atomicExch(&g_mmqd_error, code);
    *abort_flag = 1u;
    return false;
}
// The same wait made by lane 0 for its warp (one poller instead of 32).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, uint32_t code)
{
    uint32_t ok = 1u;
    if ((threadIdx.x & 31u) == 0u) ok = mbar_wait_d(bar, parity, abort_flag, code) ? 1u : 0u;
    return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0u;
}

// Contiguous global -> shared copy by the TMA unit (no tensor map), completion counted on `bar`.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

template <int FMT> struct DeqTraits {
    static constexpr bool has_min = (FMT == Q4_K || FMT == Q5_K || FMT == Q5_1);
    static constexpr bool sup_scale = (FMT == Q4_K || FMT == Q5_K || FMT == Q6_K); // f16 d per superblock
    static constexpr int raw_planes = (FMT == Q8_0) ? 2 : 1;
    static constexpr uint32_t raw_bytes = raw_planes * kBM * 16;
};

template <int BN> struct DeqCfg {
    // Sub-blocks (K = 32 each) per operand-ring stage.  A ring hand-over costs about 0.25 us whatever it
    // carries; at the 32-column expert tiles the MMAs of one sub-block last a tenth of that, so a stage
    // carries four of them and the hand-overs per tile drop fourfold.
    static constexpr uint32_t ks = BN == 32 ? 4 : 1;
    static constexpr uint32_t stages = (BN == 512 || BN == 32) ? 4 : 8;
    static constexpr uint32_t bufs = 512 / BN;
};

template <int FMT, int BN> struct SmemD {
    static constexpr uint32_t stages = DeqCfg<BN>::stages;
    // the raw weight planes come from HBM and run far ahead of the operand ring, in a ring of their own
    static constexpr uint32_t ks = DeqCfg<BN>::ks;
    // (a raw stage, like an operand stage, holds ks sub-blocks: [sub-slot][plane][row][16 B])
    static constexpr uint32_t raw_stages = ks > 1 ? (FMT == Q8_0 ? 2 : 4) : (BN >= 256 && FMT == Q8_0) ? 8 : 16;
    static constexpr uint32_t raw_stage = ks * DeqTraits<FMT>::raw_bytes;
    static constexpr uint32_t a_stage = ks * kBM * 64;  // 128 rows x 32 ks halves: [chunk 0..4 ks - 1][row][16 B]
    static constexpr uint32_t b_stage = ks * BN * 64;   // BN tokens x 32 ks halves: [chunk 0..4 ks - 1][token][16 B]
    static constexpr uint32_t raw_off = 0;
    static constexpr uint32_t a_off = raw_off + raw_stages * raw_stage;
    static constexpr uint32_t b_off = a_off + stages * a_stage;
    static constexpr uint32_t bar_off = b_off + stages * b_stage;
    static constexpr uint32_t n_bars = 2 * stages + 2 * raw_stages + 2 * DeqCfg<BN>::bufs;
    static constexpr uint32_t misc_off = bar_off + n_bars * 8;
    static constexpr uint32_t total = misc_off + 16 + 1024;
};

struct DeqParams {
    const uint8_t *w;
    const uint8_t *xh;      // f16 operand image written by activations_to_f16_kernel
    const float *inv_scale; // per token
    float *y;
    uint32_t in_dim, out_dim, n_tok, tok_ld;
    // expert-grouped form (expert_off != nullptr): rows of the image are expert-sorted entries, expert e
    // owns entries expert_off[e]..expert_off[e+1] and token tiles tile_off[e]..tile_off[e+1], its weights
    // are w + e * bytes_per_expert
    size_t bytes_per_expert;
    const int32_t *expert_off, *tile_off;
    uint32_t n_expert;
    uint32_t k_splits; // dense form only: work items per tile, each over a contiguous range of K steps, added into a zeroed y
    uint32_t debug; // measurement aid: pipeline parts to skip (results invalid): 1 expand, 2 activation copies, 4 MMAs, 8 raw loads; 64 no K split (results valid); 128 records phase timestamps
};

constexpr int kExpGroups = 4;                // groups of four expander warps, one K step each in turn
constexpr int kExpWarps = 4 * kExpGroups, kEpiWarps = 4;
constexpr int kLeadWarps = 3;                // activation producer, MMA issuer, raw weight producer
constexpr int kDeqThreads = (kLeadWarps + kExpWarps + kEpiWarps) * 32;

__device__ __forceinline__ uint4 mul_h2x4(const uint4 &v, __half2 s)
{
    return make_uint4(h2_as_u32(__hmul2(u32_as_h2(v.x), s)), h2_as_u32(__hmul2(u32_as_h2(v.y), s)),
                      h2_as_u32(__hmul2(u32_as_h2(v.z), s)), h2_as_u32(__hmul2(u32_as_h2(v.w), s)));
}
__device__ __forceinline__ uint4 add_h2x4(const uint4 &a, const uint4 &b)
{
    return make_uint4(h2_as_u32(__hadd2(u32_as_h2(a.x), u32_as_h2(b.x))), h2_as_u32(__hadd2(u32_as_h2(a.y), u32_as_h2(b.y))),
                      h2_as_u32(__hadd2(u32_as_h2(a.z), u32_as_h2(b.z))), h2_as_u32(__hadd2(u32_as_h2(a.w), u32_as_h2(b.w))));
}
__device__ __forceinline__ __half2 h2_from_bits(uint32_t bits16)
{
    const uint32_t b = bits16 & 0xFFFFu;
    return u32_as_h2(b | (b << 16));
}

// Q6_K for this kernel: (q - 32) as an exact f16 integer, times f16(d * sc) of its 16-weight half.  Two
// roundings per weight (the half's scale, the product) like the exact two-part form of expand_f16 (whose
// sum rounds beyond 2048, then the product with d), at two thirds of its instructions: the expanders
// bound this format's steps.
__device__ __forceinline__ void expand_q6k_scaled(const uint4 &q, uint32_t e0, uint32_t e1, uint32_t sm, uint32_t d_bits, uint4 (&o)[4])
{
    const uint32_t M = 0x0F0F0F0Fu;
    uint32_t g[8];
    spread_fields4(e0, g[0], g[1], g[2], g[3]);
    spread_fields4(e1, g[4], g[5], g[6], g[7]);
    const float d = f16_bits_to_f32(d_bits);
    const __half2 s_lo = __float2half2_rn(d * (float)(int)(int8_t)(sm & 0xFFu));
    const __half2 s_hi = __float2half2_rn(d * (float)(int)(int8_t)((sm >> 8) & 0xFFu));
    const __half2 one = __half2half2(__float2half(1.0f)), off = __half2half2(__float2half(-1056.0f)); // 1024 + q -> q - 32
    o[0] = mul_h2x4(kc_block((q.x & M) | g[0], (q.y & M) | g[2], one, off), s_lo);
    o[1] = mul_h2x4(kc_block((q.z & M) | g[4], (q.w & M) | g[6], one, off), s_lo);
    o[2] = mul_h2x4(kc_block(((q.x >> 4) & M) | g[1], ((q.y >> 4) & M) | g[3], one, off), s_hi);
    o[3] = mul_h2x4(kc_block(((q.z >> 4) & M) | g[5], ((q.w >> 4) & M) | g[7], one, off), s_hi);
}

struct DeqTile {
    uint32_t m0, tok0, n_valid, e;
};

// Tile id -> weight-row tile, first token row of the image, valid tokens, expert.  Dense: ids walk the
// row tiles of one token tile after another.  Grouped: the same with global token tiles of BN entries,
// mapped to (expert, local tile) by binary search over tile_off (kernels/mmq_gemm_q4k_grouped.cpp:49-60).
template <int BN, bool GR, bool SPLIT = false>
__device__ __forceinline__ DeqTile deq_tile(const DeqParams &P, uint32_t id, uint32_t tiles_m)
{
    DeqTile t;
    t.m0 = (id % tiles_m) * kBM;
    uint32_t gt = id / tiles_m;
    if constexpr (!GR) {
        t.e = 0;
        if constexpr (SPLIT) gt %= (P.n_tok + BN - 1) / BN; // the K split is the slowest index of a dense tile id
        t.tok0 = gt * BN;
        t.n_valid = min((uint32_t)BN, P.n_tok - t.tok0);
    } else {
        uint32_t lo = 0, hi = P.n_expert;
        while (lo + 1 < hi) {
            const uint32_t mid = (lo + hi) >> 1;
            if ((uint32_t)P.tile_off[mid] <= gt) lo = mid; else hi = mid;
        }
        t.e = lo;
        t.tok0 = (uint32_t)P.expert_off[lo] + (gt - (uint32_t)P.tile_off[lo]) * BN;
        t.n_valid = min((uint32_t)BN, (uint32_t)P.expert_off[lo + 1] - t.tok0);
    }
    return t;
}

// SPLIT: the K-split form of the dense kernel, a separate instantiation so that the plain one keeps its
// register budget (the kernel runs at the 80-register cap of its 736 threads).
template <int FMT, int BN, bool GR, bool SPLIT = false>
__global__ void __launch_bounds__(kDeqThreads, 1) mmqd_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap bmap, const DeqParams P)
{
    using L = SmemD<FMT, BN>;
    using T = DeqTraits<FMT>;
    constexpr uint32_t S = L::stages, R = L::raw_stages, NB = DeqCfg<BN>::bufs, KS = L::ks;
    constexpr bool kAllDrain = (NB == 1);
    constexpr uint32_t kDrainWarps = kAllDrain ? kExpWarps + kEpiWarps : kEpiWarps;
    constexpr uint32_t kExpanders = 4; // arrivals per stage: lane 0 of each warp of one expander group
    static_assert(KS > 1 || (L::stages % kExpGroups == 0 && L::raw_stages % kExpGroups == 0), "a stage always belongs to the same expander group");
    static_assert(KS == 1 || KS == kExpGroups, "with several sub-blocks per stage, group g always fills sub-slot g");
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bars = sbase + L::bar_off;
    auto op_full = [&](uint32_t s) { return bars + s * 8u; };
    auto op_empty = [&](uint32_t s) { return bars + (S + s) * 8u; };
    auto raw_full = [&](uint32_t s) { return bars + (2 * S + s) * 8u; };
    auto raw_empty = [&](uint32_t s) { return bars + (2 * S + R + s) * 8u; };
    auto tm_full = [&](uint32_t b) { return bars + (2 * S + 2 * R + b) * 8u; };
    auto tm_empty = [&](uint32_t b) { return bars + (2 * S + 2 * R + NB + b) * 8u; };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::misc_off);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const bool trace = (P.debug & 128u) && blockIdx.x < 160u;
    if (trace && threadIdx.x == 0) g_mmqd_trace[blockIdx.x * 8 + 0] = global_ns();
    const uint32_t n_sub = P.in_dim >> 5;
    const uint32_t n_extra = T::has_min ? (n_sub + 31u) / 32u : 0u; // K=32 steps over the sub-block minima
    const uint32_t n_real = n_sub + n_extra;
    const uint32_t n_iters = (n_real + KS - 1u) / KS * KS; // per tile; steps past n_real carry zero weights (the image's zero tail as B)
    const uint32_t tiles_m = (P.out_dim + kBM - 1) / kBM;
    const uint32_t tiles_n = GR ? (uint32_t)P.tile_off[P.n_expert] : (P.n_tok + BN - 1) / BN; // grouped: known on the device only
    const uint32_t k_splits = SPLIT ? P.k_splits : 1u;
    const uint32_t n_tiles = tiles_m * tiles_n * k_splits;
    // K steps [k0, k1) of work item id
    auto krange = [&](uint32_t id, uint32_t &k0, uint32_t &k1) {
        if (k_splits <= 1u) {
            k0 = 0u;
            k1 = n_iters;
        } else {
            const uint32_t per = (n_real + k_splits - 1u) / k_splits;
            k0 = (id / (tiles_m * tiles_n)) * per;
            k1 = min(n_real, k0 + per);
        }
    };

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; s++) {
            mbar_init(op_full(s), KS * kExpanders + 1); // expanders (A) of every sub-slot + the producer's expect_tx (B)
            mbar_init(op_empty(s), 1);             // the commit after the stage's MMAs
        }
        for (uint32_t s = 0; s < R; s++) {
            mbar_init(raw_full(s), 1);
            mbar_init(raw_empty(s), KS * kExpanders);
        }
        for (uint32_t b = 0; b < NB; b++) {
            mbar_init(tm_full(b), 1);
            mbar_init(tm_empty(b), kDrainWarps);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (trace && threadIdx.x == 0) g_mmqd_trace[blockIdx.x * 8 + 1] = global_ns();
    pdl_launch_dependents();
    pdl_wait(); // the activation image is the predecessor's output
    if (trace && threadIdx.x == 0) g_mmqd_trace[blockIdx.x * 8 + 2] = global_ns();

    // Tensor memory -> y for one finished tile: the warp's lane quarter, the 32-column chunks rank,
    // rank + n_ranks, ...; one inverse token scale per column.  Arrives on tm_empty when done.
    auto drain = [&](uint32_t id, uint32_t tile, uint32_t rank, uint32_t n_ranks) -> bool {
        const uint32_t quarter = warp & 3u; // tensor-memory lanes this warp may read
        const DeqTile tl = deq_tile<BN, GR, SPLIT>(P, id, tiles_m);
        const uint32_t m0 = tl.m0, tok0 = tl.tok0, n_valid = tl.n_valid;
        const uint32_t buf = tile % NB;
        const uint32_t row = m0 + quarter * 32u + lane;
        if (!mbar_wait_d(tm_full(buf), (tile / NB) & 1u, abort_flag, 7u)) return false;
        tc_fence_after();
        if (trace && warp == kLeadWarps + kExpWarps && lane == 0) g_mmqd_trace[blockIdx.x * 8 + 5] = global_ns();
        float *yrow = P.y + (size_t)tok0 * P.out_dim + row;
        for (uint32_t ch = rank; ch < BN / 32u; ch += n_ranks) {
            const uint32_t col0 = ch * 32u;
            if (col0 >= n_valid) break; // warp-uniform
            uint32_t d[32];
            tmem_ld32(tmem_base + ((quarter * 32u) << 16) + buf * BN + col0, d);
            const float inv = (col0 + lane < n_valid) ? __ldg(P.inv_scale + tok0 + col0 + lane) : 0.0f; // lane c: column col0 + c
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; c++) {
                const float sc = __shfl_sync(0xFFFFFFFFu, inv, c);
                if (row < P.out_dim && col0 + c < n_valid) {
                    if (k_splits > 1u) atomicAdd(&yrow[(size_t)(col0 + c) * P.out_dim], __uint_as_float(d[c]) * sc);
                    else yrow[(size_t)(col0 + c) * P.out_dim] = __uint_as_float(d[c]) * sc;
                }
            }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tm_empty(buf));
        if (trace && warp == kLeadWarps + kExpWarps && lane == 0) g_mmqd_trace[blockIdx.x * 8 + 6] = global_ns();
        return true;
    };
    // With a single accumulator buffer (BN = 512) the next tile cannot start before this one is
    // drained, so the expander warps drain too: five warps per lane quarter.

    if (warp == 0) {
        if constexpr (KS == 1) {
            // ---- activation producer: chunks 4i..4i+3 of the image per K step, by bulk copies -------------
            if (lane == 0) {
                uint32_t it = 0;
                for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
                    const uint32_t tok0 = deq_tile<BN, GR, SPLIT>(P, id, tiles_m).tok0;
                    const uint32_t n_rows_b = min((uint32_t)BN, P.tok_ld - tok0); // rows present in the image (a grouped tile may
                                                                                  // take the next expert's first rows along: unused columns)
                    uint32_t k0, k1;
                    krange(id, k0, k1);
                    for (uint32_t i = k0; i < k1; i++, it++) {
                        const uint32_t s = it % S;
                        if (it >= S && !mbar_spin_d(op_empty(s), ((it / S) - 1u) & 1u, abort_flag, 2u)) goto prod_done;
                        if (P.debug & 2u) {
                            mbar_arrive(op_full(s));
                            continue;
                        }
                        mbar_expect_tx(op_full(s), 4u * n_rows_b * 16u);
                        // (the xsum chunks follow the main ones seamlessly)
                        const uint8_t *src = P.xh + ((size_t)(4u * i) * P.tok_ld + tok0) * 16u;
                        for (uint32_t c = 0; c < 4; c++)
                            bulk_load(sbase + L::b_off + s * L::b_stage + c * BN * 16u, src + (size_t)c * P.tok_ld * 16u,
                                      n_rows_b * 16u, op_full(s));
                    }
                }
            prod_done:;
            }
        } else {
            // ---- activation producer, KS > 1: chunks 4i .. 4(i + KS) - 1 of the image per stage in ONE tiled TMA
            // load (box 16 B x BN tokens x 4 KS chunks of the 3-D view in bmap; sixteen separate bulk copies per
            // stage were on the critical path of the narrow tiles).  The image has a whole tile of spare rows
            // and a zero tail of chunks, so no box leaves it.
            if (lane == 0) {
                uint32_t m = 0; // stages issued
                for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
                    const uint32_t tok0 = deq_tile<BN, GR, SPLIT>(P, id, tiles_m).tok0;
                    uint32_t k0, k1;
                    krange(id, k0, k1);
                    for (uint32_t i = k0; i < k1; i += KS, m++) {
                        const uint32_t s = m % S;
                        if (m >= S && !mbar_spin_d(op_empty(s), ((m / S) - 1u) & 1u, abort_flag, 2u)) goto prod4_done;
                        if (P.debug & 2u) {
                            mbar_arrive(op_full(s));
                            continue;
                        }
                        mbar_expect_tx(op_full(s), L::b_stage);
                        tma_load_3d(sbase + L::b_off + s * L::b_stage, &bmap, op_full(s), 0, (int)tok0, (int)(4u * i));
                    }
                }
            prod4_done:;
            }
        }
    } else if (warp == 2) {
        // ---- raw weight producer: one 16-byte x 128-row box per plane and sub-block, by tiled TMA; one
        // barrier round per stage of KS sub-blocks ----------------------------------------------------------
        if (lane == 0) {
            uint32_t m = 0; // stages issued
            for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
                const DeqTile tl = deq_tile<BN, GR, SPLIT>(P, id, tiles_m);
                const uint32_t m0 = tl.m0;
                uint32_t k0, k1;
                krange(id, k0, k1);
                for (uint32_t i = k0; i < k1; i += KS, m++) {
                    const uint32_t s = m % R;
                    if (m >= R && !mbar_spin_d(raw_empty(s), ((m / R) - 1u) & 1u, abort_flag, 1u)) goto raw_done;
                    const uint32_t n_raw = i < n_sub ? min((uint32_t)KS, n_sub - i) : 0u; // sub-blocks with weights in this stage
                    if (n_raw && !(P.debug & 8u)) {
                        // the map's box is 16 KS bytes wide: the stage's sub-blocks of a row in one load, landing
                        // as [plane][row][16 KS bytes] (columns past the row's last sub-block arrive as padding)
                        mbar_expect_tx(raw_full(s), L::raw_stage);
                        for (int pl = 0; pl < T::raw_planes; pl++)
                            tma_load_4d(sbase + L::raw_off + s * L::raw_stage + pl * (KS * kBM * 16), &tmap, raw_full(s), (int)(i * 16u), (int)m0,
                                        pl, (int)tl.e);
                    } else {
                        mbar_arrive(raw_full(s)); // nothing raw in a minima stage; keeps the ring in phase
                    }
                }
            }
        raw_done:;
        }
    } else if (warp == 1) {
        // ---- MMA issuer -------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t NI = BN > 256 ? 256 : BN; // columns per instruction
            constexpr uint32_t idesc = make_idesc_f16(NI);
            // Descriptors differ from stage 0's only in the start-address field (bits 0..13, in units of
            // 16 bytes; shared memory never carries out of it): one add per MMA instead of rebuilding them,
            // which keeps this thread's instruction stream shorter than the MMAs it feeds.
            const uint64_t da0 = make_desc(sbase + L::a_off, kBM * 16, 128);
            const uint64_t db0 = make_desc(sbase + L::b_off, BN * 16, 128);
            const bool do_mma = !(P.debug & 4u);
            uint32_t it = 0, tile = 0;
            for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x, tile++) {
                const uint32_t buf = tile % NB;
                if (tile >= NB && !mbar_spin_d(tm_empty(buf), ((tile / NB) - 1u) & 1u, abort_flag, 3u)) goto mma_done;
                tc_fence_after();
                const uint32_t d0 = tmem_base + buf * BN;
                uint32_t k0, k1;
                krange(id, k0, k1);
                for (uint32_t i = k0; i < k1; i += KS, it++) { // it counts stages here
                    const uint32_t s = it % S;
                    if (!mbar_test(op_full(s), (it / S) & 1u) && !mbar_spin_d(op_full(s), (it / S) & 1u, abort_flag, 4u)) goto mma_done;
                    tc_fence_after();
                    if (trace && it == 0) g_mmqd_trace[blockIdx.x * 8 + 3] = global_ns();
                    const uint64_t da = da0 + (uint64_t)(s * (L::a_stage >> 4));
                    const uint64_t db = db0 + (uint64_t)(s * (L::b_stage >> 4));
                    if (do_mma) {
#pragma unroll
                        for (uint32_t kh = 0; kh < 2 * KS; kh++) { // K = 16 per instruction: two chunks
#pragma unroll
                            for (uint32_t nh = 0; nh < BN / NI; nh++) {
                                mma_f16(d0 + nh * NI, da + kh * ((2 * kBM * 16) >> 4), db + ((kh * 2 * BN * 16 + nh * NI * 16) >> 4), idesc,
                                        ((i - k0) | kh) ? 1u : 0u); // the work item's first K=16 step overwrites every column
                            }
                        }
                    }
                    mma_commit(op_empty(s));
                }
                mma_commit(tm_full(buf));
                if (trace) g_mmqd_trace[blockIdx.x * 8 + 4] = global_ns();
            }
        mma_done:;
        }
    } else if (warp < kLeadWarps + kExpWarps) {
        // ---- expanders: kExpGroups groups of 128 threads take the K steps in turn; in a group thread r
        // owns weight row m0 + r.  Side planes (scales, high bits) come from HBM: they are requested three
        // of the group's steps early, into three fixed register slots used in turn.
        constexpr uint32_t G = kExpGroups;
        const uint32_t grp = (warp - kLeadWarps) >> 2, r = (threadIdx.x - kLeadWarps * 32u) & 127u;
        struct Side { uint32_t e0, e1, smw, ddw; };
        uint32_t tile_it0 = 0, tile_no = 0; // global step number of the work item's first step; work items done
        uint32_t k0 = 0, k1 = 0;
        for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x, tile_it0 += k1 - k0, tile_no += SPLIT ? 1u : 0u) {
            const DeqTile tl = deq_tile<BN, GR, SPLIT>(P, id, tiles_m);
            krange(id, k0, k1);
            const Planes pl = planes_of<FMT>(P.w + (size_t)tl.e * P.bytes_per_expert, P.in_dim, P.out_dim);
            const uint32_t row = min(tl.m0 + r, P.out_dim - 1u);
            const uint8_t *scp = pl.sc + (size_t)row * pl.nsp * (FMT == Q5_1 ? 4u : 2u);
            const uint8_t *auxp = (FMT == Q5_K || FMT == Q5_1 || FMT == Q6_K) ? pl.aux + (size_t)row * pl.nsp * (FMT == Q6_K ? 8u : 4u) : nullptr;
            const uint8_t *supp = T::sup_scale ? pl.sup + (size_t)row * pl.n_super * (FMT == Q6_K ? 2u : 4u) : nullptr;
            auto request = [&](Side &slot, uint32_t i) {
                slot = Side{0u, 0u, 0u, 0u};
                if (i < n_sub) {
                    if constexpr (FMT == Q5_K || FMT == Q5_1) slot.e0 = ld_stream_u32(auxp + i * 4u);
                    if constexpr (FMT == Q6_K) {
                        const uint2 h = ld_stream_u2(auxp + i * 8u);
                        slot.e0 = h.x;
                        slot.e1 = h.y;
                    }
                    if constexpr (FMT == Q5_1) slot.smw = ld_stream_u32(scp + i * 4u); // d | m << 16; d is the f16 scale
                    else slot.smw = ld_nc_u16(scp + i * 2u);
                    if constexpr (T::has_min && T::sup_scale) slot.ddw = ld_nc_u16(supp + (i >> 3) * 4u);
                    if constexpr (FMT == Q6_K) slot.ddw = ld_nc_u16(supp + (i >> 3) * 2u);
                }
            };
            auto step = [&](Side &slot, uint32_t i) -> bool {
                const Side cur = slot;
                request(slot, i + 3u * G);
                const uint32_t it = tile_it0 + (i - k0), mst = it / KS, s = mst % S, rs = mst % R;
                uint4 o[4];
                if (i >= n_sub) o[0] = o[1] = o[2] = o[3] = make_uint4(0u, 0u, 0u, 0u); // minima steps fill it below; steps past the last are zero
                if constexpr (T::has_min) {
                    if (i >= n_sub && i < n_real) {
                        // minima step: chunk c = superblock (i - n_sub) * 4 + c, one half per sub-block: -dmin * m
                        const uint32_t sb0 = (i - n_sub) * 4u;
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            uint32_t h[4] = {0u, 0u, 0u, 0u};
                            if constexpr (FMT == Q5_1) {
                                // the term is + m * xsum: the raw fp16 m of sub-blocks 8 * (sb0 + c) + 0..7
#pragma unroll
                                for (int u = 0; u < 4; u++) {
                                    const uint32_t s0 = (sb0 + c) * 8u + 2u * u;
                                    const uint32_t m_lo = s0 < n_sub ? ld_nc_u16(scp + s0 * 4u + 2u) : 0u;
                                    const uint32_t m_hi = s0 + 1u < n_sub ? ld_nc_u16(scp + (s0 + 1u) * 4u + 2u) : 0u;
                                    h[u] = m_lo | (m_hi << 16);
                                }
                            } else if (sb0 + c < pl.n_super) {
                                const uint32_t dmin_bits = ld_nc_u16(supp + (sb0 + c) * 4u + 2u);
                                const __half2 ndm = __hneg2(h2_from_bits(dmin_bits));
#pragma unroll
                                for (int u = 0; u < 4; u++) {
                                    const uint32_t m_lo = ld_nc_u16(scp + ((sb0 + c) * 8u + 2 * u) * 2u) >> 8;
                                    const uint32_t m_hi = ld_nc_u16(scp + ((sb0 + c) * 8u + 2 * u + 1) * 2u) >> 8;
                                    const __half2 mm = __halves2half2(__ushort2half_rn((unsigned short)m_lo),
                                                                      __ushort2half_rn((unsigned short)m_hi));
                                    h[u] = h2_as_u32(__hmul2(mm, ndm));
                                }
                            }
                            o[c] = make_uint4(h[0], h[1], h[2], h[3]);
                        }
                    }
                }
                if (!mbar_wait_d(raw_full(rs), (mst / R) & 1u, abort_flag, 6u)) return false;
                if (i < n_sub && !(P.debug & 1u)) {
                    const uint32_t rp = sbase + L::raw_off + rs * L::raw_stage + r * (16u * KS) + (it % KS) * 16u;
                    const uint4 q = lds_u4(rp);
                    uint4 q2 = make_uint4(0, 0, 0, 0);
                    if constexpr (FMT == Q8_0) q2 = lds_u4(rp + KS * kBM * 16);
                    if constexpr (FMT == Q6_K) {
                        expand_q6k_scaled(q, cur.e0, cur.e1, cur.smw, cur.ddw, o);
                    } else {
                        uint4 t[2][4];
                        expand_f16<FMT>(q, q2, cur.e0, cur.e1, cur.smw, t); // exact integers: sc * q, q - 8, q, codebook value
                        const __half2 sc = h2_from_bits(T::sup_scale ? cur.ddw : cur.smw);
#pragma unroll
                        for (int c = 0; c < 4; c++) o[c] = mul_h2x4(t[0][c], sc);
                    }
                }
                // the operand slot is needed only now: the expansion above ran while its MMAs finished
                if (mst >= S && !mbar_wait_d(op_empty(s), ((mst / S) - 1u) & 1u, abort_flag, 5u)) return false;
                const uint32_t ap = sbase + L::a_off + s * L::a_stage + (it % KS) * (4u * kBM * 16u) + r * 16u;
#pragma unroll
                for (int c = 0; c < 4; c++) sts_u4(ap + c * kBM * 16, o[c]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp(); // one arrival per warp
                if (lane == 0) {
                    mbar_arrive(op_full(s));
                    mbar_arrive(raw_empty(rs));
                }
                return true;
            };
            uint32_t i = k0 + (grp + G - (tile_it0 % G)) % G; // the group's first step in this work item
            Side slot0, slot1, slot2;
            request(slot0, i);
            request(slot1, i + G);
            request(slot2, i + 2u * G);
            bool ok = true;
            while (ok && i < k1) {
                ok = step(slot0, i);
                i += G;
                if (ok && i < k1) {
                    ok = step(slot1, i);
                    i += G;
                }
                if (ok && i < k1) {
                    ok = step(slot2, i);
                    i += G;
                }
            }
            if (!ok) break;
            if constexpr (kAllDrain) {
                if (!drain(id, SPLIT ? tile_no : tile_it0 / n_iters, grp, kExpGroups + 1u)) break;
            }
        }
    } else {
        // ---- epilogue warps ---------------------------------------------------------------------------------
        uint32_t tile = 0;
        for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x, tile++)
            if (!drain(id, tile, kAllDrain ? (uint32_t)kExpGroups : 0u, kAllDrain ? kExpGroups + 1u : 1u)) break;
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
        if (trace && lane == 0) g_mmqd_trace[blockIdx.x * 8 + 7] = global_ns();
    }
}

// ---- activations: f32 rows -> the f16 operand image ---------------------------------------------------
//
// One CTA of 32 warps per 8 consecutive tokens (gridDim.y CTAs share the sub-blocks of those tokens).
// Pass 1: the tokens' largest magnitudes (four warps per token), giving the power-of-two scales.
// Pass 2: a warp takes one sub-block of all 8 tokens at a time: the BlockQ8 quantizer of
// quantize_q8_kernel (kernels/quantize_q8.cpp:23-66: same sum butterfly, same IEEE divides, same
// rounding), a = f16((d * q) * s) and f16(xsum * s); the 8 x 32 halves are transposed through shared
// memory so that every store instruction writes one chunk of the 8 tokens: 128 contiguous bytes of
// the image.  Tokens n_tok..tok_ld-1 are written as zeros.
constexpr int kActTokens = 8, kActWarps = 32;

// Where row t of the image comes from: row (index ? index[t] / div : t) of x, rows row_stride floats
// apart; with act >= 0 a source row is [gate | up] of 2 * in_dim floats and the value is
// act(gate) * up (0: tanh GELU, 1: SiLU; kernels/moe_geglu_q8.cpp:20-32, kernels/swiglu.cpp:11-21).
struct ActSource {
    const float *x;
    const int32_t *index;
    uint32_t div;
    size_t row_stride;
    int act;
};

__device__ __forceinline__ float act_value(const float *row, uint32_t i, uint32_t in_dim, int act)
{
    if (act < 0) return row[i];
    const float g = row[i], u = row[in_dim + i];
    float a;
    if (act == 0) {
        const float c = g + 0.044715f * g * g * g;
        a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * c));
    } else {
        a = g / (1.0f + expf(-g));
    }
    return __fmul_rn(a, u);
}

__global__ void __launch_bounds__(kActWarps * 32) activations_to_f16_kernel(const ActSource src, uint8_t *__restrict__ out,
                                                                             uint32_t in_dim, uint32_t n_tok, uint32_t tok_ld,
                                                                             uint32_t n_xchunks)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t n_sub = in_dim >> 5, n_kc = in_dim >> 3;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t tok0 = blockIdx.x * kActTokens;
    float *inv_scale = reinterpret_cast<float *>(out + (size_t)(n_kc + n_xchunks) * tok_ld * 16u);
    __shared__ float s_part[kActTokens][4];
    __shared__ float s_scale[kActTokens];
    __shared__ __align__(16) __half s_tile[kActWarps][kActTokens][32];

    {   // pass 1: warp -> (token, quarter of the row)
        const uint32_t t = warp >> 2, qk = warp & 3u, tok = tok0 + t;
        float amax = 0.0f;
        // an entry the sort dropped (perm = -1: an expert id outside the table) is a row of zeros, never a load
        if (tok < n_tok && !(src.index && src.index[tok] < 0)) {
            const float *row = src.x + (size_t)(src.index ? (uint32_t)src.index[tok] / src.div : tok) * src.row_stride;
            const uint32_t per = in_dim / 4u, lo = qk * per, hi = lo + per; // in_dim is a multiple of 32
            if (src.act >= 0) {
#pragma unroll 4
                for (uint32_t i = lo + lane; i < hi; i += 32u) amax = fmaxf(amax, fabsf(act_value(row, i, in_dim, src.act)));
            } else if ((reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
                const float4 *r4 = reinterpret_cast<const float4 *>(row);
#pragma unroll 4
                for (uint32_t i = lo / 4u + lane; i < hi / 4u; i += 32u) {
                    const float4 v = __ldg(r4 + i);
                    amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
                }
            } else {
#pragma unroll 4
                for (uint32_t i = lo + lane; i < hi; i += 32u) amax = fmaxf(amax, fabsf(row[i]));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        if (lane == 0) s_part[t][qk] = amax;
    }
    __syncthreads();
    if (threadIdx.x < kActTokens) {
        const uint32_t t = threadIdx.x;
        const float amax = fmaxf(fmaxf(s_part[t][0], s_part[t][1]), fmaxf(s_part[t][2], s_part[t][3]));
        // s = 2^(8 - floor(log2 amax)): amax * s in [256, 512); a block sum is then below 2^14
        const uint32_t ebits = (__float_as_uint(amax) >> 23) & 0xFFu;
        const bool scaled = ebits >= 9u && ebits <= 254u;
        s_scale[t] = scaled ? __uint_as_float((262u - ebits) << 23) : 1.0f;
        if (blockIdx.y == 0 && tok0 + t < tok_ld)
            inv_scale[tok0 + t] = tok0 + t >= n_tok ? 0.0f : scaled ? __uint_as_float((ebits - 8u) << 23) : 1.0f;
    }
    __syncthreads();

    // pass 2: sub-blocks warp + 32 * (blockIdx.y + gridDim.y * k)
    const uint32_t tl = lane >> 2, pair = lane & 3u; // store role: token tl, halves 2*pair, 2*pair + 1 of a chunk
    const float s_mine = s_scale[lane & 7u];         // lane t < 8 also does token t's divides and xsum
    const float *rows[kActTokens];
    uint32_t live = 0u; // bit t: token t of the group has a source row
#pragma unroll
    for (int t = 0; t < kActTokens; t++) {
        const uint32_t tok = min(tok0 + t, n_tok - 1u);
        const bool dropped = src.index && src.index[tok] < 0;
        rows[t] = src.x + (size_t)(src.index ? (dropped ? 0u : (uint32_t)src.index[tok] / src.div) : tok) * src.row_stride;
        if (tok0 + t < n_tok && !dropped) live |= 1u << t;
    }
    for (uint32_t sb = warp + 32u * blockIdx.y; sb < n_sub; sb += 32u * gridDim.y) {
        float v[kActTokens], sum[kActTokens];
        uint32_t bmax[kActTokens]; // |v| as bits: non-negative floats order like unsigned integers
#pragma unroll
        for (int t = 0; t < kActTokens; t++) {
            v[t] = ((live >> t) & 1u) ? act_value(rows[t], sb * 32u + lane, in_dim, src.act) : 0.0f;
            const float a = fabsf(v[t]);
            bmax[t] = __reduce_max_sync(0xFFFFFFFFu, a == a ? __float_as_uint(a) : 0u); // fmaxf skips a NaN: so does this
            sum[t] = v[t];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int t = 0; t < kActTokens; t++) sum[t] = __fadd_rn(sum[t], __shfl_xor_sync(0xFFFFFFFFu, sum[t], o));
        }
        // the two IEEE divides of a block, once per token: lane t does token t's
        float my_max = 0.0f, my_sum = 0.0f;
#pragma unroll
        for (int t = 0; t < kActTokens; t++) {
            if ((int)(lane & 7u) == t) {
                my_max = __uint_as_float(bmax[t]);
                my_sum = sum[t];
            }
        }
        const float my_d = my_max > 0.0f ? __fdiv_rn(my_max, 127.0f) : 1.0f;
        const float my_inv = my_max > 0.0f ? __fdiv_rn(127.0f, my_max) : 0.0f;
#pragma unroll
        for (int t = 0; t < kActTokens; t++) {
            const float d = __shfl_sync(0xFFFFFFFFu, my_d, t), inv = __shfl_sync(0xFFFFFFFFu, my_inv, t);
            int q = __float2int_rn(__fmul_rn(v[t], inv));
            q = max(-127, min(127, q));
            s_tile[warp][t][lane] = __float2half_rn(__fmul_rn(__fmul_rn(d, (float)q), s_scale[t]));
        }
        __syncwarp();
        if (tok0 + tl < tok_ld) {
#pragma unroll
            for (uint32_t c = 0; c < 4; c++) {
                const uint32_t h2 = *reinterpret_cast<const uint32_t *>(&s_tile[warp][tl][8u * c + 2u * pair]);
                *reinterpret_cast<uint32_t *>(out + ((size_t)(sb * 4u + c) * tok_ld + tok0 + tl) * 16u + pair * 4u) = h2;
            }
        }
        if (lane < kActTokens && tok0 + lane < tok_ld)
            *reinterpret_cast<__half *>(out + ((size_t)(n_kc + (sb >> 3)) * tok_ld + tok0 + lane) * 16u + (sb & 7u) * 2u) =
                __float2half_rn(__fmul_rn(my_sum, s_mine));
        __syncwarp();
    }
    // xsum slots past the last sub-block (the minima steps read whole groups of four chunks)
    if (blockIdx.y == 0)
        for (uint32_t i = n_sub * kActTokens + threadIdx.x; i < n_xchunks * 8u * kActTokens; i += blockDim.x) {
            const uint32_t slot = i / kActTokens, t = i % kActTokens;
            if (tok0 + t < tok_ld)
                *reinterpret_cast<__half *>(out + ((size_t)(n_kc + (slot >> 3)) * tok_ld + tok0 + t) * 16u + (slot & 7u) * 2u) = __float2half(0.0f);
        }
}

// Chunks after the main ones: the sub-block sums (eight per chunk, a whole K = 32 step of four chunks at a
// time), then zero chunks up to a whole stage of the widest ring (four sub-blocks).
uint32_t xchunks_of(uint32_t in_dim)
{
    const uint32_t n_sub = in_dim >> 5;
    const uint32_t steps = (n_sub + (n_sub + 31u) / 32u + 3u) & ~3u; // K = 32 steps of a tile, with the minima, padded
    return 4u * (steps - n_sub);
}
uint32_t tok_ld_of(uint32_t n_tok) { return (n_tok + 7u) & ~7u; }

template <int FMT, int BN>
int launch_deq(cudaStream_t s, const DeqParams &P)
{
    CUtensorMap map;
    int rc = make_tmap<FMT>(&map, P.w, 0, 1u, P.in_dim, P.out_dim);
    if (rc) return rc;
    const uint32_t tiles = ((P.out_dim + kBM - 1) / kBM) * ((P.n_tok + BN - 1) / BN) * P.k_splits;
    const uint32_t grid = min(tiles, (uint32_t)sm_count());
    if (P.k_splits > 1u)
        return (int)launch_pdl(mmqd_kernel<FMT, BN, false, true>, dim3(grid), dim3(kDeqThreads), SmemD<FMT, BN>::total, s, map, map, P);
    return (int)launch_pdl(mmqd_kernel<FMT, BN, false>, dim3(grid), dim3(kDeqThreads), SmemD<FMT, BN>::total, s, map, map, P); // (no image map: bulk copies)
}

constexpr int kGroupedDeqBN = 32; // the expert tile of rc_moe_sort

template <int FMT>
int launch_deq_grouped(cudaStream_t s, const DeqParams &P)
{
    CUtensorMap map;
    int rc = make_tmap<FMT>(&map, P.w, P.bytes_per_expert, P.n_expert, P.in_dim, P.out_dim, 16u * DeqCfg<kGroupedDeqBN>::ks);
    if (rc) return rc;
    // the tile count lives on the device (tile_off[n_expert]); this is its upper bound
    const uint64_t tiles = (uint64_t)((P.out_dim + kBM - 1) / kBM) * ((P.n_tok + kGroupedDeqBN - 1) / kGroupedDeqBN + P.n_expert);
    const uint32_t grid = (uint32_t)std::min<uint64_t>(tiles, (uint64_t)sm_count());
    // 3-D view of the activation image: (16 bytes of a chunk, image row, chunk); one box = a stage of the B ring
    CUtensorMap bmap;
    {
        EncodeTiledFn fn = encode_fn();
        if (!fn) return RC_ERR_NO_DEVICE;
        const uint64_t n_chunks = (uint64_t)(P.in_dim >> 3) + xchunks_of(P.in_dim);
        const cuuint64_t dims[3] = {16, P.tok_ld, n_chunks};
        const cuuint64_t strides[2] = {16, (cuuint64_t)P.tok_ld * 16u};
        const cuuint32_t box[3] = {16, (cuuint32_t)kGroupedDeqBN, 4u * DeqCfg<kGroupedDeqBN>::ks};
        const cuuint32_t estr[3] = {1, 1, 1};
        if (fn(&bmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t *>(P.xh), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return RC_ERR_BAD_ARGUMENT;
    }
    return (int)launch_pdl(mmqd_kernel<FMT, kGroupedDeqBN, true>, dim3(grid), dim3(kDeqThreads), SmemD<FMT, kGroupedDeqBN>::total, s,
                           map, bmap, P);
}

template <int FMT>
int launch_deq_bn(cudaStream_t s, const DeqParams &P, uint32_t bn)
{
    if (bn == 512) return launch_deq<FMT, 512>(s, P);
    if (bn == 256) return launch_deq<FMT, 256>(s, P);
    return launch_deq<FMT, 128>(s, P);
}

template <int FMT> int set_attr_deq()
{
    int rc = (int)cudaFuncSetAttribute(mmqd_kernel<FMT, 512, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SmemD<FMT, 512>::total);
    rc |= (int)cudaFuncSetAttribute(mmqd_kernel<FMT, 256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SmemD<FMT, 256>::total);
    rc |= (int)cudaFuncSetAttribute(mmqd_kernel<FMT, 128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SmemD<FMT, 128>::total);
    rc |= (int)cudaFuncSetAttribute(mmqd_kernel<FMT, 512, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SmemD<FMT, 512>::total);
    rc |= (int)cudaFuncSetAttribute(mmqd_kernel<FMT, 256, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SmemD<FMT, 256>::total);
    rc |= (int)cudaFuncSetAttribute(mmqd_kernel<FMT, 128, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SmemD<FMT, 128>::total);
    rc |= (int)cudaFuncSetAttribute(mmqd_kernel<FMT, kGroupedDeqBN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)SmemD<FMT, kGroupedDeqBN>::total);
    return rc;
}

int g_deq_bn = 0; // 0: by shape
int g_deq_debug = 0;

} // namespace

int mmq_deq_set_attributes()
{
    return set_attr_deq<Q4_0>() | set_attr_deq<Q5_1>() | set_attr_deq<Q8_0>() | set_attr_deq<Q4_K>() | set_attr_deq<Q5_K>() | set_attr_deq<Q6_K>() |
           set_attr_deq<IQ4_XS>() | set_attr_deq<IQ3_S>();
}

void mmq_deq_set_bn(int bn)
{
    g_deq_debug = bn >> 12;
    bn &= 0xFFF;
    g_deq_bn = (bn == 128 || bn == 256 || bn == 512) ? bn : 0;
}

int mmq_deq_read_trace(void *out, size_t bytes)
{
    return (int)cudaMemcpyFromSymbol(out, g_mmqd_trace, bytes < sizeof(g_mmqd_trace) ? bytes : sizeof(g_mmqd_trace));
}

int mmq_deq_device_error(unsigned int *out, bool clear)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, g_mmqd_error, sizeof(unsigned int));
    if (e == cudaSuccess && clear && *out) {
        const unsigned int zero = 0;
        e = cudaMemcpyToSymbol(g_mmqd_error, &zero, sizeof(unsigned int));
    }
    return (int)e;
}

size_t mmq_deq_scratch_bytes(uint32_t in_dim, uint32_t n_tok)
{
    const size_t ld = tok_ld_of(n_tok);
    return ((size_t)(in_dim >> 3) + xchunks_of(in_dim)) * ld * 16u + ld * sizeof(float);
}

// x f32 [n_tok][in_dim] -> y f32 [n_tok][out_dim]; scratch 16-byte aligned, mmq_deq_scratch_bytes large.
int launch_mmq_deq_f32(cudaStream_t s, int type, const void *w, const float *x, float *y, uint32_t in_dim, uint32_t out_dim,
                       uint32_t n_tok, void *scratch)
{
    const uint32_t ld = tok_ld_of(n_tok), n_xc = xchunks_of(in_dim);
    // 8 tokens per CTA; a second CTA shares their sub-blocks while that still adds SMs
    const uint32_t groups = ld / kActTokens, ysplit = groups * 2u <= (uint32_t)sm_count() ? 2u : 1u;
    // Few tiles (a narrow matrix, or a row shard of one): every tile runs its whole K on one SM while the
    // others idle, and a K step costs the same at every width.  Then each tile becomes up to four work
    // items over contiguous ranges of K steps that add their partial sums into a zeroed y.
    const uint32_t bn = g_deq_bn ? (uint32_t)g_deq_bn : n_tok > 256u ? 512u : n_tok > 128u ? 256u : 128u;
    uint32_t k_splits = 1;
    {
        const uint32_t n_sub = in_dim >> 5;
        const bool has_min = type == Q4_K || type == Q5_K || type == Q5_1;
        const uint32_t n_real = n_sub + (has_min ? (n_sub + 31u) / 32u : 0u);
        const uint32_t tiles = ((out_dim + kBM - 1) / kBM) * ((n_tok + bn - 1u) / bn);
        if (!(g_deq_debug & 64) && tiles * 2u <= (uint32_t)sm_count())
            k_splits = std::max(1u, std::min(std::min(4u, (uint32_t)sm_count() / tiles), n_real / 32u));
        if (k_splits > 1u) {
            cudaError_t e0 = cudaMemsetAsync(y, 0, (size_t)n_tok * out_dim * sizeof(float), s);
            if (e0 != cudaSuccess) return (int)e0;
        }
    }
    const ActSource src = {x, nullptr, 1u, (size_t)in_dim, -1};
    cudaError_t e = launch_pdl(activations_to_f16_kernel, dim3(groups, ysplit), dim3(kActWarps * 32), 0, s, src, (uint8_t *)scratch, in_dim,
                               n_tok, ld, n_xc);
    if (e != cudaSuccess) return (int)e;
    DeqParams P;
    P.bytes_per_expert = 0;
    P.expert_off = P.tile_off = nullptr;
    P.n_expert = 1;
    P.k_splits = k_splits;
    P.w = (const uint8_t *)w;
    P.xh = (const uint8_t *)scratch;
    P.inv_scale = reinterpret_cast<const float *>((const uint8_t *)scratch + ((size_t)(in_dim >> 3) + n_xc) * ld * 16u);
    P.y = y;
    P.in_dim = in_dim;
    P.out_dim = out_dim;
    P.n_tok = n_tok;
    P.tok_ld = ld;
    P.debug = (uint32_t)g_deq_debug;
    // The widest token tile the batch fills: a K step costs about the same at every width (it is
    // bound by the latency of the operand ring, not by the MMA), so fewer, wider tiles win, and every
    // weight is expanded once per tile column.
    switch (type) {
    case Q4_0: return launch_deq_bn<Q4_0>(s, P, bn);
    case Q5_1: return launch_deq_bn<Q5_1>(s, P, bn);
    case Q8_0: return launch_deq_bn<Q8_0>(s, P, bn);
    case Q4_K: return launch_deq_bn<Q4_K>(s, P, bn);
    case Q5_K: return launch_deq_bn<Q5_K>(s, P, bn);
    case Q6_K: return launch_deq_bn<Q6_K>(s, P, bn);
    case IQ4_XS: return launch_deq_bn<IQ4_XS>(s, P, bn);
    case IQ3_S: return launch_deq_bn<IQ3_S>(s, P, bn);
    }
    return RC_ERR_BAD_TYPE;
}

// ---- expert-grouped form -----------------------------------------------------------------------------
// Image rows = expert-sorted entries (plus one tile of zero rows, so a tile's copy never leaves the image).
static uint32_t grouped_ld(uint32_t n_entries) { return tok_ld_of(n_entries) + kGroupedDeqBN; }

size_t mmq_deq_grouped_scratch_bytes(uint32_t in_dim, uint32_t n_entries)
{
    const size_t ld = grouped_ld(n_entries);
    return ((size_t)(in_dim >> 3) + xchunks_of(in_dim)) * ld * 16u + ld * sizeof(float);
}

// Entry j of the sorted order takes its activations from row (index ? index[j] / div : j) of x (rows
// row_stride floats apart; act >= 0: rows are [gate | up] and the value is act(gate) * up).
// y f32 [n_entries][out_dim] in sorted order.
int launch_mmq_deq_grouped_f32(cudaStream_t s, int type, const void *slab, size_t bytes_per_expert, const int32_t *expert_off,
                               const int32_t *tile_off, uint32_t n_expert, const float *x, const int32_t *index, uint32_t div,
                               size_t row_stride, int act, float *y, uint32_t in_dim, uint32_t out_dim, uint32_t n_entries,
                               void *scratch)
{
    const uint32_t ld = grouped_ld(n_entries), n_xc = xchunks_of(in_dim);
    const uint32_t groups = ld / kActTokens, ysplit = groups * 2u <= (uint32_t)sm_count() ? 2u : 1u;
    const ActSource src = {x, index, div ? div : 1u, row_stride, act};
    cudaError_t e = launch_pdl(activations_to_f16_kernel, dim3(groups, ysplit), dim3(kActWarps * 32), 0, s, src, (uint8_t *)scratch, in_dim,
                               n_entries, ld, n_xc);
    if (e != cudaSuccess) return (int)e;
    DeqParams P;
    P.w = (const uint8_t *)slab;
    P.xh = (const uint8_t *)scratch;
    P.inv_scale = reinterpret_cast<const float *>((const uint8_t *)scratch + ((size_t)(in_dim >> 3) + n_xc) * ld * 16u);
    P.y = y;
    P.in_dim = in_dim;
    P.out_dim = out_dim;
    P.n_tok = n_entries;
    P.tok_ld = ld;
    P.bytes_per_expert = bytes_per_expert;
    P.expert_off = expert_off;
    P.tile_off = tile_off;
    P.n_expert = n_expert;
    P.k_splits = 1;
    P.debug = (uint32_t)g_deq_debug;
    switch (type) {
    case Q4_0: return launch_deq_grouped<Q4_0>(s, P);
    case Q5_1: return launch_deq_grouped<Q5_1>(s, P);
    case Q8_0: return launch_deq_grouped<Q8_0>(s, P);
    case Q4_K: return launch_deq_grouped<Q4_K>(s, P);
    case Q5_K: return launch_deq_grouped<Q5_K>(s, P);
    case Q6_K: return launch_deq_grouped<Q6_K>(s, P);
    case IQ4_XS: return launch_deq_grouped<IQ4_XS>(s, P);
    case IQ3_S: return launch_deq_grouped<IQ3_S>(s, P);
    }
    return RC_ERR_BAD_TYPE;
}

} // namespace rc
