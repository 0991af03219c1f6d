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

namespace rc {
namespace {

constexpr int kBM = 128;     // weight rows per tile = tensor-memory lanes
constexpr int kKS = 4;       // sub-blocks (K=32 MMA steps) per pipeline stage
constexpr int kStages = 4;   // operand ring depth
constexpr int kBufs = 4;     // tensor-memory accumulator buffers
constexpr int kThreads = 384;
constexpr int kExpanderThreads = 64;
constexpr int kEpilogueWarps = 8;
constexpr uint64_t kWaitLimitNs = 500ull * 1000 * 1000; // far beyond any legal wait (microseconds)

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
};

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
__device__ __forceinline__ uint64_t global_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after kWaitLimitNs of wall time.  False when the limit ran out (records
// `code`, raises the abort flag) or when another role already raised the flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t code)
{
    if (mbar_try(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > kWaitLimitNs) break;
        }
    }
    atomicExch(&g_mmq_error, code);
    *abort_flag = 1u;
    return false;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1,
                                            int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, "
                 "%4, %5}], [%6];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
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
        iq4_lookup8(q.x, a0, a1);
        iq4_lookup8(q.y, b0, b1);
        iq4_lookup8(q.z, c0, c1);
        iq4_lookup8(q.w, d0, d1);
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
    static constexpr uint32_t raw_off = 0;
    static constexpr uint32_t a_off = raw_off + kStages * raw_stage;
    static constexpr uint32_t b_off = a_off + kStages * kKS * a_sub;
    static constexpr uint32_t dx_off = b_off + kStages * kKS * b_sub;
    static constexpr uint32_t xs_off = dx_off + kStages * kKS * sx_sub;
    static constexpr uint32_t bar_off = xs_off + kStages * kKS * sx_sub;
    // barriers: raw_full, raw_empty, op_full, op_empty [kStages each]; tm_full, tm_empty [kBufs each]
    static constexpr uint32_t n_bars = 4 * kStages + 2 * kBufs;
    static constexpr uint32_t misc_off = bar_off + n_bars * 8; // tmem base slot, abort flag
    static constexpr uint32_t total = misc_off + 16 + 1024;    // + alignment slack
};

template <int FMT, int BN>
__global__ void __launch_bounds__(kThreads, 1)
mmq_kernel(const __grid_constant__ CUtensorMap tmap, const MmqParams P)
{
    using L = Smem<FMT, BN>;
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
            mbar_init(raw_empty(s), kExpanderThreads);
            mbar_init(op_full(s), kExpanderThreads);
            mbar_init(op_empty(s), 1 + kEpilogueWarps);
        }
        for (uint32_t b = 0; b < kBufs; b++) {
            mbar_init(tm_full(b), 1);
            mbar_init(tm_empty(b), kEpilogueWarps);
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
                    if (it >= kStages && !mbar_wait(raw_empty(s), ((it / kStages) - 1u) & 1u, abort_flag, 1u)) break;
                    const uint32_t nsteps = min((uint32_t)kKS, n_sub - i * kKS);
                    mbar_expect_tx(raw_full(s), nsteps * MmqTraits<FMT>::raw_bytes);
                    for (uint32_t j = 0; j < nsteps; j++)
                        for (int pl = 0; pl < MmqTraits<FMT>::raw_planes; pl++)
                            tma_load_4d(sbase + L::raw_off + s * L::raw_stage + j * MmqTraits<FMT>::raw_bytes + pl * kBM * 16,
                                        &tmap, raw_full(s), (int)((i * kKS + j) * 16u), (int)t.m0, pl, (int)t.e);
                }
            }
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
                    mma_commit(op_empty(s)); // the stage's operands are free once its MMAs have run
                }
            }
        mma_done:;
        }
    } else if (warp < 4) {
        // ---- expanders ------------------------------------------------------------------------------
        const uint32_t tid = threadIdx.x - 64u; // 0..63
        constexpr int ROWS_PT = kBM / kExpanderThreads;            // weight rows per thread
        constexpr int ITEMS_PT = BN * kKS / kExpanderThreads;      // (token, sub-block) items per thread
        uint32_t it = 0;
        for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
            const Tile t = decode_tile<BN>(P, id);
            const Planes pl = planes_of<FMT>(P.w + (size_t)t.e * P.bytes_per_expert, P.in_dim, P.out_dim);
            for (uint32_t i = 0; i < n_iters; i++, it++) {
                const uint32_t s = it % kStages;
                const uint32_t k0 = i * kKS, nsteps = min((uint32_t)kKS, n_sub - k0);
                // global loads first: activations of this stage (and the format's side plane)
                uint2 xb[ITEMS_PT][5];
#pragma unroll
                for (int n = 0; n < ITEMS_PT; n++) {
                    const uint32_t q = tid + n * kExpanderThreads, tok = q % BN, j = q / BN;
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
                uint32_t extra[ROWS_PT][kKS];
                if constexpr (FMT == Q5_K) {
#pragma unroll
                    for (int rr = 0; rr < ROWS_PT; rr++) {
                        const uint32_t row = min(t.m0 + tid + rr * kExpanderThreads, P.out_dim - 1u);
#pragma unroll
                        for (int j = 0; j < kKS; j++)
                            if (j < (int)nsteps) extra[rr][j] = ld_stream_u32(pl.aux + ((size_t)row * pl.nsp + k0 + j) * 4);
                    }
                }
                if (it >= kStages && !mbar_wait(op_empty(s), ((it / kStages) - 1u) & 1u, abort_flag, 4u)) goto exp_done;
                if (!mbar_wait(raw_full(s), (it / kStages) & 1u, abort_flag, 5u)) goto exp_done;
                // A: whole weight rows of the tile
#pragma unroll
                for (int rr = 0; rr < ROWS_PT; rr++) {
                    const uint32_t r = tid + rr * kExpanderThreads;
#pragma unroll
                    for (int j = 0; j < kKS; j++) {
                        if (j < (int)nsteps) {
                            const uint8_t *rp = smem + L::raw_off + s * L::raw_stage + j * MmqTraits<FMT>::raw_bytes + r * 16u;
                            const uint4 q = *reinterpret_cast<const uint4 *>(rp);
                            uint4 q2 = make_uint4(0, 0, 0, 0);
                            if constexpr (FMT == Q8_0) q2 = *reinterpret_cast<const uint4 *>(rp + kBM * 16);
                            uint4 lo, hi;
                            expand_weights<FMT>(q, q2, FMT == Q5_K ? extra[rr][j] : 0u, lo, hi);
                            uint8_t *ap = smem + L::a_off + (s * kKS + j) * L::a_sub + r * 16u;
                            *reinterpret_cast<uint4 *>(ap) = lo;
                            *reinterpret_cast<uint4 *>(ap + kBM * 16) = hi;
                        }
                    }
                }
                // B: the int8 quants in the same layout, the scales beside them
#pragma unroll
                for (int n = 0; n < ITEMS_PT; n++) {
                    const uint32_t q = tid + n * kExpanderThreads, tok = q % BN, j = q / BN;
                    if (j < nsteps) {
                        uint8_t *bp = smem + L::b_off + (s * kKS + j) * L::b_sub + tok * 16u;
                        *reinterpret_cast<uint4 *>(bp) = make_uint4(xb[n][1].x, xb[n][1].y, xb[n][2].x, xb[n][2].y);
                        *reinterpret_cast<uint4 *>(bp + BN * 16) = make_uint4(xb[n][3].x, xb[n][3].y, xb[n][4].x, xb[n][4].y);
                        reinterpret_cast<uint32_t *>(smem + L::dx_off + (s * kKS + j) * L::sx_sub)[tok] = xb[n][0].x;
                        reinterpret_cast<uint32_t *>(smem + L::xs_off + (s * kKS + j) * L::sx_sub)[tok] = xb[n][0].y;
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
        const uint32_t half = (warp - 4u) >> 2;    // which half of the BN columns
        constexpr int COLS = BN / 2;               // columns per thread
        constexpr int CHUNKS = COLS / 32 > 0 ? COLS / 32 : 1;
        constexpr int CW = COLS < 32 ? COLS : 32;  // columns per tensor-memory load
        static_assert(COLS == 16 || COLS % 32 == 0, "BN must be 32 or a multiple of 64");
        float acc[COLS];
        uint32_t it = 0, kc = 0;
        for (uint32_t id = blockIdx.x; id < n_tiles && !*abort_flag; id += gridDim.x) {
            const Tile t = decode_tile<BN>(P, id);
            const Planes pl = planes_of<FMT>(P.w + (size_t)t.e * P.bytes_per_expert, P.in_dim, P.out_dim);
            const bool sup_a4 = (reinterpret_cast<uintptr_t>(pl.sup) & 3u) == 0;
            const uint32_t row_raw = t.m0 + quarter * 32u + lane;
            const uint32_t row = min(row_raw, P.out_dim - 1u);
#pragma unroll
            for (int c = 0; c < COLS; c++) acc[c] = 0.0f;
            StageScales cur, nxt;
            load_scales<FMT>(cur, pl, sup_a4, row, 0, min((uint32_t)kKS, n_sub));
            for (uint32_t i = 0; i < n_iters; i++, it++) {
                const uint32_t s = it % kStages;
                const uint32_t k0 = i * kKS, nsteps = min((uint32_t)kKS, n_sub - k0);
                if (i + 1 < n_iters) load_scales<FMT>(nxt, pl, sup_a4, row, k0 + kKS, min((uint32_t)kKS, n_sub - k0 - kKS));
                // the stage's activation scales were written before op_full completed
                if (!mbar_wait(op_full(s), (it / kStages) & 1u, abort_flag, 6u)) goto epi_done;
                float d_sup = 0.0f, dmin_sup = 0.0f;
                if constexpr (MmqTraits<FMT>::has_min) {
                    d_sup = f16_bits_to_f32(cur.dd);
                    dmin_sup = f16_bits_to_f32(cur.dd >> 16);
                }
#pragma unroll
                for (int j = 0; j < kKS; j++) {
                    if (j < (int)nsteps) {
                        const uint32_t b = kc % kBufs;
                        if (!mbar_wait(tm_full(b), (kc / kBufs) & 1u, abort_flag, 7u)) goto epi_done;
                        tc_fence_after();
                        float dsc, ndeff = 0.0f;
                        if constexpr (MmqTraits<FMT>::has_min) {
                            dsc = d_sup * (float)(cur.s[j] & 0xFFu);
                            ndeff = -dmin_sup * (float)(cur.s[j] >> 8);
                        } else {
                            dsc = f16_bits_to_f32(cur.s[j]);
                        }
                        const float *dxp = reinterpret_cast<const float *>(smem + L::dx_off + (s * kKS + j) * L::sx_sub) + half * COLS;
                        const float *xsp = reinterpret_cast<const float *>(smem + L::xs_off + (s * kKS + j) * L::sx_sub) + half * COLS;
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
#pragma unroll
                            for (int c = 0; c < CW; c += 4) {
                                const float4 dx4 = *reinterpret_cast<const float4 *>(dxp + ch * 32 + c);
                                float4 xs4 = make_float4(0.f, 0.f, 0.f, 0.f);
                                if constexpr (MmqTraits<FMT>::has_min) xs4 = *reinterpret_cast<const float4 *>(xsp + ch * 32 + c);
                                const float dxv[4] = {dx4.x, dx4.y, dx4.z, dx4.w};
                                const float xsv[4] = {xs4.x, xs4.y, xs4.z, xs4.w};
#pragma unroll
                                for (int u = 0; u < 4; u++) {
                                    // exact int -> float: bias into [2^23, 2^24) as an integer, remove it as a float
                                    const float z = __uint_as_float(d[c + u] + 0x4B400000u) - 12582912.0f;
                                    float a = acc[ch * 32 + c + u];
                                    a = fmaf(dsc, z * dxv[u], a);
                                    if constexpr (MmqTraits<FMT>::has_min) a = fmaf(ndeff, xsv[u], a);
                                    acc[ch * 32 + c + u] = a;
                                }
                            }
                        }
                        kc++;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(op_empty(s)); // done with the stage's activation scales
                cur = nxt;
            }
            // tile end: Y[tok][row], a warp writes 32 consecutive rows of one token per store
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
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
template <int FMT>
int make_tmap(CUtensorMap *map, const void *w, size_t bytes_per_expert, uint32_t n_expert, uint32_t in_dim,
              uint32_t out_dim)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return RC_ERR_NO_DEVICE;
    const uint64_t nsp = nsp_of(in_dim >> 5);
    const cuuint64_t dims[4] = {nsp * 16, out_dim, (cuuint64_t)MmqTraits<FMT>::raw_planes, n_expert};
    const uint64_t plane = (uint64_t)out_dim * nsp * 16;
    const cuuint64_t strides[3] = {nsp * 16, plane, n_expert > 1 ? (cuuint64_t)bytes_per_expert : plane * 2};
    const cuuint32_t box[4] = {16, kBM, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(w), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? RC_OK : RC_ERR_BAD_ARGUMENT;
}

template <int FMT, int BN>
int launch_tc(cudaStream_t s, const MmqParams &P, uint32_t tiles_upper_bound)
{
    CUtensorMap map;
    int rc = make_tmap<FMT>(&map, P.w, P.bytes_per_expert, P.expert_off ? P.n_expert : 1u, P.in_dim, P.out_dim);
    if (rc) return rc;
    const uint32_t grid = min(tiles_upper_bound, (uint32_t)sm_count());
    mmq_kernel<FMT, BN><<<grid, kThreads, Smem<FMT, BN>::total, s>>>(map, P);
    return (int)cudaGetLastError();
}

template <int FMT, int BN> int set_attr()
{
    return (int)cudaFuncSetAttribute(mmq_kernel<FMT, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)Smem<FMT, BN>::total);
}

constexpr int kDenseBN = 128;
constexpr int kGroupedBN = 32;

bool g_force_dp4a = false;

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
    rc |= set_attr<Q4_0, kGroupedBN>();
    rc |= set_attr<Q8_0, kGroupedBN>();
    rc |= set_attr<Q4_K, kGroupedBN>();
    rc |= set_attr<Q5_K, kGroupedBN>();
    rc |= set_attr<IQ4_XS, kGroupedBN>();
    return rc;
}

void mmq_force_dp4a(int on) { g_force_dp4a = on != 0; }

int mmq_device_error(unsigned int *out)
{
    return (int)cudaMemcpyFromSymbol(out, g_mmq_error, sizeof(unsigned int));
}

// Formats with one scale per 32-wide sub-block run on the tensor cores.  Q6_K scales each half
// of a sub-block separately (kernels/mmq_gemm_q6k_repacked.cpp), which a K=32 int8 MMA cannot
// keep apart; it goes through the dp4a kernel in slabs of 16 activation rows.
int launch_mmq_gemm(cudaStream_t s, int type, const void *w, const void *xq, float *y,
                    uint32_t in_dim, uint32_t out_dim, uint32_t p_rows)
{
    const uint32_t n_sub = in_dim >> 5;
    if (type != Q6_K && !g_force_dp4a) {
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
        const uint32_t tiles = ((out_dim + kBM - 1) / kBM) * ((p_rows + kDenseBN - 1) / kDenseBN);
        switch (type) {
        case Q4_0: return launch_tc<Q4_0, kDenseBN>(s, P, tiles);
        case Q8_0: return launch_tc<Q8_0, kDenseBN>(s, P, tiles);
        case Q4_K: return launch_tc<Q4_K, kDenseBN>(s, P, tiles);
        case Q5_K: return launch_tc<Q5_K, kDenseBN>(s, P, tiles);
        case IQ4_XS: return launch_tc<IQ4_XS, kDenseBN>(s, P, tiles);
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

// Expert tiles are kGroupedBN tokens wide (the width rc_moe_sort must be given): at a mean of
// 16 tokens per expert a wider tile would be mostly padding, and the kernel is bound by the
// expert weights it streams, not by the MMA shape.
int launch_mmq_grouped(cudaStream_t s, int type, const void *slab, size_t bytes_per_expert,
                       const int32_t *expert_off, const int32_t *tile_off, uint32_t n_expert,
                       const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
                       uint32_t n_entries)
{
    if (type != Q6_K && !g_force_dp4a) {
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
        // the tile count lives on the device (tile_off[n_expert]); this is its upper bound
        const uint32_t tiles = ((out_dim + kBM - 1) / kBM) * ((n_entries + kGroupedBN - 1) / kGroupedBN + n_expert);
        switch (type) {
        case Q4_0: return launch_tc<Q4_0, kGroupedBN>(s, P, tiles);
        case Q8_0: return launch_tc<Q8_0, kGroupedBN>(s, P, tiles);
        case Q4_K: return launch_tc<Q4_K, kGroupedBN>(s, P, tiles);
        case Q5_K: return launch_tc<Q5_K, kGroupedBN>(s, P, tiles);
        case IQ4_XS: return launch_tc<IQ4_XS, kGroupedBN>(s, P, tiles);
        }
        return RC_ERR_BAD_TYPE;
    }
    return launch_matvec_grouped(s, type, slab, bytes_per_expert, expert_off, tile_off, n_expert,
                                 xq, y, in_dim, out_dim, n_entries);
}

} // namespace rc
