// Dense prefill MMQ GEMM with exact integer block dots (tcgen05 kind::f16 on integer-valued operands).
//
// What is computed is the block-scaled contraction of the reference's MMQ kernels
// (kernels/mmq_gemm_q4k_repacked.cpp:63-208 and siblings):
//   Y[tok][row] = sum_sb  dsc[row,sb] * dx[tok,sb] * idot[row,tok,sb]  -  deff[row,sb] * xsum[tok,sb]
// with idot the exact integer dot of one 32-wide sub-block of quantized weights and BlockQ8
// activations.  Both operands of the tensor-core product are small integers held exactly in f16
// (activations -127..127; weights q, q - 8, q - 32, a codebook value, and for the K-quants sc * q with
// the 6-bit integer sub-scale folded in, at most 63 * 31), every product and every 32-term sum stays
// below 2^24, so the f32 accumulator tile of one K = 32 step IS the integer block dot (times the
// integer sub-scale), bit for bit.  Each sub-block's tile leaves tensor memory and is scaled on the
// CUDA cores, because dx differs per (token, sub-block).
//
// What makes the drain cheap:
//  * tokens are the tensor-memory LANES (the MMA's M side), weight rows the columns: dx[tok, sb] is one
//    scalar per epilogue thread, so a sub-block costs one packed FMA per two elements,
//        inner[col] += dx * tile[col],
//    and only once per superblock of eight sub-blocks the per-row f16 scale comes in:
//        acc[col] += d[row(col), superblock] * inner[col]          (Q4_K, Q5_K, Q6_K)
//    with acc parked in tensor memory between superblocks (registers hold `inner` only);
//  * the "- deff * xsum" term of Q4_K / Q5_K never touches the CUDA cores: -(dmin * m) and xsum are each
//    split into two bf16 pieces and their four cross products ride as extra K steps (one per superblock,
//    issued after the tile's first superblock) that accumulate straight into the parked accumulator
//    (relative error of that term 2^-16; it is not an integer quantity in the reference either: xsum is
//    the f32 sum of the unquantized activations);
//  * formats with one f16 scale per sub-block and no superblock (Q4_0, Q8_0, IQ4_XS, IQ3_S) pay one more
//    packed multiply per pair: acc[col] += (dx * tile[col]) * d[row(col), sb].
//
// Activations arrive from activations_to_q16_kernel as the shared-memory image of the token operand:
//   [16-byte chunk of K][token][8 halves]  main part, in_dim/8 chunks of f16(q);
//   then the minima chunks (bf16: per sub-block xsum_hi, xsum_mid, xsum_hi, xsum_mid; two sub-blocks
//   per chunk, four chunks = one K = 32 step per superblock); then dx as f32 [sub-block][token].
//
// One persistent CTA per SM, 16 warps in three warpgroups with their own register budgets (setmaxnreg):
//   warp 0        one thread issuing the token-operand TMA loads (four 2 KB rows per K step) and the dx box of
//                 each superblock
//   warps 1, 3    two MMA-issuing threads that take the main steps in turn: one thread's barrier probes, MMA
//                 issues and commits of a step last several times longer than the step's MMAs (each barrier
//                 operation costs its thread a round trip to the SM's barrier unit).  Each publishes the index
//                 of its next own step; neither runs more than two steps past the other's, because a parity
//                 probe cannot tell a barrier's coming phase from the one a whole ring cycle earlier
//   warp 2        one thread issuing the raw weight TMA loads
//   warps 4..11   two groups of expanders (thread = weight row) that take the K steps in turn
//   warps 12..15  the epilogue: one warp per tensor-memory lane quarter, thread = one token x the tile's 128
//                 weight rows, the tile's columns streamed through two register buffers so that the next
//                 tensor-memory load is in flight while the current chunk is accumulated
// A tile is 128 tokens x 128 weight rows; tensor memory holds 3..4 transient sub-block tiles and the parked
// accumulator.  Every wait is bounded: when a limit runs out the kernel records a code, raises a CTA-wide abort
// flag, every role leaves its loop, tensor memory is freed and the launch ends.
//
// Rings without an "empty" barrier (dx boxes, per-superblock row scales, per-sub-block row scales) rely
// on the bounded skew of the pipeline: a producer or expander is never more than S + NB main steps
// ahead of an epilogue warp (operand ring depth + transient tiles), and each of those rings is deeper
// than that.
//
// Measurement aids (results invalid or timing perturbed; rc_tune_mmq kinds 64..66): a PROF instantiation with
// per-role cycle counters, and a mask of pipeline parts to skip.  What they showed on B200: with every load,
// MMA, expansion and FMA skipped the kernel took as long as with all of them, i.e. the serial single-thread
// roles and their barrier operations set the pace, not the tensor pipe (14 % busy) nor the FP32 pipes.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>

#include "rc_common.cuh"
#include "rc_internal.h"
#include "rc_tc.cuh"

namespace rc {
namespace {

__device__ unsigned int g_mmqx_error;
// measurement aid (PROF instantiations only): per CTA, per role, cycles spent in each wait / phase
__device__ unsigned long long g_mmqx_prof[160 * 32];

// The CTA-wide abort flag lives in shared memory and is passed around as its 32-bit shared address.
__device__ __forceinline__ uint32_t flag_get(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void flag_set(uint32_t addr, uint32_t v)
{
    asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ bool mbar_wait_x(uint32_t bar, uint32_t parity, uint32_t abort_flag, uint32_t code)
{
    if (mbar_test(bar, parity)) return true;
    long long t0 = 0;
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (flag_get(abort_flag)) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitCycles) break;
        }
    }
    atomicExch(&g_mmqx_error, code);
    flag_set(abort_flag, 1u);
    return false;
}
// the MMA issuers: a tight spin on the non-blocking probe (the roles whose wake-up latency is on the critical path)
__device__ __forceinline__ bool mbar_spin_x(uint32_t bar, uint32_t parity, uint32_t abort_flag, uint32_t code)
{
    long long t0 = 0;
    for (uint32_t spin = 1;; spin++) {
        if (mbar_test(bar, parity)) return true;
        if ((spin & 1023u) == 0u) {
            if (flag_get(abort_flag)) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitCycles) break;
        }
    }
    atomicExch(&g_mmqx_error, code);
    flag_set(abort_flag, 1u);
    return false;
}

__device__ __forceinline__ void tmem_ld8x(uint32_t taddr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st8x(uint32_t taddr, const uint32_t (&r)[8])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16x(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st16x(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                 "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// packed pairs of f32: one issue slot for two elements
__device__ __forceinline__ unsigned long long pk2(uint32_t lo, uint32_t hi)
{
    unsigned long long d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
__device__ __forceinline__ void upk2(unsigned long long v, uint32_t &lo, uint32_t &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long xmul2(unsigned long long a, unsigned long long b)
{
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long xadd2(unsigned long long a, unsigned long long b)
{
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long xfma2(unsigned long long a, unsigned long long b, unsigned long long c)
{
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void lds_v4(uint32_t addr, uint4 &q)
{
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(addr) : "memory");
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v)
{
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// f32 accumulator, bf16 A and B, both K-major, M = 128 (the minima steps)
__host__ __device__ constexpr uint32_t make_idesc_bf16(uint32_t n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

constexpr uint32_t kXT = 128;       // tokens per tile: tensor-memory lanes, the MMA's M
constexpr uint32_t kXN = 128;       // weight rows per tile: tensor-memory columns, the MMA's N
constexpr uint32_t kXGroups = 2;    // expander groups of four warps
constexpr uint32_t kXLead = 4, kXExpW = 4 * kXGroups, kXEpiW = 4; // lead: token producer, MMA issuer, raw producer, second MMA issuer
constexpr uint32_t kXThreads = (kXLead + kXExpW + kXEpiW) * 32;
constexpr uint32_t kSupSlots = 4;   // superblocks of dx / row scales in flight
constexpr uint32_t kSbSlots = 16;   // per-sub-block row scales in flight (formats without superblocks)

template <int FMT> struct XTraits {
    static constexpr bool has_min = (FMT == Q4_K || FMT == Q5_K);
    static constexpr bool sup = (FMT == Q4_K || FMT == Q5_K || FMT == Q6_K); // integer sub-scales under an f16 d per 256
    static constexpr uint32_t w_parts = (FMT == Q6_K) ? 2 : 1;                // operands accumulated per sub-block
    static constexpr uint32_t raw_planes = (FMT == Q8_0) ? 2 : 1;
    static constexpr uint32_t raw_bytes = raw_planes * kXN * 16;
    static constexpr uint32_t S = (FMT == Q6_K) ? 6 : 8;   // operand ring
    static constexpr uint32_t R = (FMT == Q8_0) ? 8 : 16;  // raw weight ring (runs ahead: it comes from HBM)
    static constexpr uint32_t NB = sup ? 3 : 4;            // transient sub-block tiles in tensor memory
    static constexpr uint32_t acc_col = NB * kXN;          // parked accumulator (sup formats); the minima steps of
                                                           // Q4_K / Q5_K accumulate straight into it
    static_assert(S % kXGroups == 0 && R % kXGroups == 0, "a stage always belongs to the same expander group");
    static_assert(8 * (kSupSlots - 1) >= S + NB + 8, "superblock rings deeper than the pipeline's skew");
    static_assert(kSbSlots >= S + NB + 1, "sub-block scale ring deeper than the pipeline's skew");
};

template <int FMT> struct SmemX {
    using T = XTraits<FMT>;
    static constexpr uint32_t tok_stage = kXT * 64;              // [chunk 0..3][token][16 B]
    static constexpr uint32_t w_stage = T::w_parts * kXN * 64;   // [part][chunk 0..3][row][16 B]
    static constexpr uint32_t raw_off = 0;
    static constexpr uint32_t tok_off = raw_off + T::R * T::raw_bytes;
    static constexpr uint32_t w_off = tok_off + T::S * tok_stage;
    static constexpr uint32_t dx_off = w_off + T::S * w_stage;                 // [slot][8 sub-blocks][token] f32
    static constexpr uint32_t dcol_off = dx_off + kSupSlots * 8 * kXT * 4;     // sup: [slot][row] f32; else [slot 0..15][row] f32
    static constexpr uint32_t dcol_bytes = (T::sup ? kSupSlots : kSbSlots) * kXN * 4;
    static constexpr uint32_t bar_off = dcol_off + dcol_bytes;
    // op_full[S] op_empty[S] raw_full[R] raw_empty[R] tm_full[NB] tm_empty[NB] sup_full[kSupSlots] acc_ready acc_free
    static constexpr uint32_t n_bars = 2 * T::S + 2 * T::R + 2 * T::NB + kSupSlots + 2;
    static constexpr uint32_t misc_off = bar_off + n_bars * 8;
    // per epilogue warp: 32 tokens x 32 finished columns, rows 144 bytes apart (16-byte accesses without bank conflicts both
    // ways), for the transposed stores into the peers' outputs
    static constexpr uint32_t xpose_row = 144, xpose_warp = 32 * xpose_row;
    static constexpr uint32_t xpose_off = (misc_off + 16 + 15) & ~15u;
    static constexpr uint32_t total = misc_off + 16 + 1024; // misc: tmem base, abort flag, the two issuers' progress words
    static constexpr uint32_t total_gather = xpose_off + 4 * xpose_warp + 1024; // the instantiation that stores into peers
    static_assert(total_gather <= 227u * 1024u, "shared memory budget");
};

struct XParams {
    const uint8_t *w;
    float *y[RC_MAX_PEERS]; // the output matrix on this device and, for a row shard that gathers itself, its peers' copies
    uint32_t n_y, ld_out, col_off; // copies; row pitch of the output; first column (weight row) this launch owns
    int32_t *dump;   // debug variant: the integer tile of every (token, row, sub-block)
    uint32_t in_dim, out_dim, n_tok, tok_ld;
    uint32_t y_vec4; // y rows may be written with 16-byte stores
    uint32_t debug;  // measurement aid, pipeline parts to skip (results invalid): 1 the drain's arithmetic, 2 the weight expansion, 4 the MMAs, 8 the drain's tensor-memory loads, 16 the raw weight loads, 32 the token loads, 64 the side-plane loads, 128 the expanders' proxy fence
};

struct XTile {
    uint32_t m0, tok0, n_valid;
};
// token tile fastest: CTAs running at the same time share a weight row tile (it comes from HBM once)
__device__ __forceinline__ XTile x_tile(const XParams &P, uint32_t id, uint32_t tiles_t)
{
    XTile t;
    t.m0 = (id / tiles_t) * kXN;
    t.tok0 = (id % tiles_t) * kXT;
    t.n_valid = min(kXT, P.n_tok - t.tok0);
    return t;
}

__device__ __forceinline__ uint32_t bf16_bits(float v) { return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float bf16_val(uint32_t b) { return __uint_as_float(b << 16); }

template <int FMT, bool DUMP, bool PROF = false, bool GATHER = false>
__global__ void __launch_bounds__(kXThreads, 1)
mmqx_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap tokmap,
            const __grid_constant__ CUtensorMap dxmap, const XParams P)
{
    using L = SmemX<FMT>;
    using T = XTraits<FMT>;
    constexpr uint32_t S = T::S, R = T::R, NB = T::NB, G = kXGroups;
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
    auto sup_full = [&](uint32_t q) { return bars + (2 * S + 2 * R + 2 * NB + q) * 8u; };
    const uint32_t acc_ready = bars + (2 * S + 2 * R + 2 * NB + kSupSlots) * 8u, acc_free = acc_ready + 8u;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::misc_off);
    const uint32_t abort_flag = sbase + L::misc_off + 4u;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n_sub = P.in_dim >> 5;
    const uint32_t n_sup = (n_sub + 7u) >> 3;            // superblocks (dx boxes) per tile
    const uint32_t n_main = 8u * n_sup;                  // main steps, padded to whole superblocks (padding: zero tokens, zero scale)
    const uint32_t n_extra = T::has_min ? n_sup : 0u;    // minima steps: one K = 32 step per superblock
    const uint32_t n_steps = n_main + n_extra;
    const uint32_t n_chunks = (P.in_dim >> 3) + 4u * n_sup; // chunks of the image; a box at or past it arrives as zeros
    const uint32_t tiles_t = (P.n_tok + kXT - 1) / kXT;
    const uint32_t n_tiles = ((P.out_dim + kXN - 1) / kXN) * tiles_t;
    // Order of a tile's K steps.  Q4_K / Q5_K: the first superblock's main steps, then all the minima steps
    // (they accumulate into the parked accumulator, which the epilogue first touches at the end of the first
    // superblock: by then they are done, and the previous tile's last read of it is long past when they
    // start), then the remaining main steps.  Other formats: main steps only.
    auto step_of = [&](uint32_t p, bool &is_min) -> uint32_t {
        is_min = false;
        if constexpr (T::has_min) {
            if (p < 8u) return p;
            if (p < 8u + n_extra) {
                is_min = true;
                return p - 8u;
            }
            return p - n_extra;
        } else {
            return p;
        }
    };

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; s++) {
            mbar_init(op_full(s), 4 + 1);  // the four warps of one expander group + the producer's expect_tx
            mbar_init(op_empty(s), 1);     // the commit after the stage's MMAs
        }
        for (uint32_t s = 0; s < R; s++) {
            mbar_init(raw_full(s), 1);
            mbar_init(raw_empty(s), 4);
        }
        for (uint32_t b = 0; b < NB; b++) {
            mbar_init(tm_full(b), 1);
            mbar_init(tm_empty(b), kXEpiW);
        }
        for (uint32_t q = 0; q < kSupSlots; q++) mbar_init(sup_full(q), T::sup ? 1 + 4 : 1); // dx box (+ the row scales)
        mbar_init(acc_ready, 1);
        mbar_init(acc_free, kXEpiW);
        flag_set(abort_flag, 0u);
        flag_set(abort_flag + 4u, 0u); // index of the first issuer's next own step
        flag_set(abort_flag + 8u, 1u); // ... and of the second's
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
    pdl_launch_dependents();
    pdl_wait(); // the activation image is the predecessor's output
    // PROF: tick(k) adds the cycles since the previous tick to counter k of this thread's role
    long long pt = 0;
    unsigned long long pc[6] = {0, 0, 0, 0, 0, 0};
    auto tick = [&](int k) {
        if constexpr (PROF) {
            const long long now = clock64();
            pc[k] += (unsigned long long)(now - pt);
            pt = now;
        }
    };
    auto prof_out = [&](uint32_t role) {
        if constexpr (PROF) {
            if (blockIdx.x < 160u)
                for (int k = 0; k < 6; k++) g_mmqx_prof[blockIdx.x * 32u + role * 6u + k] = pc[k];
        }
    };
    if constexpr (PROF) pt = clock64();

    // Registers follow the roles (setmaxnreg works on whole warpgroups of four warps): the launch gives each of
    // the 512 threads 128; the lead warpgroup keeps 40 and the expanders 112, which frees 15360 registers, of
    // which the epilogue warpgroup takes 13312 to reach 232 (128 for a token's 128 running sums, 64 for two
    // 32-column chunks in flight).
    // Each setmaxnreg sits at the top of its role's branch, so that no other role's code follows it.
    if (warp < kXLead) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
      if (warp == 0) {
        // ---- token-operand producer: one tiled TMA load per K step (16 B x 128 tokens x 4 chunks), and the
        // dx box (128 tokens x 8 sub-blocks) when a superblock begins -----------------------------------------
        if (lane == 0) {
            uint32_t it = 0, sj = 0;
            for (uint32_t id = blockIdx.x; id < n_tiles && !flag_get(abort_flag); id += gridDim.x) {
                const XTile t = x_tile(P, id, tiles_t);
                for (uint32_t p = 0; p < n_steps; p++, it++) {
                    const uint32_t s = it % S;
                    bool is_min;
                    const uint32_t i = step_of(p, is_min);
                    tick(0);
                    if (it >= S && !mbar_wait_x(op_empty(s), ((it / S) - 1u) & 1u, abort_flag, 1u)) goto tok_done;
                    tick(1);
                    if (!is_min && (i & 7u) == 0u) {
                        const uint32_t q = sj % kSupSlots;
                        mbar_expect_tx(sup_full(q), 8u * kXT * 4u); // a whole box: parts outside the plane arrive as zeros
                        tma_load_2d(sbase + L::dx_off + q * (8u * kXT * 4u), &dxmap, sup_full(q), (int)t.tok0, (int)i);
                        sj++;
                    }
                    if (P.debug & 32u) {
                        mbar_arrive(op_full(s));
                        continue;
                    }
                    mbar_expect_tx(op_full(s), L::tok_stage);
                    // main chunks 4 i ..; the minima chunks follow the main ones; a padding step reads past the image (zeros)
                    tma_load_2d(sbase + L::tok_off + s * L::tok_stage, &tokmap, op_full(s), (int)(t.tok0 * 2u),
                                (int)(is_min ? 4u * (n_sub + i) : i < n_sub ? 4u * i : n_chunks));
                }
            }
        tok_done:;
            prof_out(0);
        }
      } else if (warp == 2) {
        // ---- raw weight producer: one 16-byte x 128-row box per plane and sub-block -------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            for (uint32_t id = blockIdx.x; id < n_tiles && !flag_get(abort_flag); id += gridDim.x) {
                const XTile t = x_tile(P, id, tiles_t);
                for (uint32_t p = 0; p < n_steps; p++, it++) {
                    const uint32_t rs = it % R;
                    bool is_min;
                    const uint32_t i = step_of(p, is_min);
                    if (it >= R && !mbar_wait_x(raw_empty(rs), ((it / R) - 1u) & 1u, abort_flag, 2u)) goto raw_done;
                    if (!is_min && !(P.debug & 16u)) { // (a padding step's box lies past the row: zeros)
                        mbar_expect_tx(raw_full(rs), T::raw_bytes);
                        for (uint32_t pl = 0; pl < T::raw_planes; pl++)
                            tma_load_4d(sbase + L::raw_off + rs * T::raw_bytes + pl * (kXN * 16u), &wmap, raw_full(rs), (int)(i * 16u),
                                        (int)t.m0, (int)pl, 0);
                    } else {
                        mbar_arrive(raw_full(rs)); // nothing raw in a minima step; keeps the ring in phase
                    }
                }
            }
        raw_done:;
        }
      } else if (warp == 1 || warp == 3) {
        // ---- MMA issuers: two threads take the main steps in turn (one thread's barrier probes, MMA issues and
        // commits of a step outlast the step's MMAs several times over); the minima steps, which accumulate into one
        // tile in order, all belong to the first ----------------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(kXN), idesc_min = make_idesc_bf16(kXN);
            const uint64_t dt0 = make_desc(sbase + L::tok_off, kXT * 16, 128);
            const uint64_t dw0 = make_desc(sbase + L::w_off, kXN * 16, 128);
            const uint32_t me = warp == 1 ? 0u : 1u;
            const uint32_t prog_me = abort_flag + 4u + 4u * me, prog_other = abort_flag + 4u + 4u * (me ^ 1u);
            uint32_t it = 0, tile = 0, turn = 0; // turn: whose main step comes next
            uint32_t b = 0, bph = 0, brounds = 0; // transient tile in turn, its phase, whether every tile has been used once
            for (uint32_t id = blockIdx.x; id < n_tiles && !flag_get(abort_flag); id += gridDim.x, tile++) {
                for (uint32_t p = 0; p < n_steps; p++, it++) {
                    const uint32_t s = it % S;
                    bool is_min;
                    const uint32_t j = step_of(p, is_min);
                    if (is_min ? me != 0u : turn != me) {
                        // the other issuer's step: keep the bookkeeping in step
                        if (!is_min) {
                            turn ^= 1u;
                            if (++b == NB) {
                                b = 0;
                                bph ^= 1u;
                                brounds = 1u;
                            }
                        }
                        continue;
                    }
                    tick(0);
                    // Never more than two steps ahead of the other issuer's next step: a parity probe only tells the
                    // coming phase of a barrier from the one a whole ring cycle earlier if that earlier step has been
                    // issued (the second issuer would otherwise leap over the minima steps, several ring cycles).
                    if (it >= 2u && flag_get(prog_other) < it - 2u) {
                        long long t0 = clock64();
                        while (flag_get(prog_other) < it - 2u) {
                            if (flag_get(abort_flag)) goto mma_done;
                            if (clock64() - t0 > kWaitLimitCycles) {
                                atomicExch(&g_mmqx_error, 12u);
                                flag_set(abort_flag, 1u);
                                goto mma_done;
                            }
                        }
                    }
                    {
                        // both probes in flight together; the spins only run for the one that failed
                        const bool t1 = mbar_test(op_full(s), (it / S) & 1u);
                        const bool t2 = (is_min || !brounds) ? true : mbar_test(tm_empty(b), bph ^ 1u);
                        if (!t1 && !mbar_spin_x(op_full(s), (it / S) & 1u, abort_flag, 3u)) goto mma_done;
                        if (!t2 && !mbar_spin_x(tm_empty(b), bph ^ 1u, abort_flag, 4u)) goto mma_done;
                    }
                    tick(1);
                    const uint64_t dt = dt0 + (uint64_t)(s * (L::tok_stage >> 4));
                    const uint64_t dw = dw0 + (uint64_t)(s * (L::w_stage >> 4));
                    if (!is_min) {
                        tick(2);
                        tc_fence_after();
#pragma unroll
                        for (uint32_t part = 0; part < T::w_parts; part++) {
#pragma unroll
                            for (uint32_t kh = 0; kh < 2; kh++) // K = 16 per instruction: two chunks
                                if (!(P.debug & 4u)) mma_f16(tmem_base + b * kXN, dt + kh * ((2 * kXT * 16) >> 4),
                                        dw + ((part * kXN * 64 + kh * 2 * kXN * 16) >> 4), idesc, (part | kh) ? 1u : 0u);
                        }
                        if (P.debug & 256u) mbar_arrive(tm_full(b)); else mma_commit(tm_full(b));
                        if (P.debug & 512u) mbar_arrive(op_empty(s)); else mma_commit(op_empty(s));
                        turn ^= 1u;
                        if (++b == NB) {
                            b = 0;
                            bph ^= 1u;
                            brounds = 1u;
                        }
                        tick(3);
                    } else {
                        // the previous tile's last read of the parked accumulator (all epilogue warps) before its first overwrite
                        if (j == 0 && tile > 0 && !mbar_spin_x(acc_free, (tile - 1u) & 1u, abort_flag, 6u)) goto mma_done;
                        tc_fence_after();
#pragma unroll
                        for (uint32_t kh = 0; kh < 2; kh++)
                            mma_f16(tmem_base + T::acc_col, dt + kh * ((2 * kXT * 16) >> 4), dw + ((kh * 2 * kXN * 16) >> 4), idesc_min,
                                    (j | kh) ? 1u : 0u);
                        mma_commit(op_empty(s));
                        if (j + 1u == n_extra) mma_commit(acc_ready);
                        tick(5);
                    }
                    {
                        // publish the index of this issuer's next own step (past the last tile: none)
                        const bool last_tile = id + gridDim.x >= n_tiles;
                        uint32_t q = p + 1u, nit = it + 1u, tn = turn;
                        for (;;) {
                            if (q == n_steps) {
                                if (last_tile) {
                                    nit = 0xFFFFFFFFu;
                                    break;
                                }
                                q = 0u;
                            }
                            bool m;
                            step_of(q, m);
                            if (m ? me == 0u : tn == me) break;
                            if (!m) tn ^= 1u;
                            q++;
                            nit++;
                        }
                        flag_set(prog_me, nit);
                    }
                }
            }
        mma_done:;
            prof_out(1);
        }
      }
    } else if (warp < kXLead + kXExpW) {
        // ---- expanders: two groups of 128 threads take the K steps in turn; thread r owns weight row m0 + r.
        // Side planes (scales, high bits) come from global memory: requested three of the group's steps early.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 112;" ::: "memory");
        const uint32_t grp = (warp - kXLead) >> 2, r = (threadIdx.x - kXLead * 32u) & 127u;
        struct Side { uint32_t e0, e1, smw, ddw; };
        uint32_t tile_it0 = 0, tile_no = 0;
        for (uint32_t id = blockIdx.x; id < n_tiles && !flag_get(abort_flag); id += gridDim.x, tile_it0 += n_steps, tile_no++) {
            const XTile tl = x_tile(P, id, tiles_t);
            const Planes pl = planes_of<FMT>(P.w, P.in_dim, P.out_dim);
            const uint32_t row = min(tl.m0 + r, P.out_dim - 1u);
            const uint8_t *scp = pl.sc + (size_t)row * pl.nsp * 2u;
            const uint8_t *auxp = (FMT == Q5_K || FMT == Q6_K) ? pl.aux + (size_t)row * pl.nsp * (FMT == Q6_K ? 8u : 4u) : nullptr;
            const uint8_t *supp = T::sup ? pl.sup + (size_t)row * pl.n_super * (FMT == Q6_K ? 2u : 4u) : nullptr;
            auto request = [&](Side &slot, uint32_t p) {
                slot = Side{0u, 0u, 0u, 0u};
                bool req_min;
                const uint32_t i = step_of(p, req_min);
                if (!req_min && i < n_sub && !(P.debug & 64u)) {
                    if constexpr (FMT == Q5_K) slot.e0 = ld_stream_u32(auxp + i * 4u);
                    if constexpr (FMT == Q6_K) {
                        const uint2 h = ld_stream_u2(auxp + i * 8u);
                        slot.e0 = h.x;
                        slot.e1 = h.y;
                    }
                    slot.smw = ld_nc_u16(scp + i * 2u);
                    if constexpr (T::has_min) slot.ddw = ld_nc_u16(supp + (i >> 3) * 4u);
                    if constexpr (FMT == Q6_K) slot.ddw = ld_nc_u16(supp + (i >> 3) * 2u);
                }
            };
            auto step = [&](Side &slot, uint32_t p) -> bool {
                const Side cur = slot;
                request(slot, p + 3u * G);
                const uint32_t it = tile_it0 + p, s = it % S, rs = it % R;
                bool is_min;
                const uint32_t i = step_of(p, is_min);
                tick(0);
                {
                    // both probes in flight together; the slow paths below only run for the one that failed
                    const bool r1 = mbar_test(raw_full(rs), (it / R) & 1u);
                    const bool r2 = it < S || mbar_test(op_empty(s), ((it / S) - 1u) & 1u);
                    if (!r1 && !mbar_wait_x(raw_full(rs), (it / R) & 1u, abort_flag, 7u)) return false;
                    if (!r2 && !mbar_wait_x(op_empty(s), ((it / S) - 1u) & 1u, abort_flag, 8u)) return false;
                }
                tick(1);
                // (with eight operand stages the slot is almost always free already; waiting for it before the
                // expansion lets every expanded chunk go straight to shared memory instead of living in registers)
                tick(3);
                const uint32_t wp = sbase + L::w_off + s * L::w_stage + r * 16u;
                const bool main_step = !is_min;
                if (main_step && !(P.debug & 2u)) { // (a padding step expands the zero bytes of a box past the row; its scale is 0)
                    const uint32_t rp = sbase + L::raw_off + rs * T::raw_bytes + r * 16u;
                    const uint4 q = lds_u4(rp);
                    uint4 q2 = make_uint4(0, 0, 0, 0);
                    if constexpr (FMT == Q8_0) q2 = lds_u4(rp + kXN * 16);
                    uint4 t[2][4];
                    expand_f16<FMT>(q, q2, cur.e0, cur.e1, cur.smw, t); // exact integers: sc * q, q - 8, (q - 32) * sc parts, q, codebook value
#pragma unroll
                    for (uint32_t part = 0; part < T::w_parts; part++) {
#pragma unroll
                        for (int c = 0; c < 4; c++) sts_u4(wp + part * (kXN * 64u) + c * (kXN * 16u), t[part][c]);
                    }
                } else if (T::has_min && !main_step) {
                    // minima step of superblock j: per sub-block the two bf16 pieces of -(dmin * m), laid out
                    // [hi, hi, mid, mid] against the image's [xsum_hi, xsum_mid, xsum_hi, xsum_mid]
                    const uint32_t j = i;
                    const float ndmin = -f16_bits_to_f32(ld_nc_u16(supp + j * 4u + 2u));
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        uint32_t w4[4];
#pragma unroll
                        for (int u = 0; u < 2; u++) {
                            const float v = ndmin * (float)(ld_nc_u16(scp + (j * 8u + 2 * c + u) * 2u) >> 8);
                            const uint32_t hi = bf16_bits(v);
                            const uint32_t mid = bf16_bits(v - bf16_val(hi));
                            w4[2 * u] = hi | (hi << 16);
                            w4[2 * u + 1] = mid | (mid << 16);
                        }
                        sts_u4(wp + c * (kXN * 16u), make_uint4(w4[0], w4[1], w4[2], w4[3]));
                    }
                }
                tick(2);
                bool sup_arrive = false;
                if constexpr (T::sup) {
                    if (main_step && (i & 7u) == 0u) {
                        // the row's f16 d of this superblock, for the epilogue's once-per-superblock step
                        const uint32_t q = (tile_no * n_sup + (i >> 3)) % kSupSlots;
                        sts_f32(sbase + L::dcol_off + q * (kXN * 4u) + r * 4u, tl.m0 + r < P.out_dim ? f16_bits_to_f32(cur.ddw) : 0.0f);
                        sup_arrive = true;
                    }
                } else {
                    if (main_step)
                        sts_f32(sbase + L::dcol_off + (it % kSbSlots) * (kXN * 4u) + r * 4u,
                                tl.m0 + r < P.out_dim ? f16_bits_to_f32(cur.smw) : 0.0f);
                }
                if (!(P.debug & 128u)) asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic writes -> MMA reads
                __syncwarp(); // one arrival per warp
                if (lane == 0) {
                    if (sup_arrive) mbar_arrive(sup_full((tile_no * n_sup + (i >> 3)) % kSupSlots));
                    mbar_arrive(op_full(s));
                    mbar_arrive(raw_empty(rs));
                }
                tick(4);
                return true;
            };
            uint32_t i = (grp + G - (tile_it0 % G)) % G; // the group's first step in this tile
            Side slot0, slot1, slot2;
            request(slot0, i);
            request(slot1, i + G);
            request(slot2, i + 2u * G);
            bool ok = true;
            while (ok && i < n_steps) {
                ok = step(slot0, i);
                i += G;
                if (ok && i < n_steps) {
                    ok = step(slot1, i);
                    i += G;
                }
                if (ok && i < n_steps) {
                    ok = step(slot2, i);
                    i += G;
                }
            }
            if (!ok) break;
        }
        if (r == 0) prof_out(2 + grp);
    } else {
        // ---- epilogue: four warps, one per lane quarter; thread = one token x the tile's 128 weight rows.  The 128
        // columns of a transient tile come in as four 32-column chunks through two register buffers: the load of the
        // next chunk (of the next step, after the last chunk) is in flight while the current one is accumulated.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");
        const uint32_t quarter = warp & 3u;                 // tensor-memory lanes this warp may read
        const uint32_t tlane = quarter * 32u + lane;        // token within the tile
        const uint32_t tm_row = tmem_base + ((quarter * 32u) << 16);
        // sup formats: the running superblock; others: the tile's accumulator.  Plain f32 FMAs: measured on this
        // part, a packed fma.rn.f32x2 occupies the heavy FMA pipe for about four cycles per warp, two scalar FMAs
        // issue back to back on both pipes.
        float inner[128];
#pragma unroll
        for (int k = 0; k < 128; k++) inner[k] = 0.0f;
        uint32_t xa0[16], xa1[16], xb0[16], xb1[16];        // chunk buffers A and B (columns 0..15, 16..31 of a chunk)
        uint32_t sj = 0, tile = 0; // superblocks and tiles done
        uint32_t b = 0, bph = 0;   // transient tile in turn and its phase
        for (uint32_t id = blockIdx.x; id < n_tiles && !flag_get(abort_flag); id += gridDim.x, tile++) {
            // writes 32 finished columns (rows m0 + 32 c ..) of this thread's token; everything it needs is recomputed
            // from the tile id, so that nothing but the id stays live through the K loop
            auto store32 = [&](const uint32_t (&v0)[16], const uint32_t (&v1)[16], uint32_t c) {
                const XTile t = x_tile(P, id, tiles_t);
                const uint32_t rowc = t.m0 + c * 32u;
                if constexpr (!GATHER) {
                    // one output matrix, rows out_dim apart (the instantiation that every plain call runs: the copies
                    // and the transposed stores below cost the steady-state loop registers and time even when unused)
                    if (tlane >= t.n_valid) return;
                    float *dst = P.y[0] + (size_t)(t.tok0 + tlane) * P.out_dim + rowc;
                    if (P.y_vec4 && rowc + 32u <= P.out_dim) {
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            *reinterpret_cast<uint4 *>(dst + 4 * k) = make_uint4(v0[4 * k], v0[4 * k + 1], v0[4 * k + 2], v0[4 * k + 3]);
                            *reinterpret_cast<uint4 *>(dst + 16 + 4 * k) = make_uint4(v1[4 * k], v1[4 * k + 1], v1[4 * k + 2], v1[4 * k + 3]);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 16; k++) {
                            if (rowc + k < P.out_dim) dst[k] = __uint_as_float(v0[k]);
                            if (rowc + 16u + k < P.out_dim) dst[16 + k] = __uint_as_float(v1[k]);
                        }
                    }
                    return;
                }
                if (P.y_vec4 && rowc + 32u <= P.out_dim) {
                    // This GPU's output and its peers' (plain stores over NVLink, issued as the tile finishes while other
                    // tiles compute).  A thread holds 128 contiguous bytes of ITS token, so a warp's store instruction
                    // would touch 32 rows with 16 bytes each: 16-byte packets on the links.  The warp turns the 32 x 32
                    // block through shared memory instead: eight lanes then write the 128 bytes of one token, four
                    // tokens per instruction.
                    const uint32_t xs = sbase + L::xpose_off + quarter * L::xpose_warp;
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        sts_v4(xs + lane * L::xpose_row + 16u * k, v0[4 * k], v0[4 * k + 1], v0[4 * k + 2], v0[4 * k + 3]);
                        sts_v4(xs + lane * L::xpose_row + 64u + 16u * k, v1[4 * k], v1[4 * k + 1], v1[4 * k + 2], v1[4 * k + 3]);
                    }
                    __syncwarp();
                    const uint32_t piece = lane & 7u;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint32_t trow = 4u * j + (lane >> 3), tok = quarter * 32u + trow;
                        uint4 q;
                        lds_v4(xs + trow * L::xpose_row + 16u * piece, q);
                        if (tok < t.n_valid) {
                            const size_t o = (size_t)(t.tok0 + tok) * P.ld_out + P.col_off + rowc + 4u * piece;
                            for (uint32_t g = 0; g < P.n_y; g++) *reinterpret_cast<uint4 *>(P.y[g] + o) = q;
                        }
                    }
                    return;
                }
                if (tlane >= t.n_valid) return;
                const size_t off = (size_t)(t.tok0 + tlane) * P.ld_out + P.col_off + rowc;
                for (uint32_t g = 0; g < P.n_y; g++) {
                    float *dst = P.y[g] + off;
#pragma unroll
                    for (int k = 0; k < 16; k++) {
                        if (rowc + k < P.out_dim) dst[k] = __uint_as_float(v0[k]);
                        if (rowc + 16u + k < P.out_dim) dst[16 + k] = __uint_as_float(v1[k]);
                    }
                }
            };
            for (uint32_t sbk = 0; sbk < n_sup; sbk++, sj++) {
                const uint32_t dxq = sj % kSupSlots; // this superblock's slot of the dx / row-scale rings
                tick(0);
                if (!mbar_wait_x(sup_full(dxq), (sj / kSupSlots) & 1u, abort_flag, 9u)) goto epi_done;
                const uint32_t dxa = sbase + L::dx_off + dxq * (8u * kXT * 4u) + tlane * 4u;
                // non-sup formats: the per-sub-block row scales of step 8 sj + u sit in slot (8 sj + u) % 16
                const uint32_t dsa = sbase + L::dcol_off + ((sj & 1u) * 8u) * (kXN * 4u);
                for (uint32_t u = 0; u < 8; u++) {
                    uint32_t tcol = tm_row + b * kXN;
                    if (u == 0u) { // (later steps: requested at the end of the previous one)
                        tick(0);
                        if (!mbar_wait_x(tm_full(b), bph, abort_flag, 10u)) goto epi_done;
                        tick(1);
                        tc_fence_after();
                        tmem_ld16x(tcol, xa0);
                        tmem_ld16x(tcol + 16u, xa1);
                    }
                    const float dxf = __uint_as_float(lds_u32(dxa + u * (kXT * 4u)));
                    // accumulates chunk c (32 columns) from the two halves x0, x1
                    auto math = [&](const uint32_t (&x0)[16], const uint32_t (&x1)[16], const uint32_t c) {
                        if (P.debug & 1u) return;
                        if constexpr (DUMP) {
                            const uint32_t i = sbk * 8u + u;
                            const XTile t = x_tile(P, id, tiles_t);
                            const uint32_t row0 = t.m0 + c * 32u;
                            if (tlane < t.n_valid && i < n_sub) {
#pragma unroll
                                for (int k = 0; k < 16; k++) {
                                    if (row0 + k < P.out_dim)
                                        P.dump[((size_t)(t.tok0 + tlane) * P.out_dim + row0 + k) * n_sub + i] = __float2int_rn(__uint_as_float(x0[k]));
                                    if (row0 + 16u + k < P.out_dim)
                                        P.dump[((size_t)(t.tok0 + tlane) * P.out_dim + row0 + 16u + k) * n_sub + i] = __float2int_rn(__uint_as_float(x1[k]));
                                }
                            }
                        }
                        if constexpr (T::sup) {
#pragma unroll
                            for (int k = 0; k < 16; k++) inner[32 * c + k] = fmaf(__uint_as_float(x0[k]), dxf, inner[32 * c + k]);
#pragma unroll
                            for (int k = 0; k < 16; k++) inner[32 * c + 16 + k] = fmaf(__uint_as_float(x1[k]), dxf, inner[32 * c + 16 + k]);
                        } else {
                            const uint32_t dsp = dsa + u * (kXN * 4u) + c * 128u;
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                const uint4 dd = lds_u4(dsp + k * 16u); // the scales of columns 4k .. 4k + 3 of the chunk
                                const float dv[4] = {__uint_as_float(dd.x), __uint_as_float(dd.y), __uint_as_float(dd.z), __uint_as_float(dd.w)};
#pragma unroll
                                for (int e = 0; e < 4; e++)
                                    inner[32 * c + 4 * k + e] = fmaf(__uint_as_float(x0[4 * k + e]) * dxf, dv[e], inner[32 * c + 4 * k + e]);
                            }
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                const uint4 dd = lds_u4(dsp + 64u + k * 16u);
                                const float dv[4] = {__uint_as_float(dd.x), __uint_as_float(dd.y), __uint_as_float(dd.z), __uint_as_float(dd.w)};
#pragma unroll
                                for (int e = 0; e < 4; e++)
                                    inner[32 * c + 16 + 4 * k + e] = fmaf(__uint_as_float(x1[4 * k + e]) * dxf, dv[e], inner[32 * c + 16 + 4 * k + e]);
                            }
                        }
                    };
                    tick(2);
                    const bool do_ld = !(P.debug & 8u);
                    tmem_wait_ld(); // chunk 0 in A
                    if (do_ld) {
                        tmem_ld16x(tcol + 32u, xb0);
                        tmem_ld16x(tcol + 48u, xb1);
                    }
                    math(xa0, xa1, 0u);
                    tmem_wait_ld(); // chunk 1 in B
                    if (do_ld) {
                        tmem_ld16x(tcol + 64u, xa0);
                        tmem_ld16x(tcol + 80u, xa1);
                    }
                    math(xb0, xb1, 1u);
                    tmem_wait_ld(); // chunk 2 in A
                    if (do_ld) {
                        tmem_ld16x(tcol + 96u, xb0);
                        tmem_ld16x(tcol + 112u, xb1);
                    }
                    math(xa0, xa1, 2u);
                    tmem_wait_ld(); // chunk 3 in B: every column of the transient tile is in registers
                    tick(3);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tm_empty(b));
                    if (++b == NB) {
                        b = 0;
                        bph ^= 1u;
                    }
                    if (u < 7u) {
                        // the next step's first chunk goes out before this step's last one is accumulated
                        tick(0);
                        if (!mbar_wait_x(tm_full(b), bph, abort_flag, 10u)) goto epi_done;
                        tick(1);
                        tc_fence_after();
                        tcol = tm_row + b * kXN;
                        tmem_ld16x(tcol, xa0);
                        tmem_ld16x(tcol + 16u, xa1);
                    }
                    math(xb0, xb1, 3u);
                    tick(2);
                }
                if constexpr (T::sup) {
                    // superblock end: acc += d[row] * inner; acc is parked in tensor memory between superblocks.
                    // Q4_K / Q5_K: the accumulator already holds the tile's minima term when the first superblock ends
                    const bool first = !T::has_min && sbk == 0u, last = sbk + 1u == n_sup;
                    if constexpr (T::has_min) {
                        if (sbk == 0u) {
                            if (!mbar_wait_x(acc_ready, tile & 1u, abort_flag, 11u)) goto epi_done;
                            tc_fence_after();
                        }
                    }
                    const uint32_t acol = tm_row + T::acc_col;
                    const uint32_t dsp = sbase + L::dcol_off + dxq * (kXN * 4u);
                    // a = inner * d (+ a) for chunk c, inner cleared
                    auto fold = [&](uint32_t (&a0)[16], uint32_t (&a1)[16], const uint32_t c) {
#pragma unroll
                        for (int k = 0; k < 8; k++) {
                            const uint4 dd = lds_u4(dsp + c * 128u + k * 16u); // d of columns 32 c + 4k .. + 3
                            const float dv[4] = {__uint_as_float(dd.x), __uint_as_float(dd.y), __uint_as_float(dd.z), __uint_as_float(dd.w)};
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                uint32_t &a = k < 4 ? a0[4 * k + e] : a1[4 * (k - 4) + e];
                                const float v = inner[32 * c + 4 * k + e];
                                a = __float_as_uint(first ? v * dv[e] : fmaf(v, dv[e], __uint_as_float(a)));
                                inner[32 * c + 4 * k + e] = 0.0f;
                            }
                        }
                    };
                    auto park = [&](const uint32_t (&a0)[16], const uint32_t (&a1)[16], const uint32_t c) {
                        if (!last) {
                            tmem_st16x(acol + c * 32u, a0);
                            tmem_st16x(acol + c * 32u + 16u, a1);
                        } else {
                            store32(a0, a1, c);
                        }
                    };
                    if (!first) {
                        if (sbk > 0u) tmem_wait_st(); // the previous superblock's parking stores (long done)
                        tmem_ld16x(acol, xa0);
                        tmem_ld16x(acol + 16u, xa1);
                        tmem_wait_ld();
                        tmem_ld16x(acol + 32u, xb0);
                        tmem_ld16x(acol + 48u, xb1);
                    }
                    fold(xa0, xa1, 0u);
                    park(xa0, xa1, 0u);
                    if (!first) {
                        tmem_wait_ld();
                        tmem_ld16x(acol + 64u, xa0); // (a store has read its source registers when it issues)
                        tmem_ld16x(acol + 80u, xa1);
                    }
                    fold(xb0, xb1, 1u);
                    park(xb0, xb1, 1u);
                    if (!first) {
                        tmem_wait_ld();
                        tmem_ld16x(acol + 96u, xb0);
                        tmem_ld16x(acol + 112u, xb1);
                    }
                    fold(xa0, xa1, 2u);
                    park(xa0, xa1, 2u);
                    if (!first) tmem_wait_ld();
                    fold(xb0, xb1, 3u);
                    park(xb0, xb1, 3u);
                    // (the parking stores are waited for before the next superblock's loads of the same columns)
                    if (last) {
                      if constexpr (T::has_min) {
                        // this warp's last read of the parked accumulator: the next tile's minima steps may overwrite it
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_free);
                      }
                    }
                    tick(4);
                }
            }
            if constexpr (!T::sup) {
                // tile end: the accumulator is in registers
#pragma unroll
                for (uint32_t c = 0; c < 4; c++) {
                    uint32_t a0[16], a1[16];
#pragma unroll
                    for (int k = 0; k < 16; k++) {
                        a0[k] = __float_as_uint(inner[32 * c + k]);
                        a1[k] = __float_as_uint(inner[32 * c + 16 + k]);
                        inner[32 * c + k] = 0.0f;
                        inner[32 * c + 16 + k] = 0.0f;
                    }
                    store32(a0, a1, c);
                }
            }
        }
    epi_done:;
        if (lane == 0 && warp == kXLead + kXExpW) prof_out(4);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- activations: f32 rows -> the integer f16 operand image -------------------------------------------
//
// One CTA of 32 warps per 8 consecutive tokens (gridDim.y CTAs share the sub-blocks of those tokens).  A
// warp takes one sub-block of all 8 tokens at a time: the BlockQ8 quantizer of quantize_q8_kernel
// (kernels/quantize_q8.cpp:23-54: same sum butterfly, same IEEE divides, same rounding), the quants as
// exact f16 integers transposed through shared memory so that every store instruction writes one chunk
// of the 8 tokens (128 contiguous bytes of the image), d into the dx plane, xsum as two bf16 pieces into
// the minima chunks.  Tokens n_tok .. tok_ld - 1 are written as zeros.
constexpr int kQTokens = 8, kQWarps = 32;

__global__ void __launch_bounds__(kQWarps * 32) activations_to_q16_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                                           uint32_t in_dim, uint32_t n_tok, uint32_t tok_ld)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t n_sub = in_dim >> 5, n_kc = in_dim >> 3, n_sup = (n_sub + 7u) >> 3;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t tok0 = blockIdx.x * kQTokens;
    uint8_t *minima = out + (size_t)n_kc * tok_ld * 16u;
    float *dxp = reinterpret_cast<float *>(minima + (size_t)(4u * n_sup) * tok_ld * 16u);
    __shared__ __align__(16) unsigned short s_tile[kQWarps][kQTokens][32];

    const uint32_t tl = lane >> 2, pair = lane & 3u; // store role: token tl, halves 2*pair, 2*pair + 1 of a chunk
    const float *rows[kQTokens];
#pragma unroll
    for (int t = 0; t < kQTokens; t++) rows[t] = x + (size_t)min(tok0 + t, n_tok - 1u) * in_dim;
    for (uint32_t sb = warp + 32u * blockIdx.y; sb < n_sub; sb += 32u * gridDim.y) {
        float v[kQTokens], sum[kQTokens];
        uint32_t bmax[kQTokens]; // |v| as bits: non-negative floats order like unsigned integers
#pragma unroll
        for (int t = 0; t < kQTokens; t++) {
            v[t] = (tok0 + t < n_tok) ? rows[t][sb * 32u + lane] : 0.0f;
            const float a = fabsf(v[t]);
            bmax[t] = __reduce_max_sync(0xFFFFFFFFu, a == a ? __float_as_uint(a) : 0u); // fmaxf skips a NaN: so does this
            sum[t] = v[t];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int t = 0; t < kQTokens; t++) sum[t] = __fadd_rn(sum[t], __shfl_xor_sync(0xFFFFFFFFu, sum[t], o));
        }
        // the two IEEE divides of a block, once per token: lane t does token t's
        float my_max = 0.0f, my_sum = 0.0f;
#pragma unroll
        for (int t = 0; t < kQTokens; t++) {
            if ((int)(lane & 7u) == t) {
                my_max = __uint_as_float(bmax[t]);
                my_sum = sum[t];
            }
        }
        const float my_d = my_max > 0.0f ? __fdiv_rn(my_max, 127.0f) : 1.0f;
        const float my_inv = my_max > 0.0f ? __fdiv_rn(127.0f, my_max) : 0.0f;
#pragma unroll
        for (int t = 0; t < kQTokens; t++) {
            const float inv = __shfl_sync(0xFFFFFFFFu, my_inv, t);
            int q = __float2int_rn(__fmul_rn(v[t], inv));
            q = max(-127, min(127, q));
            s_tile[warp][t][lane] = __half_as_ushort(__int2half_rn(q));
        }
        __syncwarp();
        if (tok0 + tl < tok_ld) {
#pragma unroll
            for (uint32_t c = 0; c < 4; c++) {
                const uint32_t h2 = *reinterpret_cast<const uint32_t *>(&s_tile[warp][tl][8u * c + 2u * pair]);
                *reinterpret_cast<uint32_t *>(out + ((size_t)(sb * 4u + c) * tok_ld + tok0 + tl) * 16u + pair * 4u) = h2;
            }
        }
        if (lane < kQTokens && tok0 + lane < tok_ld) {
            const bool live = tok0 + lane < n_tok;
            dxp[(size_t)sb * tok_ld + tok0 + lane] = live ? my_d : 0.0f;
            const float xs = live ? my_sum : 0.0f;
            const uint32_t hi = bf16_bits(xs);
            const uint32_t mid = bf16_bits(xs - bf16_val(hi));
            const uint32_t word = hi | (mid << 16);
            // chunk of the sub-block pair (sb / 2), second half of it for an odd sub-block
            *reinterpret_cast<uint2 *>(minima + ((size_t)(sb >> 1) * tok_ld + tok0 + lane) * 16u + (sb & 1u) * 8u) = make_uint2(word, word);
        }
        __syncwarp();
    }
    // minima slots past the last sub-block (a superblock's step reads four whole chunks)
    if (blockIdx.y == 0)
        for (uint32_t i = n_sub * kQTokens + threadIdx.x; i < n_sup * 8u * kQTokens; i += blockDim.x) {
            const uint32_t sb = i / kQTokens, t = i % kQTokens;
            if (tok0 + t < tok_ld)
                *reinterpret_cast<uint2 *>(minima + ((size_t)(sb >> 1) * tok_ld + tok0 + t) * 16u + (sb & 1u) * 8u) = make_uint2(0u, 0u);
        }
}

uint32_t x_tok_ld(uint32_t n_tok) { return (n_tok + 7u) & ~7u; }

int g_x_prof = 0, g_x_debug = 0;

template <int FMT, bool DUMP>
int launch_x(cudaStream_t s, const XParams &P, const void *image)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return RC_ERR_NO_DEVICE;
    CUtensorMap wmap, tokmap, dxmap;
    int rc = make_tmap<FMT>(&wmap, P.w, 0, 1u, P.in_dim, P.out_dim);
    if (rc) return rc;
    const uint32_t n_sub = P.in_dim >> 5, n_sup = (n_sub + 7u) >> 3;
    const uint64_t n_chunks = (uint64_t)(P.in_dim >> 3) + 4u * n_sup;
    {
        // 2-D view of the image in 8-byte elements: (position in a chunk row = 2 per token, chunk).  The 128 tokens of
        // a tile are 2 KB contiguous within a chunk, so a K = 32 step is a box of four 2 KB rows: four requests to the
        // TMA unit (described as 16 bytes x token x chunk it is 512, and the unit, not the SM, bounds the kernel)
        const cuuint64_t dims[2] = {(cuuint64_t)P.tok_ld * 2u, n_chunks};
        const cuuint64_t strides[1] = {(cuuint64_t)P.tok_ld * 16u};
        const cuuint32_t box[2] = {kXT * 2u, 4};
        const cuuint32_t estr[2] = {1, 1};
        if (fn(&tokmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 2, const_cast<void *>(image), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return RC_ERR_BAD_ARGUMENT;
    }
    {
        // dx plane: (token, sub-block) f32; one box = a superblock of a token tile
        const uint8_t *dx = (const uint8_t *)image + n_chunks * P.tok_ld * 16u;
        const cuuint64_t dims[2] = {P.tok_ld, n_sub};
        const cuuint64_t strides[1] = {(cuuint64_t)P.tok_ld * 4u};
        const cuuint32_t box[2] = {kXT, 8};
        const cuuint32_t estr[2] = {1, 1};
        if (fn(&dxmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<uint8_t *>(dx), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return RC_ERR_BAD_ARGUMENT;
    }
    const uint32_t tiles = ((P.out_dim + kXN - 1) / kXN) * ((P.n_tok + kXT - 1) / kXT);
    const uint32_t grid = std::min(tiles, (uint32_t)sm_count());
    if constexpr (!DUMP && (FMT == Q4_K || FMT == Q8_0)) {
        if (g_x_prof)
            return (int)launch_pdl(mmqx_kernel<FMT, false, true>, dim3(grid), dim3(kXThreads), SmemX<FMT>::total, s, wmap, tokmap, dxmap, P);
    }
    if (!DUMP && (P.n_y > 1u || P.ld_out != P.out_dim || P.col_off != 0u))
        return (int)launch_pdl(mmqx_kernel<FMT, false, false, true>, dim3(grid), dim3(kXThreads), SmemX<FMT>::total_gather, s, wmap, tokmap, dxmap, P);
    return (int)launch_pdl(mmqx_kernel<FMT, DUMP>, dim3(grid), dim3(kXThreads), SmemX<FMT>::total, s, wmap, tokmap, dxmap, P);
}

template <int FMT> int set_attr_x()
{
    int rc = (int)cudaFuncSetAttribute(mmqx_kernel<FMT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SmemX<FMT>::total);
    rc |= (int)cudaFuncSetAttribute(mmqx_kernel<FMT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SmemX<FMT>::total);
    rc |= (int)cudaFuncSetAttribute(mmqx_kernel<FMT, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SmemX<FMT>::total_gather);
    if constexpr (FMT == Q4_K || FMT == Q8_0)
        rc |= (int)cudaFuncSetAttribute(mmqx_kernel<FMT, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SmemX<FMT>::total);
    return rc;
}

template <bool DUMP>
int launch_x_type(cudaStream_t s, int type, const XParams &P, const void *image)
{
    switch (type) {
    case Q4_0: return launch_x<Q4_0, DUMP>(s, P, image);
    case Q8_0: return launch_x<Q8_0, DUMP>(s, P, image);
    case Q4_K: return launch_x<Q4_K, DUMP>(s, P, image);
    case Q5_K: return launch_x<Q5_K, DUMP>(s, P, image);
    case Q6_K: return launch_x<Q6_K, DUMP>(s, P, image);
    case IQ4_XS: return launch_x<IQ4_XS, DUMP>(s, P, image);
    case IQ3_S: return launch_x<IQ3_S, DUMP>(s, P, image);
    }
    return RC_ERR_BAD_TYPE;
}

} // namespace

int mmq_x_set_attributes()
{
    return set_attr_x<Q4_0>() | set_attr_x<Q8_0>() | set_attr_x<Q4_K>() | set_attr_x<Q5_K>() | set_attr_x<Q6_K>() | set_attr_x<IQ4_XS>() |
           set_attr_x<IQ3_S>();
}

void mmq_x_set_prof(int on) { g_x_prof = on; }
void mmq_x_set_debug(int mask) { g_x_debug = mask; }
int mmq_x_read_prof(void *out, size_t bytes)
{
    return (int)cudaMemcpyFromSymbol(out, g_mmqx_prof, bytes < sizeof(g_mmqx_prof) ? bytes : sizeof(g_mmqx_prof));
}

bool mmq_x_supports(int type) { return type == Q4_0 || type == Q8_0 || type == Q4_K || type == Q5_K || type == Q6_K || type == IQ4_XS || type == IQ3_S; }

int mmq_x_device_error(unsigned int *out, bool clear)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, g_mmqx_error, sizeof(unsigned int));
    if (e == cudaSuccess && clear && *out) {
        const unsigned int zero = 0;
        e = cudaMemcpyToSymbol(g_mmqx_error, &zero, sizeof(unsigned int));
    }
    return (int)e;
}

// image chunks (main + minima), then the dx plane
size_t mmq_x_scratch_bytes(uint32_t in_dim, uint32_t n_tok)
{
    const size_t ld = x_tok_ld(n_tok), n_sub = in_dim >> 5, n_sup = (n_sub + 7u) >> 3;
    return ((size_t)(in_dim >> 3) + 4u * n_sup) * ld * 16u + n_sub * ld * sizeof(float);
}

// x f32 [n_tok][in_dim] -> y f32 [n_tok][out_dim]; scratch 16-byte aligned, mmq_x_scratch_bytes large.
// dump != nullptr: also the integer tiles, int32 [n_tok][out_dim][in_dim / 32].
int launch_mmq_x_f32(cudaStream_t s, int type, const void *w, const float *x, float *y, uint32_t in_dim, uint32_t out_dim,
                     uint32_t n_tok, void *scratch, int32_t *dump, float *const *y_peers, uint32_t n_peers, uint32_t ld_out,
                     uint32_t col_off)
{
    const uint32_t ld = x_tok_ld(n_tok);
    // 8 tokens per CTA; a second CTA shares their sub-blocks while that still adds SMs
    const uint32_t groups = ld / kQTokens, ysplit = groups * 2u <= (uint32_t)sm_count() ? 2u : 1u;
    cudaError_t e = launch_pdl(activations_to_q16_kernel, dim3(groups, ysplit), dim3(kQWarps * 32), 0, s, x, (uint8_t *)scratch, in_dim,
                               n_tok, ld);
    if (e != cudaSuccess) return (int)e;
    XParams P;
    P.w = (const uint8_t *)w;
    bool aligned = true;
    for (uint32_t g = 0; g < RC_MAX_PEERS; g++) P.y[g] = nullptr;
    if (y_peers) {
        P.n_y = n_peers;
        P.ld_out = ld_out;
        P.col_off = col_off;
        for (uint32_t g = 0; g < n_peers; g++) {
            P.y[g] = y_peers[g];
            aligned = aligned && ((uintptr_t)y_peers[g] & 15u) == 0;
        }
        aligned = aligned && (ld_out & 3u) == 0 && (col_off & 3u) == 0;
    } else {
        P.n_y = 1;
        P.ld_out = out_dim;
        P.col_off = 0;
        P.y[0] = y;
        aligned = ((uintptr_t)y & 15u) == 0 && (out_dim & 3u) == 0;
    }
    P.dump = dump;
    P.in_dim = in_dim;
    P.out_dim = out_dim;
    P.n_tok = n_tok;
    P.tok_ld = ld;
    P.y_vec4 = aligned ? 1u : 0u;
    P.debug = (uint32_t)g_x_debug;
    return dump ? launch_x_type<true>(s, type, P, scratch) : launch_x_type<false>(s, type, P, scratch);
}

} // namespace rc
