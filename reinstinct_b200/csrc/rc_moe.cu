// MoE expert routing sort, BlockQ8 row gather and f32 row scatter.
//
// Outputs are those of the reference's five-launch pipeline moe_sort_{zero,histogram,scan,
// zero,scatter} (kernels/moe_expert_sort.cpp:27-76): count[e], expert_off[e] (exclusive
// prefix of count, n_expert+1 entries), tile_off[e] (exclusive prefix of ceil(count/bn)) and
// perm (entry indices grouped by expert).  Here it is ONE launch of one CTA: the routing
// table is a few thousand ints, so the cost is launch latency and a single CTA with a
// shared-memory histogram removes four launches and every global atomic.  The scatter is a
// stable counting sort (ascending entry index inside an expert), which the reference
// leaves unspecified (its global atomic cursors, moe_expert_sort.cpp:73) — deterministic
// output makes runs reproducible and multi-GPU results comparable.
#include <algorithm>

#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {
namespace {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;

// Exclusive scan of one int per thread across the CTA; returns the exclusive prefix and
// leaves the grand total in *total.  scratch: kSortWarps + 1 ints of shared memory.
__device__ __forceinline__ int block_exclusive_scan(int v, int *scratch, int *total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int k = 0; k < kSortWarps; k++) {
            const int t = scratch[k];
            scratch[k] = run;
            run += t;
        }
        scratch[kSortWarps] = run;
    }
    __syncthreads();
    const int res = scratch[warp] + inc - v;
    *total = scratch[kSortWarps];
    __syncthreads();
    return res;
}

// smem: cnt[n_expert] | base[n_expert] | wcnt[kSortWarps][n_expert] | scan scratch
__global__ void __launch_bounds__(kSortThreads)
moe_sort_kernel(const int32_t *__restrict__ ids, uint32_t n_entries, uint32_t n_expert,
                uint32_t bn, int32_t *__restrict__ count, int32_t *__restrict__ cursor,
                int32_t *__restrict__ expert_off, int32_t *__restrict__ tile_off,
                int32_t *__restrict__ perm)
{
    extern __shared__ int sm[];
    int *cnt = sm;
    int *base = cnt + n_expert;
    int *wcnt = base + n_expert;
    int *scratch = wcnt + (size_t)kSortWarps * n_expert;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;

    for (uint32_t e = tid; e < n_expert; e += kSortThreads) cnt[e] = 0;
    __syncthreads();
    for (uint32_t i = tid; i < n_entries; i += kSortThreads) {
        const int e = ids[i];
        if (e >= 0 && (uint32_t)e < n_expert) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();

    // Prefix sums over experts; each thread owns a contiguous run of experts.
    const uint32_t per = (n_expert + kSortThreads - 1) / kSortThreads;
    const uint32_t e0 = min(tid * per, n_expert), e1 = min(e0 + per, n_expert);
    int my_cnt = 0, my_tiles = 0;
    for (uint32_t e = e0; e < e1; e++) {
        my_cnt += cnt[e];
        my_tiles += (int)(((uint32_t)cnt[e] + bn - 1u) / bn);
    }
    int total_cnt, total_tiles;
    int run_cnt = block_exclusive_scan(my_cnt, scratch, &total_cnt);
    int run_tiles = block_exclusive_scan(my_tiles, scratch, &total_tiles);
    for (uint32_t e = e0; e < e1; e++) {
        const int c = cnt[e];
        count[e] = c;
        cursor[e] = c; // the reference's cursors end equal to the counts
        expert_off[e] = run_cnt;
        tile_off[e] = run_tiles;
        base[e] = run_cnt;
        run_cnt += c;
        run_tiles += (int)(((uint32_t)c + bn - 1u) / bn);
    }
    if (tid == 0) {
        expert_off[n_expert] = total_cnt;
        tile_off[n_expert] = total_tiles;
    }
    // Slots past the routed total (only present when ids held out-of-range values).
    for (uint32_t p = (uint32_t)total_cnt + tid; p < n_entries; p += kSortThreads) perm[p] = -1;
    __syncthreads();

    // Stable scatter, one tile of kSortThreads entries at a time.
    for (uint32_t t0 = 0; t0 < n_entries; t0 += kSortThreads) {
        for (uint32_t k = tid; k < kSortWarps * n_expert; k += kSortThreads) wcnt[k] = 0;
        __syncthreads();
        const uint32_t i = t0 + tid;
        int e = -1;
        if (i < n_entries) {
            e = ids[i];
            if (e < 0 || (uint32_t)e >= n_expert) e = -1;
        }
        const uint32_t peers = __match_any_sync(0xFFFFFFFFu, e);
        const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
        if (e >= 0 && rank_in_warp == 0) wcnt[warp * n_expert + e] = __popc(peers);
        __syncthreads();
        if (e >= 0) {
            int before = 0;
            for (uint32_t wv = 0; wv < warp; wv++) before += wcnt[wv * n_expert + e];
            perm[base[e] + before + rank_in_warp] = (int32_t)i;
        }
        __syncthreads();
        for (uint32_t ex = tid; ex < n_expert; ex += kSortThreads) {
            int add = 0;
            for (int wv = 0; wv < kSortWarps; wv++) add += wcnt[wv * n_expert + ex];
            base[ex] += add;
        }
        __syncthreads();
    }
}

// xq_dst[p] = xq_src[perm[p] / n_used], rows of n_sub 40-byte blocks moved as 8-byte words.
__global__ void __launch_bounds__(256)
moe_gather_xq_kernel(const uint2 *__restrict__ src, const int32_t *__restrict__ perm,
                     uint2 *__restrict__ dst, uint32_t words_per_row, uint32_t n_used,
                     uint32_t n_entries)
{
    const size_t total = (size_t)n_entries * words_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t p = (uint32_t)(i / words_per_row), c = (uint32_t)(i % words_per_row);
        const int entry = perm[p];
        if (entry < 0) continue;
        dst[i] = __ldg(src + (size_t)((uint32_t)entry / n_used) * words_per_row + c);
    }
}

// dst[perm[p]] = src[p]
template <typename T>
__global__ void __launch_bounds__(256)
moe_scatter_rows_kernel(const T *__restrict__ src, const int32_t *__restrict__ perm,
                        T *__restrict__ dst, uint32_t vec_per_row, uint32_t n_entries)
{
    const size_t total = (size_t)n_entries * vec_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t p = (uint32_t)(i / vec_per_row), c = (uint32_t)(i % vec_per_row);
        const int entry = perm[p];
        if (entry < 0) continue;
        dst[(size_t)entry * vec_per_row + c] = src[i];
    }
}

uint32_t grid_for(size_t total)
{
    return (uint32_t)std::max<size_t>(1, std::min<size_t>((total + 255) / 256, (size_t)sm_count() * 16));
}

} // namespace

int launch_moe_sort(cudaStream_t s, const int32_t *ids, uint32_t n_entries, uint32_t n_expert,
                    uint32_t bn, int32_t *count, int32_t *cursor, int32_t *expert_off,
                    int32_t *tile_off, int32_t *perm)
{
    const size_t smem = ((size_t)(2 + kSortWarps) * n_expert + kSortWarps + 1) * sizeof(int);
    if (smem > 200 * 1024) return RC_ERR_BAD_ARGUMENT;
    moe_sort_kernel<<<1, kSortThreads, smem, s>>>(ids, n_entries, n_expert, bn, count, cursor,
                                                  expert_off, tile_off, perm);
    return (int)cudaGetLastError();
}

int moe_set_attributes()
{
    return (int)cudaFuncSetAttribute(moe_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     200 * 1024);
}

int launch_moe_gather_xq(cudaStream_t s, const void *xq_src, const int32_t *perm, void *xq_dst,
                         uint32_t n_sub, uint32_t n_used, uint32_t n_entries)
{
    const uint32_t words = n_sub * (RC_BLOCKQ8_BYTES / 8);
    const size_t total = (size_t)n_entries * words;
    if (!total) return RC_OK;
    moe_gather_xq_kernel<<<grid_for(total), 256, 0, s>>>((const uint2 *)xq_src, perm, (uint2 *)xq_dst,
                                                         words, n_used, n_entries);
    return (int)cudaGetLastError();
}

int launch_moe_scatter_rows(cudaStream_t s, const float *src, const int32_t *perm, float *dst,
                            uint32_t dim, uint32_t n_entries)
{
    if (!dim || !n_entries) return RC_OK;
    const bool v4 = dim % 4 == 0 && ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0);
    if (v4) {
        const size_t total = (size_t)n_entries * (dim / 4);
        moe_scatter_rows_kernel<float4><<<grid_for(total), 256, 0, s>>>(
            (const float4 *)src, perm, (float4 *)dst, dim / 4, n_entries);
    } else {
        const size_t total = (size_t)n_entries * dim;
        moe_scatter_rows_kernel<float><<<grid_for(total), 256, 0, s>>>(src, perm, dst, dim, n_entries);
    }
    return (int)cudaGetLastError();
}

} // namespace rc
