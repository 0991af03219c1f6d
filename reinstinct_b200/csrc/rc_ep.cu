// Expert parallelism without the host: routed activation rows go to the GPU that owns their expert, and the results
// come back, by plain stores into peer memory (NVLink, CUDA IPC mappings).  Shapes are static (every (source, owner) pair
// has `cap` slots; unused slots carry expert id -1, which the sort, gather and scatter kernels skip), so the whole
// layer — route, exchange, grouped GEMM, exchange back — is a fixed sequence of launches that a CUDA graph can hold.
// The reference has no expert parallelism (it pipelines layers over hipMemcpyPeerAsync, src/runtime/qwen35.rs); the
// grouped GEMM between the two exchanges is its launch_moe_grouped_gemm (src/runtime/qwen35.rs:3036).
// See include/reinstinct_cuda.h for the contract of each entry point.
#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {
namespace {

constexpr int kPlanThreads = 1024;

struct EpPeers {
    uint2 *rows[RC_MAX_PEERS];    // rank r's receive buffer of BlockQ8 rows: [2][world * cap][words]
    int32_t *ids[RC_MAX_PEERS];   // rank r's received local expert ids:      [2][world * cap]
};
struct EpRetPeers {
    float4 *ret[RC_MAX_PEERS];    // rank r's returned result rows: [world * cap][dim / 4]
};

// back[e] = owner * cap + (number of earlier entries of this rank with the same owner), or -1 for a dropped entry
// (id < 0 or beyond the experts).  One CTA, entries in order: the placement is a function of the ids alone.
__global__ void __launch_bounds__(kPlanThreads) ep_plan_kernel(const int32_t *__restrict__ ids, uint32_t n_entries,
                                                               uint32_t experts_per_rank, uint32_t cap, uint32_t world,
                                                               int32_t *__restrict__ back)
{
    __shared__ int s_warp[kPlanThreads / 32];
    __shared__ int s_run[RC_MAX_PEERS];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    if (tid < RC_MAX_PEERS) s_run[tid] = 0;
    __syncthreads();
    for (uint32_t base = 0; base < n_entries; base += kPlanThreads) {
        const uint32_t e = base + tid;
        int owner = -1;
        if (e < n_entries) {
            const int id = ids[e];
            if (id >= 0 && (uint32_t)id / experts_per_rank < world) owner = (int)((uint32_t)id / experts_per_rank);
        }
        int slot = -1;
        for (uint32_t o = 0; o < world; o++) { // at most eight rounds of a block-wide count
            const bool mine = owner == (int)o;
            const uint32_t m = __ballot_sync(0xFFFFFFFFu, mine);
            if (lane == 0) s_warp[warp] = __popc(m);
            __syncthreads();
            int before = s_run[o];
            for (uint32_t w = 0; w < warp; w++) before += s_warp[w];
            if (mine) slot = before + __popc(m & ((1u << lane) - 1u));
            __syncthreads();
            if (tid == 0) {
                int total = 0;
                for (int w = 0; w < kPlanThreads / 32; w++) total += s_warp[w];
                s_run[o] += total;
            }
            __syncthreads();
        }
        if (e < n_entries) back[e] = (owner >= 0 && (uint32_t)slot < cap) ? (int32_t)((uint32_t)owner * cap + (uint32_t)slot) : -1;
    }
}

// One warp per entry: the token's BlockQ8 row and the expert's index at its owner go into the owner's slot
// (source rank, slot).  The kernel also marks every slot of THIS rank's other receive buffer as unused: that buffer is
// written by the peers in the next step, after a barrier this rank arrives at only when this kernel has finished.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const int32_t *__restrict__ ids, const int32_t *__restrict__ back,
                                                          const uint2 *__restrict__ xq, uint32_t n_entries, uint32_t n_used,
                                                          uint32_t words, uint32_t experts_per_rank, uint32_t cap, uint32_t rank,
                                                          uint32_t world, uint32_t buf, const EpPeers peers)
{
    const uint32_t lane = threadIdx.x & 31u, warps = (gridDim.x * blockDim.x) >> 5, gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t slots = (size_t)world * cap;
    int32_t *other = peers.ids[rank] + (size_t)(buf ^ 1u) * slots;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < slots; i += (size_t)gridDim.x * blockDim.x) other[i] = -1;
    for (uint32_t e = gwarp; e < n_entries; e += warps) {
        const int b = back[e];
        if (b < 0) continue;
        const uint32_t owner = (uint32_t)b / cap, slot = (uint32_t)b % cap;
        const size_t at = (size_t)buf * slots + (size_t)rank * cap + slot;
        const uint2 *src = xq + (size_t)(e / n_used) * words;
        uint2 *dst = peers.rows[owner] + at * words;
        for (uint32_t w = lane; w < words; w += 32u) dst[w] = src[w];
        if (lane == 0) peers.ids[owner][at] = ids[e] - (int32_t)(owner * experts_per_rank);
    }
}

// One warp per received slot: the finished row goes back to its source, at (this rank, slot) of the source's buffer.
__global__ void __launch_bounds__(256) ep_return_kernel(const int32_t *__restrict__ ids_in, const float4 *__restrict__ y_in, uint32_t vec,
                                                        uint32_t cap, uint32_t rank, uint32_t world, const EpRetPeers peers)
{
    const uint32_t lane = threadIdx.x & 31u, warps = (gridDim.x * blockDim.x) >> 5, gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t slots = world * cap;
    for (uint32_t i = gwarp; i < slots; i += warps) {
        if (ids_in[i] < 0) continue;
        const uint32_t src_rank = i / cap, slot = i % cap;
        const float4 *src = y_in + (size_t)i * vec;
        float4 *dst = peers.ret[src_rank] + ((size_t)rank * cap + slot) * vec;
        for (uint32_t v = lane; v < vec; v += 32u) dst[v] = src[v];
    }
}

// One warp per entry: out[e] = the row that came back for it (zeros for a dropped entry).
__global__ void __launch_bounds__(256) ep_collect_kernel(const int32_t *__restrict__ back, const float4 *__restrict__ ret, float4 *__restrict__ out,
                                                         uint32_t vec, uint32_t n_entries)
{
    const uint32_t lane = threadIdx.x & 31u, warps = (gridDim.x * blockDim.x) >> 5, gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    for (uint32_t e = gwarp; e < n_entries; e += warps) {
        const int b = back[e];
        float4 *dst = out + (size_t)e * vec;
        if (b < 0) {
            for (uint32_t v = lane; v < vec; v += 32u) dst[v] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            continue;
        }
        // written by a peer during this step: not through the non-coherent path
        const float4 *src = ret + (size_t)b * vec;
        for (uint32_t v = lane; v < vec; v += 32u) dst[v] = __ldcg(src + v);
    }
}

uint32_t warp_grid(size_t n_warps)
{
    return (uint32_t)std::max<size_t>(1, std::min<size_t>((n_warps + 7) / 8, (size_t)sm_count() * 8));
}

} // namespace

int launch_ep_plan(cudaStream_t s, const int32_t *ids, uint32_t n_entries, uint32_t experts_per_rank, uint32_t cap, uint32_t world,
                   int32_t *back)
{
    ep_plan_kernel<<<1, kPlanThreads, 0, s>>>(ids, n_entries, experts_per_rank, cap, world, back);
    return (int)cudaGetLastError();
}

int launch_ep_dispatch(cudaStream_t s, const int32_t *ids, const int32_t *back, const void *xq, uint32_t n_entries, uint32_t n_used,
                       uint32_t n_sub, uint32_t experts_per_rank, uint32_t cap, uint32_t rank, uint32_t world, uint32_t buf,
                       void *const *rows_peers, void *const *ids_peers)
{
    EpPeers peers;
    for (uint32_t r = 0; r < RC_MAX_PEERS; r++) {
        peers.rows[r] = r < world ? (uint2 *)rows_peers[r] : nullptr;
        peers.ids[r] = r < world ? (int32_t *)ids_peers[r] : nullptr;
    }
    const size_t work = std::max<size_t>(n_entries, ((size_t)world * cap + 31) / 32);
    ep_dispatch_kernel<<<warp_grid(work), 256, 0, s>>>(ids, back, (const uint2 *)xq, n_entries, n_used, n_sub * (RC_BLOCKQ8_BYTES / 8),
                                                      experts_per_rank, cap, rank, world, buf & 1u, peers);
    return (int)cudaGetLastError();
}

int launch_ep_return(cudaStream_t s, const int32_t *ids_in, const float *y_in, uint32_t dim, uint32_t cap, uint32_t rank, uint32_t world,
                     void *const *ret_peers)
{
    EpRetPeers peers;
    for (uint32_t r = 0; r < RC_MAX_PEERS; r++) peers.ret[r] = r < world ? (float4 *)ret_peers[r] : nullptr;
    ep_return_kernel<<<warp_grid((size_t)world * cap), 256, 0, s>>>(ids_in, (const float4 *)y_in, dim / 4, cap, rank, world, peers);
    return (int)cudaGetLastError();
}

int launch_ep_collect(cudaStream_t s, const int32_t *back, const float *ret, float *out, uint32_t dim, uint32_t n_entries)
{
    if (!n_entries) return RC_OK;
    ep_collect_kernel<<<warp_grid(n_entries), 256, 0, s>>>(back, (const float4 *)ret, (float4 *)out, dim / 4, n_entries);
    return (int)cudaGetLastError();
}

} // namespace rc
