// All-gather of small row shards by direct stores into peer memory (NVLink), with a counter
// handshake instead of a library collective.  See include/reinstinct_cuda.h for the contract.
#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {
namespace {

constexpr unsigned long long kGatherWaitNs = 200ull * 1000 * 1000;

__device__ unsigned int g_gather_error;

struct GatherPeers {
    uint4 *dst[RC_MAX_PEERS];
    unsigned long long *flags[RC_MAX_PEERS];
};

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v)
{
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long gather_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// The work of one rank, by one CTA: store the shard into every rank's gathered buffer (shard i of a buffer
// belongs to rank i), publish this call's epoch in every rank's flag array, wait (bounded) for every rank's.
__device__ __forceinline__ void gather_body(const uint4 *__restrict__ src, uint32_t n16, const GatherPeers &peers,
                                            unsigned long long *epoch_ctr, uint32_t rank, uint32_t world)
{
    for (uint32_t r = 0; r < world; r++) {
        uint4 *dst = peers.dst[r] + (size_t)rank * n16;
        for (uint32_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    __shared__ unsigned long long s_epoch;
    if (threadIdx.x == 0) {
        const unsigned long long e = *epoch_ctr + 1ull;
        *epoch_ctr = e;
        s_epoch = e;
        for (uint32_t r = 0; r < world; r++) st_release_sys(peers.flags[r] + rank, e);
    }
    __syncthreads();
    if (threadIdx.x < world) {
        const unsigned long long e = s_epoch;
        const unsigned long long *mine = peers.flags[rank] + threadIdx.x;
        const unsigned long long t0 = gather_ns();
        while (ld_acquire_sys(mine) < e) {
            if (gather_ns() - t0 > kGatherWaitNs) { // a peer never arrived: record it and let the kernel end
                atomicExch(&g_gather_error, 1u);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(512)
allgather_push_kernel(const uint4 *__restrict__ src, uint32_t n16, GatherPeers peers,
                      unsigned long long *epoch_ctr, uint32_t rank, uint32_t world)
{
    pdl_launch_dependents(); // the consumer may start fetching its weights during the handshake
    pdl_wait();              // the shard comes from the preceding kernel; a peer's stores into this rank's
                             // memory (a fused producer) are complete when its own handshake kernel starts
    gather_body(src, n16, peers, epoch_ctr, rank, world);
}

// `world` logical ranks on ONE device, one CTA each, launched cooperatively so that they are co-resident
// (separate launches that wait on one another are not guaranteed to run at the same time).
struct LogicalRanks {
    const uint4 *src[RC_MAX_PEERS];
    unsigned long long *epoch[RC_MAX_PEERS];
};
__global__ void __launch_bounds__(512)
allgather_push_logical_kernel(LogicalRanks ranks, uint32_t n16, GatherPeers peers, uint32_t world)
{
    gather_body(ranks.src[blockIdx.x], n16, peers, ranks.epoch[blockIdx.x], blockIdx.x, world);
}

} // namespace

int gather_device_error(unsigned int *out, bool clear)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, g_gather_error, sizeof(unsigned int));
    if (e == cudaSuccess && clear && *out) {
        const unsigned int zero = 0;
        e = cudaMemcpyToSymbol(g_gather_error, &zero, sizeof(unsigned int));
    }
    return (int)e;
}

int launch_allgather_push(cudaStream_t s, const void *src, size_t bytes, void *const *peer_dst,
                          void *const *peer_flags, void *epoch, uint32_t rank, uint32_t world)
{
    GatherPeers p;
    for (uint32_t r = 0; r < RC_MAX_PEERS; r++) {
        p.dst[r] = r < world ? static_cast<uint4 *>(peer_dst[r]) : nullptr;
        p.flags[r] = r < world ? static_cast<unsigned long long *>(peer_flags[r]) : nullptr;
    }
    if (!matvec_pdl_enabled()) {
        allgather_push_kernel<<<1, 512, 0, s>>>(static_cast<const uint4 *>(src), (uint32_t)(bytes / 16), p,
                                                static_cast<unsigned long long *>(epoch), rank, world);
        return (int)cudaGetLastError();
    }
    return (int)launch_pdl(allgather_push_kernel, dim3(1), dim3(512), 0, s, static_cast<const uint4 *>(src),
                           (uint32_t)(bytes / 16), p, static_cast<unsigned long long *>(epoch), rank, world);
}

int launch_allgather_push_logical(cudaStream_t s, const void *const *srcs, size_t bytes, void *const *dsts, void *const *flags,
                                  void *const *epochs, uint32_t world)
{
    GatherPeers p;
    LogicalRanks lr;
    for (uint32_t r = 0; r < RC_MAX_PEERS; r++) {
        p.dst[r] = r < world ? static_cast<uint4 *>(dsts[r]) : nullptr;
        p.flags[r] = r < world ? static_cast<unsigned long long *>(flags[r]) : nullptr;
        lr.src[r] = r < world ? static_cast<const uint4 *>(srcs[r]) : nullptr;
        lr.epoch[r] = r < world ? static_cast<unsigned long long *>(epochs[r]) : nullptr;
    }
    uint32_t n16 = (uint32_t)(bytes / 16);
    void *args[] = {&lr, &n16, &p, &world};
    return (int)cudaLaunchCooperativeKernel((const void *)allgather_push_logical_kernel, dim3(world), dim3(512), args, 0, s);
}

} // namespace rc
