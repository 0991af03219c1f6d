// int8 MMQ GEMM entry points (dense and expert-grouped).
#include "rc_common.cuh"
#include "rc_internal.h"

namespace rc {

uint32_t mmq_grouped_bn() { return 16; }
int mmq_set_attributes() { return RC_OK; }

int launch_mmq_gemm(cudaStream_t s, int type, const void *w, const void *xq, float *y,
                    uint32_t in_dim, uint32_t out_dim, uint32_t p_rows)
{
    const uint32_t n_sub = in_dim >> 5;
    for (uint32_t p0 = 0; p0 < p_rows; p0 += 16) {
        const uint32_t n = min(16u, p_rows - p0);
        int rc = launch_matvec(s, type, w, (const uint8_t *)xq + (size_t)p0 * n_sub * RC_BLOCKQ8_BYTES,
                               y + (size_t)p0 * out_dim, in_dim, out_dim, n, nullptr);
        if (rc) return rc;
    }
    return RC_OK;
}

int launch_mmq_grouped(cudaStream_t s, int type, const void *slab, size_t bytes_per_expert,
                       const int32_t *expert_off, const int32_t *tile_off, uint32_t n_expert,
                       const void *xq, float *y, uint32_t in_dim, uint32_t out_dim,
                       uint32_t n_entries)
{
    return launch_matvec_grouped(s, type, slab, bytes_per_expert, expert_off, tile_off, n_expert,
                                 xq, y, in_dim, out_dim, n_entries);
}

} // namespace rc
