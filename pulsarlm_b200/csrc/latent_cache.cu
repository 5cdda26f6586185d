// Rows RMS-normed and stored into a paged cache: what a mixer that caches one low-rank
// latent per token (instead of keys and values per head) writes each step.
//
//   c[t] = z[t] * rsqrt(mean(z[t]^2) + eps) * weight          fp32, one rounding on store
//   pool[table[entry[t]][pos[t] / page], pos[t] % page] = c[t]
//
// One warp per token; the sum of squares is added in an order fixed by the rank.
#include "common.cuh"

namespace {

template <typename scalar_t>
__global__ void norm_write_paged_kernel(const scalar_t* __restrict__ z, int64_t row_stride,
                                        const float* __restrict__ weight, float eps,
                                        const int32_t* __restrict__ pos, const int32_t* __restrict__ entry,
                                        const int32_t* __restrict__ table, int table_width,
                                        scalar_t* __restrict__ pool, int64_t page_stride, int page_size, int n_pages,
                                        int rank, int n_tokens, int32_t* status) {
    pl_grid_trigger();
    pl_grid_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n_tokens) {
        return;
    }
    const scalar_t* row = z + t * row_stride;
    float square = 0.0f;
    for (int d = lane; d < rank; d += 32) {
        const float value = pl_load(row + d);
        square += value * value;
    }
    const float inv = 1.0f / sqrtf(pl_warp_sum(square) / static_cast<float>(rank) + eps);
    const int p = pos[t];
    const int page = table[static_cast<int64_t>(entry[t]) * table_width + p / page_size];
    if (page < 0 || page >= n_pages) {
        if (lane == 0 && status != nullptr) {
            atomicOr(status, 2);
        }
        return;
    }
    scalar_t* dst = pool + page * page_stride + static_cast<int64_t>(p % page_size) * rank;
    for (int d = lane; d < rank; d += 32) {
        pl_store(dst + d, pl_load(row + d) * inv * weight[d]);
    }
}

}  // namespace

// z [T, rank] with row_stride elements between rows and pool [pages, 1, page_size, rank]
// (page_stride elements between pages) in the engine's dtype; weight fp32 [rank].
PL_API int pl_norm_write_paged(const void* z, int64_t row_stride, const float* weight, float eps, const int32_t* pos,
                               const int32_t* entry, const int32_t* table, int table_width, void* pool,
                               int64_t page_stride, int page_size, int n_pages, int rank, int n_tokens, int dtype,
                               int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && rank > 0 && page_size > 0 && table_width > 0, "norm_write_paged: bad sizes tokens=%d "
               "rank=%d page=%d", n_tokens, rank, page_size);
    if (n_tokens == 0) {
        return 0;
    }
    const int warps = 4;
    PL_DISPATCH_DTYPE(dtype, "norm_write_paged", {
        pl_launch_overlapped(norm_write_paged_kernel<scalar_t>, dim3((n_tokens + warps - 1) / warps), dim3(warps * 32), 0,
                             stream, static_cast<const scalar_t*>(z), row_stride, weight, eps, pos, entry, table,
                             table_width, static_cast<scalar_t*>(pool), page_stride, page_size, n_pages, rank,
                             n_tokens, status);
    });
    PL_CHECK_LAUNCH("norm_write_paged");
    return 0;
}
