// A sublayer's output normed on its way into the residual stream, fused with the
// norm that feeds the next sublayer:
//
//   u   = y (+ bias)                                   the sublayer's output
//   v   = x + mult * u * rsqrt(mean(u^2) + eps_y) * wy  into the fp32 residual stream
//   out = v * rsqrt(mean(v^2) + eps) * w               the next sublayer's input (optional)
//
// One block per row. All statistics and the residual sum are fp32; the two sums of
// squares are added in an order that depends on the width alone, so a row's result
// does not depend on what else is in the batch.
#include "common.cuh"

namespace {

template <typename scalar_t>
__global__ void add_normed_rmsnorm_kernel(float* __restrict__ x, const scalar_t* __restrict__ y,
                                          const scalar_t* __restrict__ bias, const float* __restrict__ wy,
                                          float mult, float eps_y, const float* __restrict__ w, float eps,
                                          scalar_t* __restrict__ out, const int32_t* __restrict__ rows, int hidden) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ float row_values[];  // [hidden]: u, then v
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int64_t s = rows != nullptr ? rows[r] : r;
    float* xr = x + s * hidden;
    const scalar_t* yr = y + s * hidden;

    float local = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float u = pl_load(yr + i);
        if (bias != nullptr) {
            u += pl_load(bias + i);
        }
        row_values[i] = u;
        local += u * u;
    }
    const float inv_y = 1.0f / sqrtf(pl_block_sum(local, scratch) / static_cast<float>(hidden) + eps_y);
    local = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = xr[i] + mult * (row_values[i] * inv_y * wy[i]);
        row_values[i] = v;
        if (rows == nullptr) {
            xr[i] = v;
        }
        local += v * v;
    }
    if (out == nullptr) {
        return;
    }
    const float inv = 1.0f / sqrtf(pl_block_sum(local, scratch) / static_cast<float>(hidden) + eps);
    scalar_t* outr = out + static_cast<int64_t>(r) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        pl_store(outr + i, row_values[i] * inv * w[i]);
    }
}

}  // namespace

// x fp32 [T, hidden]; y [T, hidden] and the optional bias [hidden] in the engine's dtype;
// wy and w fp32 [hidden]. rows == nullptr: every row, x updated in place. rows given:
// output row r is made from source row rows[r] and x is left as it was. out == nullptr:
// only the residual stream is updated (w is then not read).
PL_API int pl_add_normed_rmsnorm(float* x, const void* y, const void* bias, const float* wy, float mult, float eps_y,
                                 const float* w, float eps, void* out, const int32_t* rows, int n_rows, int hidden,
                                 int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_rows >= 0 && hidden > 0, "add_normed_rmsnorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    PL_REQUIRE(out == nullptr || w != nullptr, "add_normed_rmsnorm: an output needs the second norm's weight");
    PL_REQUIRE(hidden * sizeof(float) <= 160 * 1024, "add_normed_rmsnorm: width %d is too large", hidden);
    if (n_rows == 0) {
        return 0;
    }
    int threads = ((hidden + 3) / 4 + 31) / 32 * 32;
    threads = threads < 64 ? 64 : threads > 512 ? 512 : threads;
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    PL_DISPATCH_DTYPE(dtype, "add_normed_rmsnorm", {
        if (smem > 48 * 1024) {
            cudaFuncSetAttribute(add_normed_rmsnorm_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        }
        cudaError_t err = pl_launch_overlapped(add_normed_rmsnorm_kernel<scalar_t>, dim3(n_rows), dim3(threads), smem,
                                               stream, x, static_cast<const scalar_t*>(y),
                                               static_cast<const scalar_t*>(bias), wy, mult, eps_y, w, eps,
                                               static_cast<scalar_t*>(out), rows, hidden);
        if (err != cudaSuccess) {
            return pl_fail(3, "add_normed_rmsnorm: launch failed: %s", cudaGetErrorString(err));
        }
    });
    return 0;
}
