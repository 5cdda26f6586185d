// The residual add and the norms of a block whose two sublayers read the same stream:
//
//   x <- x + s1 * y1 + s2 * y2 (+ also)          y1, y2: the sublayers' outputs, s1, s2: a scale per channel
//   h1 = x * rsqrt(mean(x^2) + eps) * w1,   h2 = the same with w2
//
// One pass over a row: the pending outputs of the block before are scaled and added into
// the fp32 stream, the sum's mean square is formed once, and both sublayers' inputs are
// written. Every term is optional (the first block has nothing pending; a layer without a
// feed-forward has no y2 and wants no h2). `also`: an fp32 row added too (the embedding's
// output entering the stream again before a repeated pass). With `rows` the kernel norms
// only the named rows and writes nothing back (the model's last norm). Sums in fp32, one
// rounding on each store; the order of additions is fixed by the width.
#include "common.cuh"

namespace {

template <typename scalar_t>
__global__ void pair_residual_norm_kernel(float* __restrict__ x, const scalar_t* __restrict__ y1,
                                          const float* __restrict__ s1, const scalar_t* __restrict__ y2,
                                          const float* __restrict__ s2, const float* __restrict__ also,
                                          const float* __restrict__ w1, const float* __restrict__ w2,
                                          scalar_t* __restrict__ h1, scalar_t* __restrict__ h2,
                                          const int32_t* __restrict__ rows, int hidden, float eps) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ float row[];  // [hidden]
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int64_t s = rows != nullptr ? rows[r] : r;
    float* xr = x + s * hidden;
    const bool write_back = rows == nullptr && (y1 != nullptr || y2 != nullptr || also != nullptr);
    float local = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = xr[i];
        float add = 0.0f;
        if (y1 != nullptr) {
            const float a = pl_load(y1 + s * hidden + i);
            add = s1 != nullptr ? a * s1[i] : a;
        }
        if (y2 != nullptr) {
            const float b = pl_load(y2 + s * hidden + i);
            add += s2 != nullptr ? b * s2[i] : b;
        }
        v += add;
        if (also != nullptr) {
            v += also[s * hidden + i];
        }
        if (write_back) {
            xr[i] = v;
        }
        row[i] = v;
        local += v * v;
    }
    const float total = pl_block_sum(local, scratch);
    const float inv_rms = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = row[i] * inv_rms;
        if (h1 != nullptr) {
            pl_store(h1 + static_cast<int64_t>(r) * hidden + i, v * w1[i]);
        }
        if (h2 != nullptr) {
            pl_store(h2 + static_cast<int64_t>(r) * hidden + i, v * w2[i]);
        }
    }
}

}  // namespace

// x fp32 [T, hidden]; y1, y2 [T, hidden] in the engine's dtype (may be null); s1, s2, w1, w2
// fp32 [hidden] (s1, s2 may be null: unscaled); also fp32 [T, hidden] (may be null); h1, h2
// [n_rows, hidden] in the engine's dtype (either may be null); rows int32 [n_rows] or null
// (every row, x updated in place).
PL_API int pl_pair_residual_norm(float* x, const void* y1, const float* s1, const void* y2, const float* s2,
                                 const float* also, const float* w1, const float* w2, void* h1, void* h2,
                                 const int32_t* rows, int n_rows, int hidden, float eps, int dtype,
                                 cudaStream_t stream) {
    PL_REQUIRE(n_rows >= 0 && hidden > 0, "pair_residual_norm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    PL_REQUIRE((h1 == nullptr || w1 != nullptr) && (h2 == nullptr || w2 != nullptr),
               "pair_residual_norm: an output without its norm's weight");
    PL_REQUIRE(static_cast<size_t>(hidden) * sizeof(float) <= 200 * 1024, "pair_residual_norm: hidden %d is too wide",
               hidden);
    if (n_rows == 0) {
        return 0;
    }
    const int threads = hidden >= 1024 ? 256 : hidden >= 256 ? 128 : 64;
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    PL_DISPATCH_DTYPE(dtype, "pair_residual_norm", {
        if (smem > 48 * 1024) {
            cudaFuncSetAttribute(pair_residual_norm_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        }
        pl_launch_overlapped(pair_residual_norm_kernel<scalar_t>, dim3(n_rows), dim3(threads), smem, stream, x,
                             static_cast<const scalar_t*>(y1), s1, static_cast<const scalar_t*>(y2), s2, also, w1, w2,
                             static_cast<scalar_t*>(h1), static_cast<scalar_t*>(h2), rows, hidden, eps);
    });
    PL_CHECK_LAUNCH("pair_residual_norm");
    return 0;
}
