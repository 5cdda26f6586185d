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
//
// In a step whose entries bring one token each, the short convolution in front of the
// next sublayer (short_conv.cu) can ride along: the row's normed value h is rounded to the
// engine's dtype, out = h + sum_j cw[:, j] * (the sequence's earlier inputs from its state
// slot, then h), and the slot's rows move up by one with h last; same arithmetic, same
// order, same bits as the two kernels apart.
#include "common.cuh"

namespace {

template <typename scalar_t>
__global__ void add_normed_rmsnorm_kernel(float* __restrict__ x, const scalar_t* __restrict__ y,
                                          const scalar_t* __restrict__ bias, const float* __restrict__ wy,
                                          float mult, float eps_y, const float* __restrict__ w, float eps,
                                          scalar_t* __restrict__ out, const int32_t* __restrict__ rows, int hidden,
                                          const float* __restrict__ conv_weight, scalar_t* __restrict__ conv_state,
                                          const int32_t* __restrict__ slots, int taps, int vectors) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ __align__(16) float row_values[];  // [hidden]: u, then v
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int64_t s = rows != nullptr ? rows[r] : r;
    float* xr = x + s * hidden;
    const scalar_t* yr = y + s * hidden;

    float local = 0.0f;
    scalar_t* outr = out + static_cast<int64_t>(r) * hidden;
    float inv_y;
    if (vectors) {
        // Four elements per thread and pass (the width is a multiple of 4, rows start on 16
        // bytes): each element's arithmetic is that of the plain loops; the sums of squares are
        // added in another order, fixed by the width as well.
        for (int i = 4 * threadIdx.x; i < hidden; i += 4 * blockDim.x) {
            float4 u = pl_load4(yr + i);
            if (bias != nullptr) {
                const float4 b = pl_load4(bias + i);
                u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
            }
            *reinterpret_cast<float4*>(row_values + i) = u;
            local += u.x * u.x;
            local += u.y * u.y;
            local += u.z * u.z;
            local += u.w * u.w;
        }
        inv_y = 1.0f / sqrtf(pl_block_sum(local, scratch) / static_cast<float>(hidden) + eps_y);
        local = 0.0f;
        for (int i = 4 * threadIdx.x; i < hidden; i += 4 * blockDim.x) {
            const float4 u = *reinterpret_cast<const float4*>(row_values + i);
            const float4 xv = pl_load4(xr + i), g = pl_load4(wy + i);
            const float4 v = make_float4(xv.x + mult * (u.x * inv_y * g.x), xv.y + mult * (u.y * inv_y * g.y),
                                         xv.z + mult * (u.z * inv_y * g.z), xv.w + mult * (u.w * inv_y * g.w));
            *reinterpret_cast<float4*>(row_values + i) = v;
            if (rows == nullptr) {
                pl_store4(xr + i, v);
            }
            local += v.x * v.x;
            local += v.y * v.y;
            local += v.z * v.z;
            local += v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float u = pl_load(yr + i);
            if (bias != nullptr) {
                u += pl_load(bias + i);
            }
            row_values[i] = u;
            local += u * u;
        }
        inv_y = 1.0f / sqrtf(pl_block_sum(local, scratch) / static_cast<float>(hidden) + eps_y);
        local = 0.0f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = xr[i] + mult * (row_values[i] * inv_y * wy[i]);
            row_values[i] = v;
            if (rows == nullptr) {
                xr[i] = v;
            }
            local += v * v;
        }
    }
    if (out == nullptr) {
        return;
    }
    // (the sum's barriers also order the row's values for the threads that read them next)
    const float inv = 1.0f / sqrtf(pl_block_sum(local, scratch) / static_cast<float>(hidden) + eps);
    if (conv_weight == nullptr && vectors) {
        for (int i = 4 * threadIdx.x; i < hidden; i += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(row_values + i);
            const float4 g = pl_load4(w + i);
            pl_store4(outr + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
        }
        return;
    }
    if (conv_weight == nullptr) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            pl_store(outr + i, row_values[i] * inv * w[i]);
        }
        return;
    }
    // (one row per entry: row r is entry r, and no other row reads or writes its slot)
    const int reach = taps - 1;
    scalar_t* mine = conv_state + static_cast<int64_t>(slots[r]) * reach * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        scalar_t rounded;
        pl_store(&rounded, row_values[i] * inv * w[i]);
        const float own = pl_load(&rounded);
        const float* cw = conv_weight + static_cast<int64_t>(i) * taps;
        float acc = 0.0f;
        for (int j = 0; j < reach; ++j) {
            const scalar_t old = mine[static_cast<int64_t>(j) * hidden + i];
            acc = fmaf(cw[j], pl_load(&old), acc);
            if (j > 0) {
                mine[static_cast<int64_t>(j - 1) * hidden + i] = old;
            }
        }
        acc = fmaf(cw[reach], own, acc);
        if (reach > 0) {
            mine[static_cast<int64_t>(reach - 1) * hidden + i] = rounded;
        }
        pl_store(outr + i, own + acc);
    }
}

}  // namespace

// x fp32 [T, hidden]; y [T, hidden] and the optional bias [hidden] in the engine's dtype;
// wy and w fp32 [hidden]. rows == nullptr: every row, x updated in place. rows given:
// output row r is made from source row rows[r] and x is left as it was. out == nullptr:
// only the residual stream is updated (w is then not read). conv_weight (fp32 [hidden,
// taps], may be nullptr) with conv_state [slots, taps - 1, hidden] and slots [n_rows]: the
// short convolution of a step of single tokens rides along (rows must be nullptr, row r is
// entry r); out is then the convolution's output and the state slots move on.
PL_API int pl_add_normed_rmsnorm(float* x, const void* y, const void* bias, const float* wy, float mult, float eps_y,
                                 const float* w, float eps, void* out, const int32_t* rows, int n_rows, int hidden,
                                 const float* conv_weight, void* conv_state, const int32_t* slots, int taps,
                                 int dtype, cudaStream_t stream) {
    PL_REQUIRE(conv_weight == nullptr || (rows == nullptr && out != nullptr && slots != nullptr && taps >= 1 &&
                                          (taps == 1 || conv_state != nullptr)),
               "add_normed_rmsnorm: the convolution rides along only over all rows, with an output, slots and a state");
    PL_REQUIRE(n_rows >= 0 && hidden > 0, "add_normed_rmsnorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    PL_REQUIRE(out == nullptr || w != nullptr, "add_normed_rmsnorm: an output needs the second norm's weight");
    PL_REQUIRE(hidden * sizeof(float) <= 160 * 1024, "add_normed_rmsnorm: width %d is too large", hidden);
    if (n_rows == 0) {
        return 0;
    }
    // The wide form where rows start on 16 bytes (whether or not a convolution rides along: a
    // width keeps one order of its sums).
    const int vectors = hidden % 4 == 0 &&
        ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(bias) |
          reinterpret_cast<uintptr_t>(wy) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
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
                                               static_cast<scalar_t*>(out), rows, hidden, conv_weight,
                                               static_cast<scalar_t*>(conv_state), slots, taps, vectors);
        if (err != cudaSuccess) {
            return pl_fail(3, "add_normed_rmsnorm: launch failed: %s", cudaGetErrorString(err));
        }
    });
    return 0;
}
