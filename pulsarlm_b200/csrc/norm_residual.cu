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

// Four elements of the engine's dtype as one load or store.
template <typename scalar_t>
struct FourOf;
template <>
struct FourOf<float> {
    using type = float4;
};
template <>
struct FourOf<__nv_bfloat16> {
    using type = bf16x4;
};
template <typename scalar_t>
using float4_or_half = typename FourOf<scalar_t>::type;

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

// The same with the row in registers (widths that are multiples of 4 up to 4 * VECS * the block
// size, rows that start on 16 bytes): one pass over memory, the weights read before the wait on
// earlier kernels. A thread holds the same elements and adds its squares in the same order as the
// wide form above, so both give the same bits.
template <typename scalar_t, int VECS>
__global__ void __launch_bounds__(512) add_normed_rmsnorm_reg_kernel(
        float* __restrict__ x, const scalar_t* __restrict__ y, const scalar_t* __restrict__ bias,
        const float* __restrict__ wy, float mult, float eps_y, const float* __restrict__ w, float eps,
        scalar_t* __restrict__ out, const int32_t* __restrict__ rows, int hidden, const float* __restrict__ conv_weight,
        scalar_t* __restrict__ conv_state, const int32_t* __restrict__ slots, int taps) {
    pl_grid_trigger();
    __shared__ float scratch[32];
    const int n_vec = hidden / 4;
    float4 gy[VECS], gw[VECS];
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        gy[i] = c < n_vec ? pl_load4(wy + 4 * c) : zero;
        gw[i] = c < n_vec && w != nullptr ? pl_load4(w + 4 * c) : zero;
    }
    pl_grid_wait();
    const int r = blockIdx.x;
    const int64_t s = rows != nullptr ? rows[r] : r;
    float* xr = x + s * hidden;
    const scalar_t* yr = y + s * hidden;
    float4 v[VECS], xv[VECS];
    float local = 0.0f;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n_vec) {
            xv[i] = pl_load4(xr + 4 * c);
            float4 u = pl_load4(yr + 4 * c);
            if (bias != nullptr) {
                const float4 b = pl_load4(bias + 4 * c);
                u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
            }
            v[i] = u;
            local += u.x * u.x;
            local += u.y * u.y;
            local += u.z * u.z;
            local += u.w * u.w;
        }
    }
    const float inv_y = 1.0f / sqrtf(pl_block_sum(local, scratch) / static_cast<float>(hidden) + eps_y);
    local = 0.0f;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n_vec) {
            const float4 u = v[i];
            v[i] = make_float4(xv[i].x + mult * (u.x * inv_y * gy[i].x), xv[i].y + mult * (u.y * inv_y * gy[i].y),
                               xv[i].z + mult * (u.z * inv_y * gy[i].z), xv[i].w + mult * (u.w * inv_y * gy[i].w));
            if (rows == nullptr) {
                pl_store4(xr + 4 * c, v[i]);
            }
            local += v[i].x * v[i].x;
            local += v[i].y * v[i].y;
            local += v[i].z * v[i].z;
            local += v[i].w * v[i].w;
        }
    }
    if (out == nullptr) {
        return;
    }
    const float inv = 1.0f / sqrtf(pl_block_sum(local, scratch) / static_cast<float>(hidden) + eps);
    scalar_t* outr = out + static_cast<int64_t>(r) * hidden;
    const int reach = taps - 1;
    scalar_t* mine = conv_weight != nullptr ? conv_state + static_cast<int64_t>(slots[r]) * reach * hidden : nullptr;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c >= n_vec) {
            continue;
        }
        const float4 h4 = make_float4(v[i].x * inv * gw[i].x, v[i].y * inv * gw[i].y, v[i].z * inv * gw[i].z,
                                      v[i].w * inv * gw[i].w);
        if (conv_weight == nullptr) {
            pl_store4(outr + 4 * c, h4);
            continue;
        }
        // The convolution of a step of single tokens (see the plain form): four channels at a time.
        alignas(16) scalar_t rounded[4];
        pl_store4(rounded, h4);
        const float4 own = pl_load4(rounded);
        const float* cw = conv_weight + static_cast<int64_t>(4 * c) * taps;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int j = 0; j < reach; ++j) {
            alignas(16) scalar_t old_raw[4];
            *reinterpret_cast<float4_or_half<scalar_t>*>(old_raw) =
                *reinterpret_cast<const float4_or_half<scalar_t>*>(mine + static_cast<int64_t>(j) * hidden + 4 * c);
            const float4 old = pl_load4(old_raw);
            acc.x = fmaf(cw[j], old.x, acc.x);
            acc.y = fmaf(cw[taps + j], old.y, acc.y);
            acc.z = fmaf(cw[2 * taps + j], old.z, acc.z);
            acc.w = fmaf(cw[3 * taps + j], old.w, acc.w);
            if (j > 0) {
                *reinterpret_cast<float4_or_half<scalar_t>*>(mine + static_cast<int64_t>(j - 1) * hidden + 4 * c) =
                    *reinterpret_cast<const float4_or_half<scalar_t>*>(old_raw);
            }
        }
        acc.x = fmaf(cw[reach], own.x, acc.x);
        acc.y = fmaf(cw[taps + reach], own.y, acc.y);
        acc.z = fmaf(cw[2 * taps + reach], own.z, acc.z);
        acc.w = fmaf(cw[3 * taps + reach], own.w, acc.w);
        if (reach > 0) {
            *reinterpret_cast<float4_or_half<scalar_t>*>(mine + static_cast<int64_t>(reach - 1) * hidden + 4 * c) =
                *reinterpret_cast<const float4_or_half<scalar_t>*>(rounded);
        }
        pl_store4(outr + 4 * c, make_float4(own.x + acc.x, own.y + acc.y, own.z + acc.z, own.w + acc.w));
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
    const bool conv_rows_aligned = conv_weight == nullptr || taps == 1 || (reinterpret_cast<uintptr_t>(conv_state) & 15) == 0;
    if (vectors && hidden <= 4 * 4 * threads && conv_rows_aligned) {
        const int vecs = (hidden / 4 + threads - 1) / threads;
#define PL_NORM_REG(V)                                                                                              \
    err = pl_launch_overlapped(add_normed_rmsnorm_reg_kernel<scalar_t, V>, dim3(n_rows), dim3(threads), 0, stream,  \
                               x, static_cast<const scalar_t*>(y), static_cast<const scalar_t*>(bias), wy, mult,     \
                               eps_y, w, eps, static_cast<scalar_t*>(out), rows, hidden, conv_weight,                \
                               static_cast<scalar_t*>(conv_state), slots, taps)
        cudaError_t err = cudaSuccess;
        if (dtype == PL_F32) {
            using scalar_t = float;
            if (vecs == 1) { PL_NORM_REG(1); } else if (vecs == 2) { PL_NORM_REG(2); } else { PL_NORM_REG(4); }
        } else if (dtype == PL_BF16) {
            using scalar_t = __nv_bfloat16;
            if (vecs == 1) { PL_NORM_REG(1); } else if (vecs == 2) { PL_NORM_REG(2); } else { PL_NORM_REG(4); }
        } else {
            return pl_fail(2, "add_normed_rmsnorm: unknown dtype code %d", dtype);
        }
#undef PL_NORM_REG
        if (err != cudaSuccess) {
            return pl_fail(3, "add_normed_rmsnorm: launch failed: %s", cudaGetErrorString(err));
        }
        return 0;
    }
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
