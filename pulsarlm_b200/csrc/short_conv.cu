// A short causal convolution over time on every channel, added to its own input:
//
//   out[t, c] = h[t, c] + sum_{j < taps} w[c, j] * h_seq[t - (taps - 1) + j, c]
//
// or, for a mixer that filters its projections (pl_short_conv_act), without the input added
// and with an activation: out = act(conv), act = silu or none; the rows of h may then be
// columns of a wider matrix (h_stride elements between rows).
//
// where h_seq is the sequence's input so far, zeros before its start. A step brings a
// sequence's next rows (an entry's rows are consecutive and in order); the taps - 1 inputs
// before them come from the sequence's state slot [taps - 1, width] (oldest first), which
// a second kernel brings up to date afterwards. Products and sums are fp32, one rounding
// on store. A row's result depends on the sequence's inputs alone, not on how they were
// cut into steps or on the rest of the batch.
#include "common.cuh"

namespace {

constexpr int kMaxTaps = 16;

// What a row stores: the convolution added to its input, or the convolution alone, then the
// activation (1: silu, z * sigmoid(z), with expf).
__device__ __forceinline__ float conv_result(float own, float acc, int residual, int act) {
    const float z = residual ? own + acc : acc;
    return act == 1 ? z / (1.0f + expf(-z)) : z;
}
__device__ __forceinline__ float4 conv_result(float4 own, float4 acc, int residual, int act) {
    return make_float4(conv_result(own.x, acc.x, residual, act), conv_result(own.y, acc.y, residual, act),
                       conv_result(own.z, acc.z, residual, act), conv_result(own.w, acc.w, residual, act));
}

template <typename scalar_t>
__global__ void short_conv_kernel(const scalar_t* __restrict__ h, const float* __restrict__ weight,
                                  const scalar_t* __restrict__ state, const int32_t* __restrict__ entry,
                                  const int32_t* __restrict__ slots, scalar_t* __restrict__ out, int n_tokens,
                                  int width, int taps, int vectors, int64_t h_stride, int residual, int act) {
    pl_grid_trigger();
    pl_grid_wait();
    const int t = blockIdx.x;
    const int e = entry[t];
    const int reach = taps - 1;
    // How many of the rows before this one belong to the same sequence (up to `reach`).
    int inside = 0;
    while (inside < reach && t - inside - 1 >= 0 && entry[t - inside - 1] == e) {
        ++inside;
    }
    const scalar_t* old = state + static_cast<int64_t>(slots[e]) * reach * width;
    if (vectors) {
        // Four channels per thread, 8- or 16-byte loads (the width is a multiple of 4 and rows start on 16 bytes).
        for (int c = 4 * threadIdx.x; c < width; c += 4 * blockDim.x) {
            const float4 own = pl_load4(h + static_cast<int64_t>(t) * h_stride + c);
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int j = 0; j < taps; ++j) {
                const int back = reach - j;
                float4 v;
                if (back == 0) {
                    v = own;
                } else if (back <= inside) {
                    v = pl_load4(h + static_cast<int64_t>(t - back) * h_stride + c);
                } else {
                    v = pl_load4(old + static_cast<int64_t>(reach - (back - inside)) * width + c);
                }
                acc.x = fmaf(weight[static_cast<int64_t>(c) * taps + j], v.x, acc.x);
                acc.y = fmaf(weight[static_cast<int64_t>(c + 1) * taps + j], v.y, acc.y);
                acc.z = fmaf(weight[static_cast<int64_t>(c + 2) * taps + j], v.z, acc.z);
                acc.w = fmaf(weight[static_cast<int64_t>(c + 3) * taps + j], v.w, acc.w);
            }
            pl_store4(out + static_cast<int64_t>(t) * width + c, conv_result(own, acc, residual, act));
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float* w = weight + static_cast<int64_t>(c) * taps;
        const float own = pl_load(h + static_cast<int64_t>(t) * h_stride + c);
        float acc = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int back = reach - j;  // this tap reads the input `back` rows before
            float v;
            if (back == 0) {
                v = own;
            } else if (back <= inside) {
                v = pl_load(h + static_cast<int64_t>(t - back) * h_stride + c);
            } else {
                v = pl_load(old + static_cast<int64_t>(reach - (back - inside)) * width + c);
            }
            acc = fmaf(w[j], v, acc);
        }
        pl_store(out + static_cast<int64_t>(t) * width + c, conv_result(own, acc, residual, act));
    }
}

// The same for the usual few taps and widths that are multiples of 4: a block walks kRowsPerBlock
// rows of 4 * 128 channels with the earlier inputs in registers, so a row of h is read once
// instead of `taps` times and the weights once a block. Same products in the same order as the
// kernel above: same bits.
constexpr int kRowsPerBlock = 16;

template <typename scalar_t, int TAPS>
__global__ void __launch_bounds__(128) short_conv_rows_kernel(
        const scalar_t* __restrict__ h, const float* __restrict__ weight, const scalar_t* __restrict__ state,
        const int32_t* __restrict__ entry, const int32_t* __restrict__ slots, scalar_t* __restrict__ out, int n_tokens,
        int width, int64_t h_stride, int residual, int act) {
    pl_grid_trigger();
    constexpr int REACH = TAPS - 1;
    const int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
    const int t0 = blockIdx.x * kRowsPerBlock;
    if (c >= width) {
        return;
    }
    float w[4][TAPS];  // (weights: read before the wait on earlier kernels)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
            w[q][j] = weight[static_cast<int64_t>(c + q) * TAPS + j];
        }
    }
    pl_grid_wait();
    float4 window[REACH > 0 ? REACH : 1];  // the inputs before the row at hand, oldest first
    float4 last = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    int last_entry = -1;
    for (int t = t0; t < min(t0 + kRowsPerBlock, n_tokens); ++t) {
        const int e = entry[t];
        if (t == t0) {
            int inside = 0;
            while (inside < REACH && t - inside - 1 >= 0 && entry[t - inside - 1] == e) {
                ++inside;
            }
            const scalar_t* old = state + static_cast<int64_t>(slots[e]) * REACH * width;
#pragma unroll
            for (int j = 0; j < REACH; ++j) {
                const int back = REACH - j;
                window[j] = back <= inside ? pl_load4(h + static_cast<int64_t>(t - back) * h_stride + c)
                                           : pl_load4(old + static_cast<int64_t>(REACH - (back - inside)) * width + c);
            }
        } else if (e != last_entry) {
            const scalar_t* old = state + static_cast<int64_t>(slots[e]) * REACH * width;
#pragma unroll
            for (int j = 0; j < REACH; ++j) {
                window[j] = pl_load4(old + static_cast<int64_t>(j) * width + c);
            }
        } else {
#pragma unroll
            for (int j = 0; j + 1 < REACH; ++j) {
                window[j] = window[j + 1];
            }
            if (REACH > 0) {
                window[REACH - 1] = last;
            }
        }
        const float4 own = pl_load4(h + static_cast<int64_t>(t) * h_stride + c);
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < REACH; ++j) {
            acc.x = fmaf(w[0][j], window[j].x, acc.x);
            acc.y = fmaf(w[1][j], window[j].y, acc.y);
            acc.z = fmaf(w[2][j], window[j].z, acc.z);
            acc.w = fmaf(w[3][j], window[j].w, acc.w);
        }
        acc.x = fmaf(w[0][REACH], own.x, acc.x);
        acc.y = fmaf(w[1][REACH], own.y, acc.y);
        acc.z = fmaf(w[2][REACH], own.z, acc.z);
        acc.w = fmaf(w[3][REACH], own.w, acc.w);
        pl_store4(out + static_cast<int64_t>(t) * width + c, conv_result(own, acc, residual, act));
        last = own;
        last_entry = e;
    }
}

// A step in which every entry brings one row: the convolution and the state's update in one
// kernel. A thread takes four channels, holds the taps - 1 earlier inputs in registers, writes
// the row's result and then the state moved up by one with the row's input last. Same
// products in the same order as the kernels above.
template <typename scalar_t, int TAPS>
__global__ void __launch_bounds__(128) short_conv_single_kernel(
        const scalar_t* __restrict__ h, const float* __restrict__ weight, scalar_t* __restrict__ state,
        const int32_t* __restrict__ entry, const int32_t* __restrict__ slots, scalar_t* __restrict__ out, int width,
        int64_t h_stride, int residual, int act) {
    pl_grid_trigger();
    constexpr int REACH = TAPS - 1;
    const int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
    const int t = blockIdx.x;
    if (c >= width) {
        return;
    }
    float w[4][TAPS];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
            w[q][j] = weight[static_cast<int64_t>(c + q) * TAPS + j];
        }
    }
    scalar_t* mine = state + static_cast<int64_t>(slots[entry[t]]) * REACH * width + c;
    pl_grid_wait();
    float4 window[REACH > 0 ? REACH : 1];
#pragma unroll
    for (int j = 0; j < REACH; ++j) {
        window[j] = pl_load4(mine + static_cast<int64_t>(j) * width);
    }
    const float4 own = pl_load4(h + static_cast<int64_t>(t) * h_stride + c);
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < REACH; ++j) {
        acc.x = fmaf(w[0][j], window[j].x, acc.x);
        acc.y = fmaf(w[1][j], window[j].y, acc.y);
        acc.z = fmaf(w[2][j], window[j].z, acc.z);
        acc.w = fmaf(w[3][j], window[j].w, acc.w);
    }
    acc.x = fmaf(w[0][REACH], own.x, acc.x);
    acc.y = fmaf(w[1][REACH], own.y, acc.y);
    acc.z = fmaf(w[2][REACH], own.z, acc.z);
    acc.w = fmaf(w[3][REACH], own.w, acc.w);
    pl_store4(out + static_cast<int64_t>(t) * width + c, conv_result(own, acc, residual, act));
#pragma unroll
    for (int j = 0; j + 1 < REACH; ++j) {
        pl_store4(mine + static_cast<int64_t>(j) * width, window[j + 1]);
    }
    if (REACH > 0) {
        pl_store4(mine + static_cast<int64_t>(REACH - 1) * width, own);
    }
}

// The state after the step: the last taps - 1 inputs of each sequence. A portion of at least
// taps - 1 rows writes them from its last rows; a shorter one is handled by its first row's
// block, which also moves the older rows up.
template <typename scalar_t>
__global__ void short_conv_state_kernel(const scalar_t* __restrict__ h, const int32_t* __restrict__ entry,
                                        const int32_t* __restrict__ slots, scalar_t* __restrict__ state,
                                        int n_tokens, int width, int taps, int64_t h_stride) {
    pl_grid_trigger();
    pl_grid_wait();
    const int t = blockIdx.x;
    const int e = entry[t];
    const int reach = taps - 1;
    int before = 0, after = 0;
    while (before < reach && t - before - 1 >= 0 && entry[t - before - 1] == e) {
        ++before;
    }
    while (after < reach && t + after + 1 < n_tokens && entry[t + after + 1] == e) {
        ++after;
    }
    scalar_t* mine = state + static_cast<int64_t>(slots[e]) * reach * width;
    // (both counts stop at `reach`: a count that got there means "at least")
    if (before == reach || after == reach || before + 1 + after >= reach) {
        // A portion of at least `reach` rows: each of its last `reach` rows writes itself.
        if (after < reach) {
            for (int c = threadIdx.x; c < width; c += blockDim.x) {
                mine[static_cast<int64_t>(reach - 1 - after) * width + c] = h[static_cast<int64_t>(t) * h_stride + c];
            }
        }
        return;
    }
    if (before != 0) {
        return;
    }
    // A portion of n < reach rows, and this is its first: rows move up by n, the new ones follow.
    const int n = 1 + after;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        for (int j = 0; j < reach - n; ++j) {
            mine[static_cast<int64_t>(j) * width + c] = mine[static_cast<int64_t>(j + n) * width + c];
        }
        for (int m = 0; m < n; ++m) {
            mine[static_cast<int64_t>(reach - n + m) * width + c] = h[static_cast<int64_t>(t + m) * h_stride + c];
        }
    }
}

}  // namespace

// h, out [T, width] and state [slots, taps - 1, width] in the engine's dtype; weight fp32
// [width, taps]; entry int32 [T] names each row's batch entry, slots int32 [entries] each
// entry's state slot. out may not alias h. The state is read, not written.
static int short_conv_launch(const void* h, int64_t h_stride, const float* weight, const void* state,
                             const int32_t* entry, const int32_t* slots, void* out, int n_tokens, int width, int taps,
                             int residual, int act, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && width > 0 && taps >= 1 && taps <= kMaxTaps, "short_conv: bad sizes tokens=%d width=%d "
               "taps=%d (at most %d)", n_tokens, width, taps, kMaxTaps);
    if (n_tokens == 0) {
        return 0;
    }
    const int vectors = width % 4 == 0 && h_stride % 4 == 0 &&
        ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    // (few rows: steps of single tokens, where a block per row is ahead of a block walking rows one after the other)
    if (vectors && taps >= 2 && taps <= 6 && n_tokens > 64) {
        const dim3 grid((n_tokens + kRowsPerBlock - 1) / kRowsPerBlock, (width / 4 + 127) / 128);
#define PL_CONV_ROWS(T)                                                                                          \
    pl_launch_overlapped(short_conv_rows_kernel<scalar_t, T>, grid, dim3(128), 0, stream,                        \
                         static_cast<const scalar_t*>(h), weight, static_cast<const scalar_t*>(state), entry,    \
                         slots, static_cast<scalar_t*>(out), n_tokens, width, h_stride, residual, act)
        if (dtype == PL_F32) {
            using scalar_t = float;
            switch (taps) {
                case 2: PL_CONV_ROWS(2); break;
                case 3: PL_CONV_ROWS(3); break;
                case 4: PL_CONV_ROWS(4); break;
                case 5: PL_CONV_ROWS(5); break;
                default: PL_CONV_ROWS(6); break;
            }
        } else if (dtype == PL_BF16) {
            using scalar_t = __nv_bfloat16;
            switch (taps) {
                case 2: PL_CONV_ROWS(2); break;
                case 3: PL_CONV_ROWS(3); break;
                case 4: PL_CONV_ROWS(4); break;
                case 5: PL_CONV_ROWS(5); break;
                default: PL_CONV_ROWS(6); break;
            }
        } else {
            return pl_fail(2, "short_conv: unknown dtype code %d", dtype);
        }
#undef PL_CONV_ROWS
        PL_CHECK_LAUNCH("short_conv");
        return 0;
    }
    const int lanes = vectors ? width / 4 : width;
    const int threads = lanes >= 256 ? 256 : ((lanes + 31) / 32) * 32;
    PL_DISPATCH_DTYPE(dtype, "short_conv", {
        pl_launch_overlapped(short_conv_kernel<scalar_t>, dim3(n_tokens), dim3(threads), 0, stream,
                             static_cast<const scalar_t*>(h), weight, static_cast<const scalar_t*>(state), entry, slots,
                             static_cast<scalar_t*>(out), n_tokens, width, taps, vectors, h_stride, residual, act);
    });
    PL_CHECK_LAUNCH("short_conv");
    return 0;
}

PL_API int pl_short_conv(const void* h, const float* weight, const void* state, const int32_t* entry,
                         const int32_t* slots, void* out, int n_tokens, int width, int taps, int dtype,
                         cudaStream_t stream) {
    return short_conv_launch(h, width, weight, state, entry, slots, out, n_tokens, width, taps, 1, 0, dtype, stream);
}

// The same with the rows of h `h_stride` elements apart, the input added only when `residual`,
// and an activation on the result (0: none, 1: silu). out [T, width] is contiguous.
PL_API int pl_short_conv_act(const void* h, int64_t h_stride, const float* weight, const void* state,
                             const int32_t* entry, const int32_t* slots, void* out, int n_tokens, int width, int taps,
                             int residual, int act, int dtype, cudaStream_t stream) {
    PL_REQUIRE(act == 0 || act == 1, "short_conv: unknown activation code %d", act);
    PL_REQUIRE(h_stride >= width, "short_conv: rows of %d columns cannot be %lld elements apart", width,
               static_cast<long long>(h_stride));
    return short_conv_launch(h, h_stride, weight, state, entry, slots, out, n_tokens, width, taps, residual, act,
                             dtype, stream);
}

// Brings every entry's state slot up to date with the step's inputs h (run after
// pl_short_conv has read the old state).
PL_API int pl_short_conv_state(const void* h, const int32_t* entry, const int32_t* slots, void* state, int n_tokens,
                               int width, int taps, int dtype, cudaStream_t stream);

// (h_stride: elements between the rows of h)
PL_API int pl_short_conv_state_strided(const void* h, int64_t h_stride, const int32_t* entry, const int32_t* slots,
                                       void* state, int n_tokens, int width, int taps, int dtype,
                                       cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && width > 0 && taps >= 1 && taps <= kMaxTaps, "short_conv_state: bad sizes tokens=%d "
               "width=%d taps=%d", n_tokens, width, taps);
    if (n_tokens == 0 || taps == 1) {
        return 0;
    }
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    PL_DISPATCH_DTYPE(dtype, "short_conv_state", {
        pl_launch_overlapped(short_conv_state_kernel<scalar_t>, dim3(n_tokens), dim3(threads), 0, stream,
                             static_cast<const scalar_t*>(h), entry, slots, static_cast<scalar_t*>(state), n_tokens,
                             width, taps, h_stride);
    });
    PL_CHECK_LAUNCH("short_conv_state");
    return 0;
}

PL_API int pl_short_conv_state(const void* h, const int32_t* entry, const int32_t* slots, void* state, int n_tokens,
                               int width, int taps, int dtype, cudaStream_t stream) {
    return pl_short_conv_state_strided(h, width, entry, slots, state, n_tokens, width, taps, dtype, stream);
}


// For a step in which every entry brings exactly one row (the caller vouches for it): the
// convolution as pl_short_conv_act and the state's update in one launch. Returns 1 without
// launching when the sizes are not the ones this form takes (taps 2 to 6, a width that is a
// multiple of 4, rows on 16 bytes): the caller then runs the two kernels.
PL_API int pl_short_conv_single(const void* h, int64_t h_stride, const float* weight, void* state,
                                const int32_t* entry, const int32_t* slots, void* out, int n_tokens, int width,
                                int taps, int residual, int act, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && width > 0 && taps >= 1 && taps <= kMaxTaps && (act == 0 || act == 1),
               "short_conv_single: bad arguments tokens=%d width=%d taps=%d act=%d", n_tokens, width, taps, act);
    const bool vectors = width % 4 == 0 && h_stride % 4 == 0 &&
        ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (!vectors || taps < 2 || taps > 6 || (dtype != PL_F32 && dtype != PL_BF16)) {
        return 1;
    }
    if (n_tokens == 0) {
        return 0;
    }
    const dim3 grid(n_tokens, (width / 4 + 127) / 128);
#define PL_CONV_SINGLE(T)                                                                                          \
    pl_launch_overlapped(short_conv_single_kernel<scalar_t, T>, grid, dim3(128), 0, stream,                        \
                         static_cast<const scalar_t*>(h), weight, static_cast<scalar_t*>(state), entry, slots,     \
                         static_cast<scalar_t*>(out), width, h_stride, residual, act)
    if (dtype == PL_F32) {
        using scalar_t = float;
        switch (taps) {
            case 2: PL_CONV_SINGLE(2); break;
            case 3: PL_CONV_SINGLE(3); break;
            case 4: PL_CONV_SINGLE(4); break;
            case 5: PL_CONV_SINGLE(5); break;
            default: PL_CONV_SINGLE(6); break;
        }
    } else {
        using scalar_t = __nv_bfloat16;
        switch (taps) {
            case 2: PL_CONV_SINGLE(2); break;
            case 3: PL_CONV_SINGLE(3); break;
            case 4: PL_CONV_SINGLE(4); break;
            case 5: PL_CONV_SINGLE(5); break;
            default: PL_CONV_SINGLE(6); break;
        }
    }
#undef PL_CONV_SINGLE
    PL_CHECK_LAUNCH("short_conv_single");
    return 0;
}
