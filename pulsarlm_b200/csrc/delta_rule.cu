// The generalized delta rule: a recurrent mixer whose state per head is a matrix S [K, V]
// kept in fp32 from token to token.
//
//   u_t = k_t / sqrt(|k_t|^2 + unit_eps)
//   w_t = exp(-decay_scale * sigmoid(w~_t + w0))          decay per key channel
//   a_t = sigmoid(a~_t + a0)                               removal rate per key channel
//   S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T
//   o_t = S_t^T r_t
//   out_t = o_t * rsqrt(mean(o_t^2) + eps) * norm * sigmoid(g_t)      per head
//
// One CTA per (batch entry, head) walks the entry's rows in order. Column j of S never
// meets another column, so each column lives in registers: `parts` lanes of a warp share
// a column, lane p holding rows p, p + parts, ... . Everything above is fp32 (the
// projections r, k, v, w~, a~, g arrive in the engine's dtype); a token's result depends on
// the tokens before it alone, not on how the prompt was cut or on the rest of the batch.
#include "common.cuh"

namespace {

constexpr int kRowsPerLane = 32;

__device__ __forceinline__ float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename scalar_t>
__global__ void delta_rule_kernel(const scalar_t* __restrict__ r, const scalar_t* __restrict__ k,
                                  const scalar_t* __restrict__ v, const scalar_t* __restrict__ g,
                                  const scalar_t* __restrict__ a_pre, int64_t row_stride,
                                  const scalar_t* __restrict__ w_pre, int64_t w_row_stride,
                                  const float* __restrict__ w0, const float* __restrict__ a0,
                                  const float* __restrict__ norm, float* __restrict__ state,
                                  const int32_t* __restrict__ first_rows, const int32_t* __restrict__ counts,
                                  const int32_t* __restrict__ slots, scalar_t* __restrict__ out,
                                  int64_t out_row_stride, int n_heads, int dim, int parts, float decay_scale,
                                  float unit_eps, float eps) {
    extern __shared__ float shared[];
    float* sk = shared;            // k
    float* su = sk + dim;          // unit key
    float* sw = su + dim;          // decay
    float* sau = sw + dim;         // removal rate times unit key
    float* sr = sau + dim;         // r
    __shared__ float scratch[32];

    const int e = blockIdx.x, head = blockIdx.y;
    const int tid = threadIdx.x;
    const int col = tid / parts, part = tid % parts;   // (threads past dim * parts only wait and shuffle)
    const bool active = col < dim;
    const int first = first_rows[e], count = counts[e];
    float* mine = state + (static_cast<int64_t>(slots[e]) * n_heads + head) * dim * dim;
    const int64_t hoff = static_cast<int64_t>(head) * dim;

    float S[kRowsPerLane];
#pragma unroll
    for (int m = 0; m < kRowsPerLane; ++m) {
        const int i = part + m * parts;
        S[m] = active && i < dim ? mine[static_cast<int64_t>(i) * dim + col] : 0.0f;
    }
    const float norm_w = active ? norm[hoff + col] : 0.0f;

    for (int t = first; t < first + count; ++t) {
        float square = 0.0f;
        if (tid < dim) {
            const float kv = pl_load(k + t * row_stride + hoff + tid);
            sk[tid] = kv;
            sr[tid] = pl_load(r + t * row_stride + hoff + tid);
            sw[tid] = expf(-decay_scale * sigmoid_f32(pl_load(w_pre + t * w_row_stride + hoff + tid) + w0[hoff + tid]));
            square = kv * kv;
        }
        const float inv = 1.0f / sqrtf(pl_block_sum(square, scratch) + unit_eps);
        if (tid < dim) {
            const float u = sk[tid] * inv;
            su[tid] = u;
            sau[tid] = sigmoid_f32(pl_load(a_pre + t * row_stride + hoff + tid) + a0[hoff + tid]) * u;
        }
        __syncthreads();
        const float vj = active ? pl_load(v + t * row_stride + hoff + col) : 0.0f;
        float dot = 0.0f;
#pragma unroll
        for (int m = 0; m < kRowsPerLane; ++m) {
            const int i = part + m * parts;
            if (i < dim) {
                dot = fmaf(su[i], S[m], dot);
            }
        }
        for (int offset = parts >> 1; offset > 0; offset >>= 1) {
            dot += __shfl_xor_sync(0xffffffffu, dot, offset);
        }
        float o = 0.0f;
#pragma unroll
        for (int m = 0; m < kRowsPerLane; ++m) {
            const int i = part + m * parts;
            if (i < dim) {
                S[m] = fmaf(sk[i], vj, fmaf(-sau[i], dot, sw[i] * S[m]));
                o = fmaf(S[m], sr[i], o);
            }
        }
        for (int offset = parts >> 1; offset > 0; offset >>= 1) {
            o += __shfl_xor_sync(0xffffffffu, o, offset);
        }
        const float total = pl_block_sum(active && part == 0 ? o * o : 0.0f, scratch);
        if (active && part == 0) {
            const float gate = sigmoid_f32(pl_load(g + t * row_stride + hoff + col));
            pl_store(out + t * out_row_stride + hoff + col,
                     o * (1.0f / sqrtf(total / static_cast<float>(dim) + eps)) * norm_w * gate);
        }
    }
#pragma unroll
    for (int m = 0; m < kRowsPerLane; ++m) {
        const int i = part + m * parts;
        if (active && i < dim) {
            mine[static_cast<int64_t>(i) * dim + col] = S[m];
        }
    }
}

}  // namespace

// r, k, v, g, a_pre: [T, heads * dim] in the engine's dtype with `row_stride` elements
// between rows (columns of one projection output); w_pre likewise with w_row_stride. w0,
// a0, norm fp32 [heads * dim]. state fp32 [slots, heads, dim, dim] (key channel, value
// channel), updated in place. first_rows, counts, slots: int32 [entries]. out [T, heads *
// dim] in the engine's dtype.
PL_API int pl_delta_rule(const void* r, const void* k, const void* v, const void* g, const void* a_pre,
                         int64_t row_stride, const void* w_pre, int64_t w_row_stride, const float* w0,
                         const float* a0, const float* norm, float* state, const int32_t* first_rows,
                         const int32_t* counts, const int32_t* slots, void* out, int64_t out_row_stride,
                         int n_entries, int n_heads, int dim, float decay_scale, float unit_eps, float eps, int dtype,
                         cudaStream_t stream) {
    PL_REQUIRE(n_entries >= 0 && n_heads > 0 && dim > 0, "delta_rule: bad sizes entries=%d heads=%d dim=%d", n_entries,
               n_heads, dim);
    PL_REQUIRE(n_heads <= 65535, "delta_rule: %d heads exceed the grid limit", n_heads);
    // Lanes per column: a power of two, so that a lane holds at most kRowsPerLane rows and a
    // CTA has at most 1024 threads.
    int parts = 1;
    while (parts < 32 && (dim + parts - 1) / parts > kRowsPerLane) {
        parts *= 2;
    }
    if (parts == 1 && dim >= 32 && dim * 2 <= 1024) {
        parts = 2;  // (shorter chains per token where the CTA has room)
    }
    PL_REQUIRE((dim + parts - 1) / parts <= kRowsPerLane && dim * parts <= 1024,
               "delta_rule: head size %d is too large (at most 128)", dim);
    if (n_entries == 0) {
        return 0;
    }
    const size_t smem = static_cast<size_t>(5 * dim) * sizeof(float);
    PL_DISPATCH_DTYPE(dtype, "delta_rule", {
        delta_rule_kernel<scalar_t><<<dim3(n_entries, n_heads), (dim * parts + 31) / 32 * 32, smem, stream>>>(
            static_cast<const scalar_t*>(r), static_cast<const scalar_t*>(k), static_cast<const scalar_t*>(v),
            static_cast<const scalar_t*>(g), static_cast<const scalar_t*>(a_pre), row_stride,
            static_cast<const scalar_t*>(w_pre), w_row_stride, w0, a0, norm, state, first_rows, counts, slots,
            static_cast<scalar_t*>(out), out_row_stride, n_heads, dim, parts, decay_scale, unit_eps, eps);
    });
    PL_CHECK_LAUNCH("delta_rule");
    return 0;
}
