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
// Two kernels. The scan: a CTA per (batch entry, head, block of value columns) walks the
// entry's rows in order. Column j of S never meets another column, so each column lives in
// registers: `parts` lanes of a warp share a column and each holds some of its rows. The
// rows are taken in chunks: while one chunk's tokens update the state one after the other
// (no block-wide wait inside: only the shuffles among a column's lanes), the next chunk's
// projections arrive in shared memory (cp.async); between chunks all threads turn them
// into the fp32 vectors u, w, a * u, k, r that the update reads (the unit-key factor by a
// warp per token, the rest one (token, channel) per thread, so that the exponentials
// overlap). Head sizes 16, 32, 64 and 128 run a form with the sizes known to the compiler:
// a lane holds consecutive rows, reads its share of the vectors one token ahead with
// 16-byte loads, and leaves its share of o in shared memory, added up after the chunk, off
// the path from one token to the next. The raw o goes to scratch in fp32; the second kernel
// norms it per head, applies the norm's weight and the gate and rounds once. Everything
// after the projections is fp32 (they arrive in the engine's dtype). The order of every sum
// depends on the head size alone, so a token's result depends on the tokens before it only,
// not on how the prompt was cut, on the chunks or on the rest of the batch. What bounds the
// scan is the chain from one token's state to the next (a dot product over a column, the
// shuffles that add its lanes' shares, the update): a prompt of one request keeps a few SMs
// busy and takes about a microsecond a token whatever the width.
#include "common.cuh"

#include "mma_helpers.cuh"

namespace {

constexpr int kRowsPerLane = 16;
constexpr int kMaxThreads = 512;
constexpr int kMaxChunk = 16;

__device__ __forceinline__ float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }

struct ScanParams {
    const void* r;
    const void* k;
    const void* v;
    const void* a_pre;
    int64_t row_stride;
    const void* w_pre;
    int64_t w_row_stride;
    const float* w0;
    const float* a0;
    float* state;
    const int32_t* first_rows;
    const int32_t* counts;
    const int32_t* slots;
    float* o_raw;  // [T, heads * dim]
    int n_heads, dim, parts, cols, chunk;
    int async_loads;  // every row of every operand starts on 16 bytes
    float decay_scale, unit_eps;
};

// One chunk's raw projections -> shared memory: [token][r, k, w~, a~][dim], then [token][cols] of v.
template <typename scalar_t>
__device__ __forceinline__ void load_chunk(const ScanParams& p, scalar_t* raw, int t0, int n, int64_t hoff, int col0,
                                           int n_cols) {
    const scalar_t* src[4] = {static_cast<const scalar_t*>(p.r), static_cast<const scalar_t*>(p.k),
                              static_cast<const scalar_t*>(p.w_pre), static_cast<const scalar_t*>(p.a_pre)};
    const int dim = p.dim;
    scalar_t* raw_v = raw + p.chunk * 4 * dim;
    if (p.async_loads) {
        constexpr int kPer = 16 / sizeof(scalar_t);
        const int gv = dim / kPer, gc = p.cols / kPer;
        const int per_token = 4 * gv + gc;
        for (int idx = threadIdx.x; idx < n * per_token; idx += blockDim.x) {
            const int c = idx / per_token, g = idx % per_token;
            if (g < 4 * gv) {
                const int which = g / gv, e = (g % gv) * kPer;
                const int64_t stride = which == 2 ? p.w_row_stride : p.row_stride;
                cp_async_16(raw + (c * 4 + which) * dim + e, src[which] + (t0 + c) * stride + hoff + e);
            } else {
                const int e = (g - 4 * gv) * kPer;
                if (e < n_cols) {  // (n_cols is a multiple of kPer here)
                    cp_async_16(raw_v + c * p.cols + e,
                                static_cast<const scalar_t*>(p.v) + (t0 + c) * p.row_stride + hoff + col0 + e);
                }
            }
        }
    } else {
        const int per_token = 4 * dim + n_cols;
        for (int idx = threadIdx.x; idx < n * per_token; idx += blockDim.x) {
            const int c = idx / per_token, g = idx % per_token;
            if (g < 4 * dim) {
                const int which = g / dim, e = g % dim;
                const int64_t stride = which == 2 ? p.w_row_stride : p.row_stride;
                raw[(c * 4 + which) * dim + e] = src[which][(t0 + c) * stride + hoff + e];
            } else {
                const int e = g - 4 * dim;
                raw_v[c * p.cols + e] = static_cast<const scalar_t*>(p.v)[(t0 + c) * p.row_stride + hoff + col0 + e];
            }
        }
    }
    cp_async_commit();
}

// The fp32 vectors of the update for one chunk: first each token's unit-key factor (a warp per
// token), then every (token, channel) on its own, so that the exponentials' latencies overlap.
// vec: [token][k, u, w, a * u, r][dim]. Ends with the block in step.
template <typename scalar_t>
__device__ __forceinline__ void prepare_chunk(const ScanParams& p, const scalar_t* raw, float* vec,
                                              const float* offsets, float* inv_norm, int n, int dim) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    for (int c = warp; c < n; c += warps) {
        const scalar_t* rk = raw + (c * 4 + 1) * dim;
        float square = 0.0f;
        for (int i = lane; i < dim; i += 32) {
            const float kv = pl_load(rk + i);
            square += kv * kv;
        }
        square = pl_warp_sum(square);
        if (lane == 0) {
            inv_norm[c] = 1.0f / sqrtf(square + p.unit_eps);
        }
    }
    __syncthreads();
    for (int idx = tid; idx < n * dim; idx += blockDim.x) {
        const int c = idx / dim, i = idx - c * dim;
        const scalar_t* token = raw + c * 4 * dim;
        const float kv = pl_load(token + dim + i);
        const float u = kv * inv_norm[c];
        float* out = vec + c * 5 * dim;
        out[i] = kv;
        out[dim + i] = u;
        out[2 * dim + i] = expf(-p.decay_scale * sigmoid_f32(pl_load(token + 2 * dim + i) + offsets[i]));
        out[3 * dim + i] = sigmoid_f32(pl_load(token + 3 * dim + i) + offsets[dim + i]) * u;
        out[4 * dim + i] = pl_load(token + i);
    }
    __syncthreads();
}

template <typename scalar_t>
__global__ void __launch_bounds__(kMaxThreads) delta_rule_scan_kernel(const ScanParams p) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    const int dim = p.dim, parts = p.parts, chunk = p.chunk;
    // [2][dim] offsets, [chunk][5][dim] vectors, then two raw buffers
    float* offsets = reinterpret_cast<float*>(smem);
    float* vec = offsets + 2 * dim;
    const int raw_elems = chunk * (4 * dim + p.cols);
    const int raw_bytes = (raw_elems * static_cast<int>(sizeof(scalar_t)) + 15) / 16 * 16;
    unsigned char* raw_base = reinterpret_cast<unsigned char*>(vec + chunk * 5 * dim);

    __shared__ float inv_norm[kMaxChunk];

    const int e = blockIdx.x, head = blockIdx.y;
    const int col0 = blockIdx.z * p.cols;
    const int n_cols = min(p.cols, dim - col0);
    const int tid = threadIdx.x;
    const int col = tid / parts, part = tid % parts;  // (threads past the last column only wait and shuffle)
    const bool active = col < n_cols;
    const int first = p.first_rows[e], count = p.counts[e];
    const int64_t hoff = static_cast<int64_t>(head) * dim;
    float* mine = p.state + (static_cast<int64_t>(p.slots[e]) * p.n_heads + head) * dim * dim;

    load_chunk<scalar_t>(p, reinterpret_cast<scalar_t*>(raw_base), first, min(chunk, count), hoff, col0, n_cols);
    for (int i = tid; i < dim; i += blockDim.x) {
        offsets[i] = p.w0[hoff + i];
        offsets[dim + i] = p.a0[hoff + i];
    }
    float S[kRowsPerLane];
#pragma unroll
    for (int m = 0; m < kRowsPerLane; ++m) {
        const int i = part + m * parts;
        S[m] = active && i < dim ? mine[static_cast<int64_t>(i) * dim + col0 + col] : 0.0f;
    }

    int buffer = 0;
    for (int done = 0; done < count; done += chunk, buffer ^= 1) {
        const int n = min(chunk, count - done);
        const scalar_t* raw = reinterpret_cast<const scalar_t*>(raw_base + buffer * raw_bytes);
        // The next chunk sets out now; this one must have landed.
        if (done + chunk < count) {
            load_chunk<scalar_t>(p, reinterpret_cast<scalar_t*>(raw_base + (buffer ^ 1) * raw_bytes),
                                 first + done + chunk, min(chunk, count - done - chunk), hoff, col0, n_cols);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        prepare_chunk<scalar_t>(p, raw, vec, offsets, inv_norm, n, dim);
        // The tokens one after the other; nothing here waits for another warp.
        const scalar_t* raw_v = raw + chunk * 4 * dim;
        for (int c = 0; c < n; ++c) {
            const float* sk = vec + c * 5 * dim;
            const float* su = sk + dim;
            const float* sw = su + dim;
            const float* sau = sw + dim;
            const float* sr = sau + dim;
            const float vj = active ? pl_load(raw_v + c * p.cols + col) : 0.0f;
            // (two running sums each, rows of even and odd m: half as long a chain of additions)
            float dot = 0.0f, dot_odd = 0.0f;
#pragma unroll
            for (int m = 0; m < kRowsPerLane; m += 2) {
                const int i = part + m * parts;
                if (i < dim) {
                    dot = fmaf(su[i], S[m], dot);
                }
                if (i + parts < dim) {
                    dot_odd = fmaf(su[i + parts], S[m + 1], dot_odd);
                }
            }
            dot += dot_odd;
            for (int offset = parts >> 1; offset > 0; offset >>= 1) {
                dot += __shfl_xor_sync(0xffffffffu, dot, offset);
            }
            float o = 0.0f, o_odd = 0.0f;
#pragma unroll
            for (int m = 0; m < kRowsPerLane; m += 2) {
                const int i = part + m * parts;
                if (i < dim) {
                    S[m] = fmaf(sk[i], vj, fmaf(-sau[i], dot, sw[i] * S[m]));
                    o = fmaf(S[m], sr[i], o);
                }
                if (i + parts < dim) {
                    S[m + 1] = fmaf(sk[i + parts], vj, fmaf(-sau[i + parts], dot, sw[i + parts] * S[m + 1]));
                    o_odd = fmaf(S[m + 1], sr[i + parts], o_odd);
                }
            }
            o += o_odd;
            for (int offset = parts >> 1; offset > 0; offset >>= 1) {
                o += __shfl_xor_sync(0xffffffffu, o, offset);
            }
            if (active && part == 0) {
                p.o_raw[static_cast<int64_t>(first + done + c) * p.n_heads * dim + hoff + col0 + col] = o;
            }
        }
        __syncthreads();  // the vectors and this raw buffer are free again
    }
#pragma unroll
    for (int m = 0; m < kRowsPerLane; ++m) {
        const int i = part + m * parts;
        if (active && i < dim) {
            mine[static_cast<int64_t>(i) * dim + col0 + col] = S[m];
        }
    }
}

// The same scan with the head size and the lanes per column known to the compiler (the common
// head sizes): a lane holds ROWS consecutive rows of its column, reads its share of the five
// vectors with 16-byte loads and needs no index arithmetic per row. Its sums run in another
// order than the kernel above (a head size uses one of the two, always the same).
template <typename scalar_t, int DIM, int PARTS>
__global__ void __launch_bounds__(kMaxThreads) delta_rule_scan_static_kernel(const ScanParams p) {
    constexpr int ROWS = DIM / PARTS;
    static_assert(ROWS % 4 == 0 && ROWS * PARTS == DIM && PARTS <= 32, "rows per lane: a multiple of four");
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    const int chunk = p.chunk;
    float* offsets = reinterpret_cast<float*>(smem);
    float* vec = offsets + 2 * DIM;
    const int raw_elems = chunk * (4 * DIM + p.cols);
    const int raw_bytes = (raw_elems * static_cast<int>(sizeof(scalar_t)) + 15) / 16 * 16;
    float* o_part = vec + chunk * 5 * DIM;  // [chunk][threads]
    unsigned char* raw_base = reinterpret_cast<unsigned char*>(o_part + chunk * blockDim.x);
    __shared__ float inv_norm[kMaxChunk];

    const int e = blockIdx.x, head = blockIdx.y;
    const int col0 = blockIdx.z * p.cols;
    const int n_cols = min(p.cols, DIM - col0);
    const int tid = threadIdx.x;
    const int col = tid / PARTS, part = tid % PARTS;
    const bool active = col < n_cols;
    const int first = p.first_rows[e], count = p.counts[e];
    const int64_t hoff = static_cast<int64_t>(head) * DIM;
    float* mine = p.state + (static_cast<int64_t>(p.slots[e]) * p.n_heads + head) * DIM * DIM;

    load_chunk<scalar_t>(p, reinterpret_cast<scalar_t*>(raw_base), first, min(chunk, count), hoff, col0, n_cols);
    for (int i = tid; i < DIM; i += blockDim.x) {
        offsets[i] = p.w0[hoff + i];
        offsets[DIM + i] = p.a0[hoff + i];
    }
    float S[ROWS];
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
        S[m] = active ? mine[static_cast<int64_t>(part * ROWS + m) * DIM + col0 + col] : 0.0f;
    }

    int buffer = 0;
    for (int done = 0; done < count; done += chunk, buffer ^= 1) {
        const int n = min(chunk, count - done);
        const scalar_t* raw = reinterpret_cast<const scalar_t*>(raw_base + buffer * raw_bytes);
        if (done + chunk < count) {
            load_chunk<scalar_t>(p, reinterpret_cast<scalar_t*>(raw_base + (buffer ^ 1) * raw_bytes),
                                 first + done + chunk, min(chunk, count - done - chunk), hoff, col0, n_cols);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        prepare_chunk<scalar_t>(p, raw, vec, offsets, inv_norm, n, DIM);
        const scalar_t* raw_v = raw + chunk * 4 * DIM;
        // A lane's share of the five vectors of a token, fetched one token ahead of its use.
        float nk[ROWS], nu[ROWS], nw[ROWS], na[ROWS], nr[ROWS];
        auto fetch = [&](int c) {
            const float* token = vec + c * 5 * DIM + part * ROWS;
#pragma unroll
            for (int q = 0; q < ROWS / 4; ++q) {
                *reinterpret_cast<float4*>(nk + 4 * q) = *reinterpret_cast<const float4*>(token + 4 * q);
                *reinterpret_cast<float4*>(nu + 4 * q) = *reinterpret_cast<const float4*>(token + DIM + 4 * q);
                *reinterpret_cast<float4*>(nw + 4 * q) = *reinterpret_cast<const float4*>(token + 2 * DIM + 4 * q);
                *reinterpret_cast<float4*>(na + 4 * q) = *reinterpret_cast<const float4*>(token + 3 * DIM + 4 * q);
                *reinterpret_cast<float4*>(nr + 4 * q) = *reinterpret_cast<const float4*>(token + 4 * DIM + 4 * q);
            }
        };
        fetch(0);
        float nv = active ? pl_load(raw_v + col) : 0.0f;
        for (int c = 0; c < n; ++c) {
            float sk[ROWS], su[ROWS], sw[ROWS], sau[ROWS], sr[ROWS];
#pragma unroll
            for (int m = 0; m < ROWS; ++m) {
                sk[m] = nk[m];
                su[m] = nu[m];
                sw[m] = nw[m];
                sau[m] = na[m];
                sr[m] = nr[m];
            }
            const float vj = nv;
            if (c + 1 < n) {
                fetch(c + 1);
                nv = active ? pl_load(raw_v + (c + 1) * p.cols + col) : 0.0f;
            }
            float dot = 0.0f, dot_odd = 0.0f;
#pragma unroll
            for (int m = 0; m < ROWS; m += 2) {
                dot = fmaf(su[m], S[m], dot);
                dot_odd = fmaf(su[m + 1], S[m + 1], dot_odd);
            }
            dot += dot_odd;
#pragma unroll
            for (int offset = PARTS >> 1; offset > 0; offset >>= 1) {
                dot += __shfl_xor_sync(0xffffffffu, dot, offset);
            }
            float o = 0.0f, o_odd = 0.0f;
#pragma unroll
            for (int m = 0; m < ROWS; m += 2) {
                S[m] = fmaf(sk[m], vj, fmaf(-sau[m], dot, sw[m] * S[m]));
                o = fmaf(S[m], sr[m], o);
                S[m + 1] = fmaf(sk[m + 1], vj, fmaf(-sau[m + 1], dot, sw[m + 1] * S[m + 1]));
                o_odd = fmaf(S[m + 1], sr[m + 1], o_odd);
            }
            // The lanes' shares of o wait in shared memory; they are added up after the chunk,
            // off the path from one token to the next.
            o_part[c * blockDim.x + tid] = o + o_odd;
        }
        __syncwarp();  // (a column's lanes sit in one warp)
        for (int c = part; c < n; c += PARTS) {
            const float* shares = o_part + c * blockDim.x + col * PARTS;
            float o = shares[0];
#pragma unroll
            for (int q = 1; q < PARTS; ++q) {
                o += shares[q];
            }
            if (active) {
                p.o_raw[static_cast<int64_t>(first + done + c) * p.n_heads * DIM + hoff + col0 + col] = o;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
        if (active) {
            mine[static_cast<int64_t>(part * ROWS + m) * DIM + col0 + col] = S[m];
        }
    }
}

template <typename scalar_t, int DIM, int PARTS>
void launch_scan_static(const ScanParams& p, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(delta_rule_scan_static_kernel<scalar_t, DIM, PARTS>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    }
    pl_launch_overlapped(delta_rule_scan_static_kernel<scalar_t, DIM, PARTS>, grid, dim3(threads), smem, stream, p);
}

template <typename scalar_t>
void launch_scan(const ScanParams& p, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
    if (p.dim == 128 && p.parts == 16) {
        launch_scan_static<scalar_t, 128, 16>(p, grid, threads, smem, stream);
    } else if (p.dim == 64 && p.parts == 8) {
        launch_scan_static<scalar_t, 64, 8>(p, grid, threads, smem, stream);
    } else if (p.dim == 32 && p.parts == 4) {
        launch_scan_static<scalar_t, 32, 4>(p, grid, threads, smem, stream);
    } else if (p.dim == 16 && p.parts == 2) {
        launch_scan_static<scalar_t, 16, 2>(p, grid, threads, smem, stream);
    } else {
        if (smem > 48 * 1024) {
            cudaFuncSetAttribute(delta_rule_scan_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        }
        pl_launch_overlapped(delta_rule_scan_kernel<scalar_t>, grid, dim3(threads), smem, stream, p);
    }
}

// A warp per (token, head): out = o * rsqrt(mean(o^2) + eps) * norm * sigmoid(g).
template <typename scalar_t>
__global__ void delta_rule_finish_kernel(const float* __restrict__ o_raw, const scalar_t* __restrict__ g,
                                         int64_t g_row_stride, const float* __restrict__ norm,
                                         scalar_t* __restrict__ out, int64_t out_row_stride, int n_tokens, int n_heads,
                                         int dim, float eps) {
    pl_grid_trigger();
    pl_grid_wait();
    const int lane = threadIdx.x & 31;
    const int64_t pair = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= static_cast<int64_t>(n_tokens) * n_heads) {
        return;
    }
    const int64_t t = pair / n_heads;
    const int64_t hoff = (pair % n_heads) * dim;
    const float* o = o_raw + t * n_heads * dim + hoff;
    float square = 0.0f;
    for (int i = lane; i < dim; i += 32) {
        square += o[i] * o[i];
    }
    const float inv = 1.0f / sqrtf(pl_warp_sum(square) / static_cast<float>(dim) + eps);
    for (int i = lane; i < dim; i += 32) {
        pl_store(out + t * out_row_stride + hoff + i,
                 o[i] * inv * norm[hoff + i] * sigmoid_f32(pl_load(g + t * g_row_stride + hoff + i)));
    }
}

}  // namespace

// r, k, v, g, a_pre: [T, heads * dim] in the engine's dtype with `row_stride` elements
// between rows (columns of one projection output); w_pre likewise with w_row_stride. w0,
// a0, norm fp32 [heads * dim]. state fp32 [slots, heads, dim, dim] (key channel, value
// channel), updated in place. first_rows, counts, slots: int32 [entries]; the entries' rows
// cover all n_tokens rows. o_raw: fp32 scratch [n_tokens, heads * dim]. out [T, heads * dim]
// in the engine's dtype.
PL_API int pl_delta_rule(const void* r, const void* k, const void* v, const void* g, const void* a_pre,
                         int64_t row_stride, const void* w_pre, int64_t w_row_stride, const float* w0,
                         const float* a0, const float* norm, float* state, const int32_t* first_rows,
                         const int32_t* counts, const int32_t* slots, float* o_raw, void* out, int64_t out_row_stride,
                         int n_tokens, int n_entries, int n_heads, int dim, float decay_scale, float unit_eps,
                         float eps, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_entries >= 0 && n_tokens >= 0 && n_heads > 0 && dim > 0,
               "delta_rule: bad sizes tokens=%d entries=%d heads=%d dim=%d", n_tokens, n_entries, n_heads, dim);
    PL_REQUIRE(n_heads <= 65535 && dim <= 32 * kRowsPerLane, "delta_rule: %d heads of size %d are too many or too "
               "large (head size at most %d)", n_heads, dim, 32 * kRowsPerLane);
    if (n_entries == 0 || n_tokens == 0) {
        return 0;
    }
    // Lanes per column: the least power of two that leaves a lane eight rows or fewer (at most a
    // warp: kRowsPerLane rows then). Short chains of additions per token are what the scan's
    // time is made of.
    int parts = 1;
    while (parts < 32 && (dim + parts - 1) / parts > 8) {
        parts *= 2;
    }
    // Columns per CTA: all of the head's where a CTA holds them (the CTAs of one head repeat the
    // work between chunks), else as many as it holds.
    int cols = kMaxThreads / parts > dim ? dim : kMaxThreads / parts;
    // Half of that where a head then still fills a warp per scheduler: two CTAs per head on two SMs
    // issue a token's instructions in half the time, and what they both do between chunks is small.
    if (cols == dim && cols * parts > 256 && cols % 2 == 0) {
        cols /= 2;
    }
    const int width = dtype == PL_F32 ? 4 : 2;
    if ((cols * width) % 16 != 0 && cols < dim) {
        int wider = (cols * width + 15) / 16 * 16 / width;  // (blocks of columns that start on 16 bytes)
        wider = wider > dim ? dim : wider;
        if (wider * parts <= kMaxThreads) {
            cols = wider;
        }
    }
    PL_REQUIRE(cols * parts <= kMaxThreads || cols == 1, "delta_rule: head size %d does not fit a CTA", dim);
    const int col_blocks = (dim + cols - 1) / cols;
    ScanParams p;
    p.r = r; p.k = k; p.v = v; p.a_pre = a_pre; p.row_stride = row_stride;
    p.w_pre = w_pre; p.w_row_stride = w_row_stride; p.w0 = w0; p.a0 = a0; p.state = state;
    p.first_rows = first_rows; p.counts = counts; p.slots = slots; p.o_raw = o_raw;
    p.n_heads = n_heads; p.dim = dim; p.parts = parts; p.cols = cols;
    p.chunk = dim <= 64 ? 16 : dim <= 128 ? 8 : 4;
    p.decay_scale = decay_scale; p.unit_eps = unit_eps;
    auto aligned = [&](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    p.async_loads = (dim * width) % 16 == 0 && (cols * width) % 16 == 0 && (row_stride * width) % 16 == 0 &&
        (w_row_stride * width) % 16 == 0 && aligned(r) && aligned(k) && aligned(v) && aligned(a_pre) && aligned(w_pre);
    const int raw_bytes = (p.chunk * (4 * dim + cols) * width + 15) / 16 * 16;
    int threads = (cols * parts + 31) / 32 * 32;
    // (offsets, a chunk's vectors, the lanes' shares of o, two buffers of raw projections)
    const size_t smem = static_cast<size_t>(2 * dim + p.chunk * 5 * dim + p.chunk * threads) * sizeof(float) +
        2 * raw_bytes;
    const dim3 grid(n_entries, n_heads, col_blocks);
    PL_DISPATCH_DTYPE(dtype, "delta_rule", {
        launch_scan<scalar_t>(p, grid, threads, smem, stream);
        PL_CHECK_LAUNCH("delta_rule");
        const int64_t pairs = static_cast<int64_t>(n_tokens) * n_heads;
        pl_launch_overlapped(delta_rule_finish_kernel<scalar_t>, dim3(static_cast<unsigned>((pairs + 3) / 4)), dim3(128),
                             0, stream, static_cast<const float*>(o_raw), static_cast<const scalar_t*>(g), row_stride,
                             norm, static_cast<scalar_t*>(out), out_row_stride, n_tokens, n_heads, dim, eps);
    });
    PL_CHECK_LAUNCH("delta_rule_finish");
    return 0;
}
