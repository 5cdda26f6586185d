// The gated delta rule with a decay per key channel: a recurrent mixer whose state per head
// is a matrix S [dim, vdim] (key channel x value channel) kept in fp32 from token to token.
//
//   q^ = q / sqrt(|q|^2 + unit_eps) * q_scale,  k^ = k / sqrt(|k|^2 + unit_eps)      per q/k head
//   g  = exp(-exp(A_h) * softplus(a~ + dt_bias))                                      per head and key channel
//   b  = sigmoid(b~)                                                                  per head
//   S <- diag(g) S;  u = b * (v - S^T k^);  S <- S + k^ u^T;  o = S^T q^               (o reads the new S)
//   out = o * rsqrt(mean(o^2) + eps) * norm * sigmoid(gate~)                          per head over vdim
//
// q, k, v arrive filtered and activated (the engine's dtype), a~, b~ and gate~ as projected;
// everything above is fp32. Head h reads q/k head h / (heads / qk_heads).
//
// The scan: a CTA per (batch entry, head, block of value columns) walks the entry's rows in
// order. A column of S never meets another column, so each column lives in registers:
// `parts` neighbouring lanes share a column and each holds every parts-th of its rows. The
// rows are taken in chunks: while one chunk is worked on, the next chunk's projections
// arrive in shared memory (cp.async); all threads turn a chunk's projections into the fp32
// vectors q^, k^, g and the scalar b (the unit factors by a warp per token, the
// exponentials one (token, channel) per thread), then the tokens update the state one after
// the other with nothing but the shuffles among a column's lanes between them. The raw o
// goes to scratch in fp32; a second kernel norms it per head, applies the norm's weight and
// the gate and rounds once. The order of every sum depends on the sizes alone, so a token's
// result depends on the tokens before it only: not on how the prompt was cut, on the chunks
// or on the rest of the batch.
#include "common.cuh"

#include "mma_helpers.cuh"

namespace {

constexpr int kRows = 16;      // rows of a column one lane holds at most
constexpr int kChunkMost = 16;

struct GatedDeltaParams {
    const void* q;
    const void* k;
    const void* v;
    int64_t qkv_stride;
    const void* b_pre;
    int64_t b_stride;
    const void* a_pre;
    int64_t a_stride;
    const float* a_log;
    const float* dt_bias;
    float* state;
    const int32_t* first_rows;
    const int32_t* counts;
    const int32_t* slots;
    float* o_raw;
    int n_heads, qk_heads, dim, vdim, parts, cols, chunk;
    int async_loads;  // every row of every operand starts on 16 bytes
    float unit_eps, q_scale;
};

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// One chunk's projections -> shared memory: [token][q, k, a~][dim], then [token][cols] of v.
template <typename scalar_t>
__device__ __forceinline__ void load_chunk(const GatedDeltaParams& p, scalar_t* raw, const scalar_t* q,
                                           const scalar_t* k, const scalar_t* a_pre, const scalar_t* v, int64_t t0,
                                           int n, int n_cols) {
    const int dim = p.dim;
    scalar_t* raw_v = raw + p.chunk * 3 * dim;
    if (p.async_loads) {
        constexpr int kPer = 16 / sizeof(scalar_t);
        const int gv = dim / kPer, gc = p.cols / kPer;
        const int per_token = 3 * gv + gc;
        for (int idx = threadIdx.x; idx < n * per_token; idx += blockDim.x) {
            const int c = idx / per_token, g = idx % per_token;
            if (g < 3 * gv) {
                const int which = g / gv, e = (g % gv) * kPer;
                const scalar_t* src = which == 0 ? q + (t0 + c) * p.qkv_stride
                                    : which == 1 ? k + (t0 + c) * p.qkv_stride : a_pre + (t0 + c) * p.a_stride;
                cp_async_16(raw + (c * 3 + which) * dim + e, src + e);
            } else {
                const int e = (g - 3 * gv) * kPer;
                if (e < n_cols) {  // (n_cols is a multiple of kPer here)
                    cp_async_16(raw_v + c * p.cols + e, v + (t0 + c) * p.qkv_stride + e);
                }
            }
        }
    } else {
        const int per_token = 3 * dim + n_cols;
        for (int idx = threadIdx.x; idx < n * per_token; idx += blockDim.x) {
            const int c = idx / per_token, g = idx % per_token;
            if (g < 3 * dim) {
                const int which = g / dim, e = g % dim;
                const scalar_t* src = which == 0 ? q + (t0 + c) * p.qkv_stride
                                    : which == 1 ? k + (t0 + c) * p.qkv_stride : a_pre + (t0 + c) * p.a_stride;
                raw[(c * 3 + which) * dim + e] = src[e];
            } else {
                const int e = g - 3 * dim;
                raw_v[c * p.cols + e] = v[(t0 + c) * p.qkv_stride + e];
            }
        }
    }
    cp_async_commit();
}

// The same by `threads` threads numbered `tid` (one half of a CTA), with the sizes given.
template <typename scalar_t>
__device__ __forceinline__ void load_chunk_by(const GatedDeltaParams& p, scalar_t* raw, const scalar_t* q,
                                              const scalar_t* k, const scalar_t* a_pre, const scalar_t* v, int64_t t0,
                                              int n, int n_cols, int tid, int threads, int dim, int cols) {
    scalar_t* raw_v = raw + p.chunk * 3 * dim;
    if (p.async_loads) {
        constexpr int kPer = 16 / sizeof(scalar_t);
        const int gv = dim / kPer, gc = cols / kPer;
        const int per_token = 3 * gv + gc;
        for (int idx = tid; idx < n * per_token; idx += threads) {
            const int c = idx / per_token, g = idx % per_token;
            if (g < 3 * gv) {
                const int which = g / gv, e = (g % gv) * kPer;
                const scalar_t* src = which == 0 ? q + (t0 + c) * p.qkv_stride
                                    : which == 1 ? k + (t0 + c) * p.qkv_stride : a_pre + (t0 + c) * p.a_stride;
                cp_async_16(raw + (c * 3 + which) * dim + e, src + e);
            } else {
                const int e = (g - 3 * gv) * kPer;
                if (e < n_cols) {
                    cp_async_16(raw_v + c * cols + e, v + (t0 + c) * p.qkv_stride + e);
                }
            }
        }
    } else {
        const int per_token = 3 * dim + cols;
        for (int idx = tid; idx < n * per_token; idx += threads) {
            const int c = idx / per_token, g = idx % per_token;
            if (g < 3 * dim) {
                const int which = g / dim, e = g % dim;
                const scalar_t* src = which == 0 ? q + (t0 + c) * p.qkv_stride
                                    : which == 1 ? k + (t0 + c) * p.qkv_stride : a_pre + (t0 + c) * p.a_stride;
                raw[(c * 3 + which) * dim + e] = src[e];
            } else {
                const int e = g - 3 * dim;
                if (e < n_cols) {
                    raw_v[c * cols + e] = v[(t0 + c) * p.qkv_stride + e];
                }
            }
        }
    }
    cp_async_commit();
}

template <typename scalar_t>
__global__ void __launch_bounds__(512) gated_delta_scan_kernel(const GatedDeltaParams p) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    const int dim = p.dim, parts = p.parts, chunk = p.chunk, cols = p.cols;
    float* sq = reinterpret_cast<float*>(smem);  // [chunk][dim]
    float* sk = sq + chunk * dim;       // [chunk][dim]
    float* sg = sk + chunk * dim;       // [chunk][dim]
    float* sb = sg + chunk * dim;       // [chunk]
    float* inv_q = sb + chunk;          // [chunk]
    float* inv_k = inv_q + chunk;       // [chunk]
    float* bias = sq + (chunk * (3 * dim + 3) + 3) / 4 * 4;  // [dim], on 16 bytes like the buffers after it
    // then two buffers of a chunk's projections as they arrive
    const int raw_elems = chunk * (3 * dim + cols);
    const int raw_bytes = (raw_elems * static_cast<int>(sizeof(scalar_t)) + 15) / 16 * 16;
    unsigned char* raw_base = reinterpret_cast<unsigned char*>(bias + ((dim + 3) / 4) * 4);

    const int e = blockIdx.x, head = blockIdx.y;
    const int qk_head = head / (p.n_heads / p.qk_heads);
    const int col0 = blockIdx.z * cols;
    const int n_cols = min(cols, p.vdim - col0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    const int col = tid / parts, part = tid % parts;
    const bool active = col < n_cols;
    const int first = p.first_rows[e], count = p.counts[e];
    const scalar_t* q = static_cast<const scalar_t*>(p.q) + static_cast<int64_t>(qk_head) * dim;
    const scalar_t* k = static_cast<const scalar_t*>(p.k) + static_cast<int64_t>(qk_head) * dim;
    const scalar_t* v = static_cast<const scalar_t*>(p.v) + static_cast<int64_t>(head) * p.vdim + col0;
    const scalar_t* a_pre = static_cast<const scalar_t*>(p.a_pre) + static_cast<int64_t>(head) * dim;
    const scalar_t* b_pre = static_cast<const scalar_t*>(p.b_pre) + head;
    const float rate = expf(p.a_log[head]);
    float* mine = p.state + ((static_cast<int64_t>(p.slots[e]) * p.n_heads + head) * dim) * p.vdim + col0;

    load_chunk<scalar_t>(p, reinterpret_cast<scalar_t*>(raw_base), q, k, a_pre, v, first, min(chunk, count), n_cols);
    for (int i = tid; i < dim; i += blockDim.x) {
        bias[i] = p.dt_bias[static_cast<int64_t>(head) * dim + i];
    }
    float S[kRows];
#pragma unroll
    for (int m = 0; m < kRows; ++m) {
        const int i = part + m * parts;
        S[m] = active && i < dim ? mine[static_cast<int64_t>(i) * p.vdim + col] : 0.0f;
    }

    int buffer = 0;
    for (int done = 0; done < count; done += chunk, buffer ^= 1) {
        const int n = min(chunk, count - done);
        const int64_t t0 = first + done;
        const scalar_t* raw = reinterpret_cast<const scalar_t*>(raw_base + buffer * raw_bytes);
        // The next chunk sets out now (its buffer was last read two chunks ago); this one must have landed.
        __syncthreads();
        if (done + chunk < count) {
            load_chunk<scalar_t>(p, reinterpret_cast<scalar_t*>(raw_base + (buffer ^ 1) * raw_bytes), q, k, a_pre, v,
                                 t0 + chunk, min(chunk, count - done - chunk), n_cols);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        for (int c = warp; c < n; c += warps) {
            float b = 0.0f;
            if (lane == 0) {
                b = pl_load(b_pre + (t0 + c) * p.b_stride);
            }
            const scalar_t* qr = raw + (c * 3) * dim;
            const scalar_t* kr = qr + dim;
            float qq = 0.0f, kk = 0.0f;
            for (int i = lane; i < dim; i += 32) {
                const float x = pl_load(qr + i), y = pl_load(kr + i);
                qq = fmaf(x, x, qq);
                kk = fmaf(y, y, kk);
            }
            qq = pl_warp_sum(qq);
            kk = pl_warp_sum(kk);
            if (lane == 0) {
                inv_q[c] = p.q_scale / sqrtf(qq + p.unit_eps);
                inv_k[c] = 1.0f / sqrtf(kk + p.unit_eps);
                sb[c] = 1.0f / (1.0f + expf(-b));
            }
        }
        __syncthreads();
        for (int idx = tid; idx < n * dim; idx += blockDim.x) {
            const int c = idx / dim, i = idx - c * dim;
            const scalar_t* token = raw + c * 3 * dim;
            sq[idx] = pl_load(token + i) * inv_q[c];
            sk[idx] = pl_load(token + dim + i) * inv_k[c];
            sg[idx] = expf(-rate * softplus_f32(pl_load(token + 2 * dim + i) + bias[i]));
        }
        __syncthreads();
        const scalar_t* raw_v = raw + chunk * 3 * dim;
        for (int c = 0; c < n; ++c) {
            const float* kq = sq + c * dim;
            const float* kk = sk + c * dim;
            const float* kg = sg + c * dim;
            const float vj = active ? pl_load(raw_v + c * cols + col) : 0.0f;
            float dot0 = 0.0f, dot1 = 0.0f;
#pragma unroll
            for (int m = 0; m < kRows; m += 2) {
                const int i = part + m * parts, i2 = i + parts;
                if (i < dim) {
                    S[m] *= kg[i];
                    dot0 = fmaf(S[m], kk[i], dot0);
                }
                if (i2 < dim) {
                    S[m + 1] *= kg[i2];
                    dot1 = fmaf(S[m + 1], kk[i2], dot1);
                }
            }
            float dot = dot0 + dot1;
            for (int offset = parts >> 1; offset > 0; offset >>= 1) {
                dot += __shfl_xor_sync(0xffffffffu, dot, offset);
            }
            const float u = sb[c] * (vj - dot);
            float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
            for (int m = 0; m < kRows; m += 2) {
                const int i = part + m * parts, i2 = i + parts;
                if (i < dim) {
                    S[m] = fmaf(kk[i], u, S[m]);
                    o0 = fmaf(S[m], kq[i], o0);
                }
                if (i2 < dim) {
                    S[m + 1] = fmaf(kk[i2], u, S[m + 1]);
                    o1 = fmaf(S[m + 1], kq[i2], o1);
                }
            }
            float o = o0 + o1;
            for (int offset = parts >> 1; offset > 0; offset >>= 1) {
                o += __shfl_xor_sync(0xffffffffu, o, offset);
            }
            if (active && part == 0) {
                p.o_raw[(t0 + c) * (static_cast<int64_t>(p.n_heads) * p.vdim) + static_cast<int64_t>(head) * p.vdim +
                        col0 + col] = o;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < kRows; ++m) {
        const int i = part + m * parts;
        if (active && i < dim) {
            mine[static_cast<int64_t>(i) * p.vdim + col] = S[m];
        }
    }
}

// The same scan with the key size and the lanes per column known to the compiler, and with the
// work split between two halves of the CTA: warps 0 to 3 hold the state's columns (a lane holds
// DIM / PARTS = 8 consecutive rows of its column, reads its share of q^, k^ and g with 16-byte
// loads one token ahead of the token whose chain it is in) and do nothing but the tokens'
// updates, one chunk after the other; warps 4 to 7 meanwhile make the next chunk ready: they
// ask for the chunk after it (cp.async), turn the one that has arrived into the fp32 vectors
// (the unit factors by a few lanes per token, all of a chunk's tokens at once; the
// exponentials one (token, channel) per thread) and leave them in the other of two buffers.
// The halves meet once a chunk. What bounds the scan is then the chain of one token's update
// alone. (A lane's rows differ from the kernel above, so the sums' order does; which kernel
// runs depends on the sizes alone.)
template <typename scalar_t, int DIM, int PARTS>
__global__ void __launch_bounds__(256, 1) gated_delta_scan_static_kernel(const GatedDeltaParams p) {
    pl_grid_trigger();
    pl_grid_wait();
    constexpr int R = DIM / PARTS;      // rows per lane
    constexpr int COLS = 128 / PARTS;   // value columns per CTA
    static_assert(R % 4 == 0 && R <= kRows, "a lane holds a multiple of four rows");
    extern __shared__ __align__(16) unsigned char smem[];
    const int chunk = p.chunk;
    // two buffers of a chunk's vectors: [chunk][DIM] q^, k^, g, [chunk][COLS] v, [chunk] b (rounded up to 4 floats)
    const int vec_floats = (chunk * (3 * DIM + COLS + 1) + 3) / 4 * 4;
    float* vec_base = reinterpret_cast<float*>(smem);
    float* inv_q = vec_base + 2 * vec_floats;   // [chunk]
    float* inv_k = inv_q + chunk;               // [chunk]
    float* bias = inv_q + (2 * chunk + 3) / 4 * 4;  // [DIM]
    const int raw_elems = chunk * (3 * DIM + COLS);
    const int raw_bytes = (raw_elems * static_cast<int>(sizeof(scalar_t)) + 15) / 16 * 16;
    unsigned char* raw_base = reinterpret_cast<unsigned char*>(bias + DIM);

    const int e = blockIdx.x, head = blockIdx.y;
    const int qk_head = head / (p.n_heads / p.qk_heads);
    const int col0 = blockIdx.z * COLS;
    const int n_cols = min(COLS, p.vdim - col0);
    const int tid = threadIdx.x;
    const bool producer = tid >= 128;
    const int first = p.first_rows[e], count = p.counts[e];
    const int n_chunks = (count + chunk - 1) / chunk;
    const scalar_t* q = static_cast<const scalar_t*>(p.q) + static_cast<int64_t>(qk_head) * DIM;
    const scalar_t* k = static_cast<const scalar_t*>(p.k) + static_cast<int64_t>(qk_head) * DIM;
    const scalar_t* v = static_cast<const scalar_t*>(p.v) + static_cast<int64_t>(head) * p.vdim + col0;
    const scalar_t* a_pre = static_cast<const scalar_t*>(p.a_pre) + static_cast<int64_t>(head) * DIM;
    const scalar_t* b_pre = static_cast<const scalar_t*>(p.b_pre) + head;

    // ---- the consumers' state
    const int col = tid / PARTS, part = tid % PARTS;
    const bool active = !producer && col < n_cols;
    float* mine = p.state + ((static_cast<int64_t>(p.slots[e]) * p.n_heads + head) * DIM) * p.vdim + col0;
    float S[R];
#pragma unroll
    for (int m = 0; m < R; ++m) {
        S[m] = active ? mine[static_cast<int64_t>(part * R + m) * p.vdim + col] : 0.0f;
    }
    // ---- the producers' constants
    const int ptid = tid - 128;
    const float rate = expf(p.a_log[head]);
    if (producer) {
        for (int i = ptid; i < DIM; i += 128) {
            bias[i] = p.dt_bias[static_cast<int64_t>(head) * DIM + i];
        }
        if (n_chunks > 0) {
            load_chunk_by<scalar_t>(p, reinterpret_cast<scalar_t*>(raw_base), q, k, a_pre, v, first, min(chunk, count),
                                    n_cols, ptid, 128, DIM, COLS);
        }
    }
    // lanes per token for the unit factors: all of a chunk's tokens at once
    const int group = min(32, 128 / chunk);

    for (int i = -1; i < n_chunks; ++i) {
        if (producer) {
            const int next = i + 1;
            if (next < n_chunks) {
                const int n = min(chunk, count - next * chunk);
                const int64_t t0 = first + static_cast<int64_t>(next) * chunk;
                if (next + 1 < n_chunks) {
                    load_chunk_by<scalar_t>(p, reinterpret_cast<scalar_t*>(raw_base + ((next + 1) & 1) * raw_bytes), q, k,
                                            a_pre, v, t0 + chunk, min(chunk, count - (next + 1) * chunk), n_cols, ptid,
                                            128, DIM, COLS);
                    cp_async_wait<1>();
                } else {
                    cp_async_wait<0>();
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const scalar_t* raw = reinterpret_cast<const scalar_t*>(raw_base + (next & 1) * raw_bytes);
                float* sq = vec_base + (next & 1) * vec_floats;
                float* sk = sq + chunk * DIM;
                float* sg = sk + chunk * DIM;
                float* sv = sg + chunk * DIM;
                float* sb = sv + chunk * COLS;
                {
                    const int c = ptid / group, sub = ptid % group;
                    float qq = 0.0f, kk = 0.0f, b = 0.0f;
                    if (c < n) {
                        if (sub == 0) {
                            b = pl_load(b_pre + (t0 + c) * p.b_stride);
                        }
                        const scalar_t* qr = raw + (c * 3) * DIM;
                        const scalar_t* kr = qr + DIM;
                        for (int j = sub; j < DIM; j += group) {
                            const float x = pl_load(qr + j), y = pl_load(kr + j);
                            qq = fmaf(x, x, qq);
                            kk = fmaf(y, y, kk);
                        }
                    }
                    for (int offset = group >> 1; offset > 0; offset >>= 1) {
                        qq += __shfl_xor_sync(0xffffffffu, qq, offset);
                        kk += __shfl_xor_sync(0xffffffffu, kk, offset);
                    }
                    if (c < n && sub == 0) {
                        inv_q[c] = p.q_scale / sqrtf(qq + p.unit_eps);
                        inv_k[c] = 1.0f / sqrtf(kk + p.unit_eps);
                        sb[c] = 1.0f / (1.0f + expf(-b));
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                for (int idx = ptid; idx < n * DIM; idx += 128) {
                    const int c = idx / DIM, j = idx - c * DIM;
                    const scalar_t* token = raw + c * 3 * DIM;
                    sq[idx] = pl_load(token + j) * inv_q[c];
                    sk[idx] = pl_load(token + DIM + j) * inv_k[c];
                    sg[idx] = expf(-rate * softplus_f32(pl_load(token + 2 * DIM + j) + bias[j]));
                }
                const scalar_t* raw_v = raw + chunk * 3 * DIM;
                for (int idx = ptid; idx < n * COLS; idx += 128) {
                    const int j = idx % COLS;
                    sv[idx] = j < n_cols ? pl_load(raw_v + idx) : 0.0f;
                }
            }
        } else if (i >= 0) {
            const int n = min(chunk, count - i * chunk);
            const int64_t t0 = first + static_cast<int64_t>(i) * chunk;
            const float* sq = vec_base + (i & 1) * vec_floats;
            const float* sk = sq + chunk * DIM;
            const float* sg = sk + chunk * DIM;
            const float* sv = sg + chunk * DIM;
            const float* sb = sv + chunk * COLS;
            // this lane's share of the vectors, one token ahead
            float4 nq[R / 4], nk[R / 4], ng[R / 4];
            float nv, nb;
            auto fetch = [&](int c) {
                const float4* q4 = reinterpret_cast<const float4*>(sq + c * DIM + part * R);
                const float4* k4 = reinterpret_cast<const float4*>(sk + c * DIM + part * R);
                const float4* g4 = reinterpret_cast<const float4*>(sg + c * DIM + part * R);
#pragma unroll
                for (int j = 0; j < R / 4; ++j) {
                    nq[j] = q4[j];
                    nk[j] = k4[j];
                    ng[j] = g4[j];
                }
                nv = sv[c * COLS + col];
                nb = sb[c];
            };
            fetch(0);
            for (int c = 0; c < n; ++c) {
                float kq[R], kk[R], kg[R];
#pragma unroll
                for (int j = 0; j < R / 4; ++j) {
                    kq[4 * j] = nq[j].x; kq[4 * j + 1] = nq[j].y; kq[4 * j + 2] = nq[j].z; kq[4 * j + 3] = nq[j].w;
                    kk[4 * j] = nk[j].x; kk[4 * j + 1] = nk[j].y; kk[4 * j + 2] = nk[j].z; kk[4 * j + 3] = nk[j].w;
                    kg[4 * j] = ng[j].x; kg[4 * j + 1] = ng[j].y; kg[4 * j + 2] = ng[j].z; kg[4 * j + 3] = ng[j].w;
                }
                const float vj = nv, beta = nb;
                if (c + 1 < n) {
                    fetch(c + 1);
                }
                float dot0 = 0.0f, dot1 = 0.0f;
#pragma unroll
                for (int m = 0; m < R; m += 2) {
                    S[m] *= kg[m];
                    dot0 = fmaf(S[m], kk[m], dot0);
                    S[m + 1] *= kg[m + 1];
                    dot1 = fmaf(S[m + 1], kk[m + 1], dot1);
                }
                float dot = dot0 + dot1;
#pragma unroll
                for (int offset = PARTS >> 1; offset > 0; offset >>= 1) {
                    dot += __shfl_xor_sync(0xffffffffu, dot, offset);
                }
                const float u = beta * (vj - dot);
                float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
                for (int m = 0; m < R; m += 2) {
                    S[m] = fmaf(kk[m], u, S[m]);
                    o0 = fmaf(S[m], kq[m], o0);
                    S[m + 1] = fmaf(kk[m + 1], u, S[m + 1]);
                    o1 = fmaf(S[m + 1], kq[m + 1], o1);
                }
                float o = o0 + o1;
#pragma unroll
                for (int offset = PARTS >> 1; offset > 0; offset >>= 1) {
                    o += __shfl_xor_sync(0xffffffffu, o, offset);
                }
                if (active && part == 0) {
                    p.o_raw[(t0 + c) * (static_cast<int64_t>(p.n_heads) * p.vdim) + static_cast<int64_t>(head) * p.vdim +
                            col0 + col] = o;
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int m = 0; m < R; ++m) {
        if (active) {
            mine[static_cast<int64_t>(part * R + m) * p.vdim + col] = S[m];
        }
    }
}

// The form for steps that bring a token or two per entry (steps of single tokens): the same
// arithmetic by one half alone, 128 threads that make a chunk ready and then walk it. There is
// nothing to overlap in such a step, and three of these CTAs fit where one of the above does.
// Same products and sums in the same order as the kernel above: a token's result does not depend
// on which of the two ran.
template <typename scalar_t, int DIM, int PARTS>
__global__ void __launch_bounds__(128) gated_delta_scan_static_single_kernel(const GatedDeltaParams p) {
    pl_grid_trigger();
    pl_grid_wait();
    constexpr int R = DIM / PARTS;  // rows per lane
    static_assert(R % 4 == 0 && R <= kRows, "a lane holds a multiple of four rows");
    extern __shared__ __align__(16) unsigned char smem[];
    const int chunk = p.chunk, cols = p.cols;
    float* sq = reinterpret_cast<float*>(smem);
    float* sk = sq + chunk * DIM;
    float* sg = sk + chunk * DIM;
    float* sb = sg + chunk * DIM;
    float* inv_q = sb + chunk;
    float* inv_k = inv_q + chunk;
    float* bias = sq + (chunk * (3 * DIM + 3) + 3) / 4 * 4;
    const int raw_elems = chunk * (3 * DIM + cols);
    const int raw_bytes = (raw_elems * static_cast<int>(sizeof(scalar_t)) + 15) / 16 * 16;
    unsigned char* raw_base = reinterpret_cast<unsigned char*>(bias + DIM);

    const int e = blockIdx.x, head = blockIdx.y;
    const int qk_head = head / (p.n_heads / p.qk_heads);
    const int col0 = blockIdx.z * cols;
    const int n_cols = min(cols, p.vdim - col0);
    const int tid = threadIdx.x;
    const int col = tid / PARTS, part = tid % PARTS;
    const bool active = col < n_cols;
    const int first = p.first_rows[e], count = p.counts[e];
    const scalar_t* q = static_cast<const scalar_t*>(p.q) + static_cast<int64_t>(qk_head) * DIM;
    const scalar_t* k = static_cast<const scalar_t*>(p.k) + static_cast<int64_t>(qk_head) * DIM;
    const scalar_t* v = static_cast<const scalar_t*>(p.v) + static_cast<int64_t>(head) * p.vdim + col0;
    const scalar_t* a_pre = static_cast<const scalar_t*>(p.a_pre) + static_cast<int64_t>(head) * DIM;
    const scalar_t* b_pre = static_cast<const scalar_t*>(p.b_pre) + head;
    const float rate = expf(p.a_log[head]);
    float* mine = p.state + ((static_cast<int64_t>(p.slots[e]) * p.n_heads + head) * DIM) * p.vdim + col0;

    load_chunk<scalar_t>(p, reinterpret_cast<scalar_t*>(raw_base), q, k, a_pre, v, first, min(chunk, count), n_cols);
    for (int i = tid; i < DIM; i += blockDim.x) {
        bias[i] = p.dt_bias[static_cast<int64_t>(head) * DIM + i];
    }
    float S[R];
#pragma unroll
    for (int m = 0; m < R; ++m) {
        S[m] = active ? mine[static_cast<int64_t>(part * R + m) * p.vdim + col] : 0.0f;
    }

    int buffer = 0;
    for (int done = 0; done < count; done += chunk, buffer ^= 1) {
        const int n = min(chunk, count - done);
        const int64_t t0 = first + done;
        const scalar_t* raw = reinterpret_cast<const scalar_t*>(raw_base + buffer * raw_bytes);
        __syncthreads();
        if (done + chunk < count) {
            load_chunk<scalar_t>(p, reinterpret_cast<scalar_t*>(raw_base + (buffer ^ 1) * raw_bytes), q, k, a_pre, v,
                                 t0 + chunk, min(chunk, count - done - chunk), n_cols);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        {
            const int group = min(32, 128 / chunk);
            const int c = tid / group, sub = tid % group;
            float qq = 0.0f, kk = 0.0f, b = 0.0f;
            if (c < n) {
                if (sub == 0) {
                    b = pl_load(b_pre + (t0 + c) * p.b_stride);
                }
                const scalar_t* qr = raw + (c * 3) * DIM;
                const scalar_t* kr = qr + DIM;
                for (int j = sub; j < DIM; j += group) {
                    const float x = pl_load(qr + j), y = pl_load(kr + j);
                    qq = fmaf(x, x, qq);
                    kk = fmaf(y, y, kk);
                }
            }
            for (int offset = group >> 1; offset > 0; offset >>= 1) {
                qq += __shfl_xor_sync(0xffffffffu, qq, offset);
                kk += __shfl_xor_sync(0xffffffffu, kk, offset);
            }
            if (c < n && sub == 0) {
                inv_q[c] = p.q_scale / sqrtf(qq + p.unit_eps);
                inv_k[c] = 1.0f / sqrtf(kk + p.unit_eps);
                sb[c] = 1.0f / (1.0f + expf(-b));
            }
        }
        __syncthreads();
        for (int idx = tid; idx < n * DIM; idx += blockDim.x) {
            const int c = idx / DIM, i = idx - c * DIM;
            const scalar_t* token = raw + c * 3 * DIM;
            sq[idx] = pl_load(token + i) * inv_q[c];
            sk[idx] = pl_load(token + DIM + i) * inv_k[c];
            sg[idx] = expf(-rate * softplus_f32(pl_load(token + 2 * DIM + i) + bias[i]));
        }
        __syncthreads();
        const scalar_t* raw_v = raw + chunk * 3 * DIM;
        // this lane's share of the vectors, one token ahead
        float4 nq[R / 4], nk[R / 4], ng[R / 4];
        float nv, nb;
        auto fetch = [&](int c) {
            const float4* q4 = reinterpret_cast<const float4*>(sq + c * DIM + part * R);
            const float4* k4 = reinterpret_cast<const float4*>(sk + c * DIM + part * R);
            const float4* g4 = reinterpret_cast<const float4*>(sg + c * DIM + part * R);
#pragma unroll
            for (int j = 0; j < R / 4; ++j) {
                nq[j] = q4[j];
                nk[j] = k4[j];
                ng[j] = g4[j];
            }
            nv = active ? pl_load(raw_v + c * cols + col) : 0.0f;
            nb = sb[c];
        };
        fetch(0);
        for (int c = 0; c < n; ++c) {
            float kq[R], kk[R], kg[R];
#pragma unroll
            for (int j = 0; j < R / 4; ++j) {
                kq[4 * j] = nq[j].x; kq[4 * j + 1] = nq[j].y; kq[4 * j + 2] = nq[j].z; kq[4 * j + 3] = nq[j].w;
                kk[4 * j] = nk[j].x; kk[4 * j + 1] = nk[j].y; kk[4 * j + 2] = nk[j].z; kk[4 * j + 3] = nk[j].w;
                kg[4 * j] = ng[j].x; kg[4 * j + 1] = ng[j].y; kg[4 * j + 2] = ng[j].z; kg[4 * j + 3] = ng[j].w;
            }
            const float vj = nv, beta = nb;
            if (c + 1 < n) {
                fetch(c + 1);
            }
            float dot0 = 0.0f, dot1 = 0.0f;
#pragma unroll
            for (int m = 0; m < R; m += 2) {
                S[m] *= kg[m];
                dot0 = fmaf(S[m], kk[m], dot0);
                S[m + 1] *= kg[m + 1];
                dot1 = fmaf(S[m + 1], kk[m + 1], dot1);
            }
            float dot = dot0 + dot1;
#pragma unroll
            for (int offset = PARTS >> 1; offset > 0; offset >>= 1) {
                dot += __shfl_xor_sync(0xffffffffu, dot, offset);
            }
            const float u = beta * (vj - dot);
            float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
            for (int m = 0; m < R; m += 2) {
                S[m] = fmaf(kk[m], u, S[m]);
                o0 = fmaf(S[m], kq[m], o0);
                S[m + 1] = fmaf(kk[m + 1], u, S[m + 1]);
                o1 = fmaf(S[m + 1], kq[m + 1], o1);
            }
            float o = o0 + o1;
#pragma unroll
            for (int offset = PARTS >> 1; offset > 0; offset >>= 1) {
                o += __shfl_xor_sync(0xffffffffu, o, offset);
            }
            if (active && part == 0) {
                p.o_raw[(t0 + c) * (static_cast<int64_t>(p.n_heads) * p.vdim) + static_cast<int64_t>(head) * p.vdim +
                        col0 + col] = o;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < R; ++m) {
        if (active) {
            mine[static_cast<int64_t>(part * R + m) * p.vdim + col] = S[m];
        }
    }
}

// A warp per (token, head): the head's norm over vdim, its weight and the gate.
template <typename scalar_t>
__global__ void gated_delta_finish_kernel(const float* __restrict__ o_raw, const float* __restrict__ norm,
                                          const scalar_t* __restrict__ gate_pre, int64_t gate_stride,
                                          scalar_t* __restrict__ out, int64_t out_stride, int n_pairs, int n_heads,
                                          int vdim, float eps) {
    pl_grid_trigger();
    pl_grid_wait();
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= n_pairs) {
        return;
    }
    const int64_t t = pair / n_heads;
    const int h = pair % n_heads;
    const float* o = o_raw + static_cast<int64_t>(pair) * vdim;
    float square = 0.0f;
    for (int d = lane; d < vdim; d += 32) {
        square = fmaf(o[d], o[d], square);
    }
    square = pl_warp_sum(square);
    const float factor = 1.0f / sqrtf(square / static_cast<float>(vdim) + eps);
    for (int d = lane; d < vdim; d += 32) {
        const float gate = 1.0f / (1.0f + expf(-pl_load(gate_pre + t * gate_stride + static_cast<int64_t>(h) * vdim + d)));
        pl_store(out + t * out_stride + static_cast<int64_t>(h) * vdim + d, o[d] * factor * norm[d] * gate);
    }
}

}  // namespace

// q, k [T, qk_heads * dim] and v [T, n_heads * vdim] with qkv_stride elements between rows; b_pre
// [T, n_heads]; a_pre [T, n_heads * dim]; gate_pre [T, n_heads * vdim]; a_log fp32 [n_heads]; dt_bias
// fp32 [n_heads * dim]; norm fp32 [vdim]; state fp32 [slots, n_heads, dim, vdim] (updated); first_rows,
// counts, slots int32 [entries]; o_raw fp32 [T, n_heads * vdim] scratch; out [T, n_heads * vdim].
PL_API int pl_gated_delta(const void* q, const void* k, const void* v, int64_t qkv_stride, const void* b_pre,
                          int64_t b_stride, const void* a_pre, int64_t a_stride, const void* gate_pre,
                          int64_t gate_stride, const float* a_log, const float* dt_bias, const float* norm,
                          float* state, const int32_t* first_rows, const int32_t* counts, const int32_t* slots,
                          float* o_raw, void* out, int64_t out_stride, int n_tokens, int n_entries, int n_heads,
                          int qk_heads, int dim, int vdim, float unit_eps, float q_scale, float eps, int dtype,
                          cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && n_entries >= 0 && n_heads > 0 && qk_heads > 0 && dim > 0 && vdim > 0,
               "gated_delta: bad sizes tokens=%d entries=%d heads=%d qk_heads=%d dim=%d vdim=%d", n_tokens, n_entries,
               n_heads, qk_heads, dim, vdim);
    PL_REQUIRE(n_heads % qk_heads == 0, "gated_delta: %d heads are not a multiple of %d q/k heads", n_heads, qk_heads);
    PL_REQUIRE(dim <= 32 * kRows, "gated_delta: key size %d exceeds the supported maximum %d", dim, 32 * kRows);
    PL_REQUIRE(n_heads <= 65535, "gated_delta: %d heads exceed the grid limit", n_heads);
    if (n_tokens == 0 || n_entries == 0) {
        return 0;
    }
    int parts = 1;
    while (parts * kRows < dim) {
        parts *= 2;
    }
    int cols = 128 / parts;
    if (cols > vdim) {
        cols = vdim;
    }
    int threads = ((cols * parts + 31) / 32) * 32;
    const size_t elem = dtype == PL_F32 ? 4 : 2;
    // Key sizes 16, 32, 64 and 128 with a full block of columns: the form with the sizes known to the
    // compiler and half of its CTA making chunks ready (256 threads, two buffers of vectors).
    // (there a lane holds eight rows: shorter chains of additions per token, more CTAs per head)
    const bool fixed = (dim == 16 || dim == 32 || dim == 64 || dim == 128) && vdim >= 128 / (dim / 8);
    if (fixed) {
        parts = dim / 8;
        cols = 128 / parts;
        threads = 128;
    }
    auto bytes_for = [&](int chunk) {
        const size_t raw = (static_cast<size_t>(chunk) * (3 * dim + cols) * elem + 15) / 16 * 16;
        if (fixed) {
            const size_t vec = (static_cast<size_t>(chunk) * (3 * dim + cols + 1) + 3) / 4 * 4;
            return (2 * vec + (2 * static_cast<size_t>(chunk) + 3) / 4 * 4 + dim) * sizeof(float) + 2 * raw;
        }
        const size_t vectors = ((static_cast<size_t>(chunk) * (3 * dim + 3) + 3) / 4 * 4 + (dim + 3) / 4 * 4) * sizeof(float);
        return vectors + 2 * raw;
    };
    int chunk = kChunkMost;
    while (chunk > 1 && bytes_for(chunk) > (fixed ? 96 : 44) * 1024) {
        chunk /= 2;
    }
    const size_t smem = bytes_for(chunk);
    PL_REQUIRE(smem <= 200 * 1024, "gated_delta: key size %d needs too much shared memory", dim);
    // A step that brings at most two tokens an entry has nothing to make ready ahead: the form without
    // the second half (the same chunk size, so the same sums).
    const bool few = fixed && n_tokens <= 2 * n_entries;
    const size_t smem_single = ((static_cast<size_t>(chunk) * (3 * dim + 3) + 3) / 4 * 4 + (dim + 3) / 4 * 4) * sizeof(float) +
        2 * ((static_cast<size_t>(chunk) * (3 * dim + cols) * elem + 15) / 16 * 16);
    const int per = static_cast<int>(16 / elem);
    const int async_loads = dim % per == 0 && cols % per == 0 && vdim % per == 0 && qkv_stride % per == 0 &&
        a_stride % per == 0 &&
        ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
          reinterpret_cast<uintptr_t>(a_pre)) & 15) == 0;
    GatedDeltaParams p;
    p.q = q; p.k = k; p.v = v; p.qkv_stride = qkv_stride; p.b_pre = b_pre; p.b_stride = b_stride; p.a_pre = a_pre;
    p.a_stride = a_stride; p.a_log = a_log; p.dt_bias = dt_bias; p.state = state; p.first_rows = first_rows;
    p.counts = counts; p.slots = slots; p.o_raw = o_raw; p.n_heads = n_heads; p.qk_heads = qk_heads; p.dim = dim;
    p.vdim = vdim; p.parts = parts; p.cols = cols; p.chunk = chunk; p.async_loads = async_loads; p.unit_eps = unit_eps; p.q_scale = q_scale;
    const dim3 grid(n_entries, n_heads, (vdim + cols - 1) / cols);
    const int n_pairs = n_tokens * n_heads;
#define PL_SCAN_STATIC(D, P)                                                                                        \
    do {                                                                                                               \
        if (smem > 48 * 1024) {                                                                                        \
            cudaFuncSetAttribute(gated_delta_scan_static_kernel<scalar_t, D, P>,                                       \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));                 \
        }                                                                                                              \
        if (few) {                                                                                                     \
            if (smem_single > 48 * 1024) {                                                                             \
                cudaFuncSetAttribute(gated_delta_scan_static_single_kernel<scalar_t, D, P>,                            \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_single));      \
            }                                                                                                          \
            pl_launch_overlapped(gated_delta_scan_static_single_kernel<scalar_t, D, P>, grid, dim3(128), smem_single,   \
                                 stream, p);                                                                           \
        } else {                                                                                                       \
            pl_launch_overlapped(gated_delta_scan_static_kernel<scalar_t, D, P>, grid, dim3(256), smem, stream, p);    \
        }                                                                                                              \
    } while (0)
    PL_DISPATCH_DTYPE(dtype, "gated_delta", {
        if (fixed && dim == 16) {
            PL_SCAN_STATIC(16, 2);
        } else if (fixed && dim == 32) {
            PL_SCAN_STATIC(32, 4);
        } else if (fixed && dim == 64) {
            PL_SCAN_STATIC(64, 8);
        } else if (fixed && dim == 128) {
            PL_SCAN_STATIC(128, 16);
        } else {
            if (smem > 48 * 1024) {
                cudaFuncSetAttribute(gated_delta_scan_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem));
            }
            pl_launch_overlapped(gated_delta_scan_kernel<scalar_t>, grid, dim3(threads), smem, stream, p);
        }
        pl_launch_overlapped(gated_delta_finish_kernel<scalar_t>, dim3((n_pairs + 3) / 4), dim3(128), 0, stream,
                             static_cast<const float*>(o_raw), norm, static_cast<const scalar_t*>(gate_pre), gate_stride,
                             static_cast<scalar_t*>(out), out_stride, n_pairs, n_heads, vdim, eps);
    });
#undef PL_SCAN_STATIC
    PL_CHECK_LAUNCH("gated_delta");
    return 0;
}
