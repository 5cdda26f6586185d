// Attention whose heads carry several score maps over one set of values (differential
// attention: two maps per head, combined by a difference), laid out for the ordinary paged
// attention kernels.
//
// A query head has `maps` sub-vectors of size dim, a key head likewise, and a value head has
// vdim values. The maps of a head become `maps` query heads of a common row size Dp >=
// max(maps * dim, vdim): map m's query sits in columns [m * dim, (m + 1) * dim) of its row and
// zeros fill the rest, so that against the key row [k map 0 | k map 1 | ... | 0] its dot
// product is the map's own score. Key rows and value rows [v | 0] go to the paged cache as
// one kv head of size Dp; the attention kernels then run `maps * heads` heads over `kv_heads`
// kv heads and know nothing of maps.
//
// pl_rope_maps_write does the layout and the position encoding in one pass: rotary pairs are
// neighbours (2i, 2i + 1) within the first `rotary` columns of every map, angle pos * f_i
// from an fp64 table, reduced in fp64 (rope_helpers.cuh), rotation in fp32.
//
// pl_diff_combine turns the maps' outputs into the head's: o = a_0 - lambda * a_1, divided by
// its root mean square over vdim (fp32), times a constant.
#include "rope_helpers.cuh"

namespace {

template <typename scalar_t>
__device__ __forceinline__ float rotated(const scalar_t* x, int e, int rotary, const float* cs, const float* sn) {
    if (e >= rotary) {
        return pl_load(x + e);
    }
    const int i = e >> 1;
    const float lo = pl_load(x + (e & ~1)), hi = pl_load(x + (e | 1));
    return (e & 1) ? rope_hi(lo, hi, cs[i], sn[i]) : rope_lo(lo, hi, cs[i], sn[i]);
}

__device__ __forceinline__ void store_pair(float* p, float lo, float hi) {
    *reinterpret_cast<float2*>(p) = make_float2(lo, hi);
}
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float lo, float hi) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(lo, hi);
}

template <typename scalar_t>
__global__ void rope_maps_write_kernel(const scalar_t* __restrict__ q, const scalar_t* __restrict__ k,
                                       const scalar_t* __restrict__ v, int64_t row_stride,
                                       const int32_t* __restrict__ pos, const int32_t* __restrict__ entry,
                                       const int32_t* __restrict__ table, int table_width,
                                       scalar_t* __restrict__ k_pool, scalar_t* __restrict__ v_pool,
                                       int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                                       const double* __restrict__ inv_freq, int rotary, int n_heads, int n_kv_heads,
                                       int maps, int dim, int vdim, int padded, int rows_per_block,
                                       scalar_t* __restrict__ q_out, int32_t* status) {
    extern __shared__ float sincos[];  // [rotary/2] cos, [rotary/2] sin
    pl_grid_trigger();
    const int t = blockIdx.x;
    const int p = pos[t];
    const int half = rotary / 2;
    float* cs = sincos;
    float* sn = sincos + half;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        rope_sincos(p, inv_freq[j], cs[j], sn[j]);
    }
    int page = table[static_cast<int64_t>(entry[t]) * table_width + p / page_size];
    if (page < 0 || page >= n_pages) {
        if (threadIdx.x == 0 && status != nullptr) {
            atomicOr(status, 2);
        }
        page = -1;
    }
    pl_grid_wait();
    __syncthreads();
    // Block (t, y) takes `rows_per_block` rows from y * rows_per_block, where rows 0 .. q_rows - 1 are the
    // query rows and the next n_kv_heads the key/value rows: a step of few tokens spreads over many blocks.
    const int q_rows = n_heads * maps;
    const int row0 = blockIdx.y * rows_per_block, row1 = min(row0 + rows_per_block, q_rows + n_kv_heads);
    const scalar_t* qt = q + t * row_stride;
    scalar_t* qo = q_out + static_cast<int64_t>(t) * q_rows * padded;
    if ((dim & 1) == 0) {
        // Two neighbouring columns per thread: a rotary pair is read once and both its halves stored.
        const int half_row = padded / 2;
        for (int idx = row0 * half_row + threadIdx.x; idx < min(row1, q_rows) * half_row; idx += blockDim.x) {
            const int hm = idx / half_row, d = 2 * (idx % half_row);
            const int m = hm % maps;
            const int e = d - m * dim;
            float lo = 0.0f, hi = 0.0f;
            if (e >= 0 && e < dim) {
                const scalar_t* x = qt + static_cast<int64_t>(hm) * dim + e;
                lo = pl_load(x);
                hi = pl_load(x + 1);
                if (e < rotary) {
                    const float c = cs[e >> 1], s = sn[e >> 1];
                    const float a = rope_lo(lo, hi, c, s), b = rope_hi(lo, hi, c, s);
                    lo = a;
                    hi = b;
                }
            }
            store_pair(qo + static_cast<int64_t>(hm) * padded + d, lo, hi);
        }
    } else {
        for (int idx = row0 * padded + threadIdx.x; idx < min(row1, q_rows) * padded; idx += blockDim.x) {
            const int hm = idx / padded, d = idx % padded;
            const int m = hm % maps;
            const int e = d - m * dim;
            float value = 0.0f;
            if (e >= 0 && e < dim) {
                value = rotated(qt + static_cast<int64_t>(hm) * dim, e, rotary, cs, sn);
            }
            pl_store(qo + idx, value);
        }
    }
    if (page < 0 || row1 <= q_rows) {
        return;
    }
    const scalar_t* kt = k + t * row_stride;
    const scalar_t* vt = v + t * row_stride;
    for (int idx = (max(row0, q_rows) - q_rows) * padded + threadIdx.x; idx < (row1 - q_rows) * padded;
         idx += blockDim.x) {
        const int g = idx / padded, d = idx % padded;
        const int64_t at = page * page_stride + g * head_stride + static_cast<int64_t>(p % page_size) * padded + d;
        float key = 0.0f;
        if (d < maps * dim) {
            key = rotated(kt + (static_cast<int64_t>(g) * maps + d / dim) * dim, d % dim, rotary, cs, sn);
        }
        pl_store(k_pool + at, key);
        if (d < vdim) {
            v_pool[at] = vt[static_cast<int64_t>(g) * vdim + d];
        } else {
            pl_store(v_pool + at, 0.0f);
        }
    }
}

// A warp per (token, head).
template <typename scalar_t>
__global__ void diff_combine_kernel(const scalar_t* __restrict__ a, scalar_t* __restrict__ out, int n_pairs,
                                    int vdim, int padded, float lambda, float eps, float mult) {
    pl_grid_trigger();
    pl_grid_wait();
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= n_pairs) {
        return;
    }
    const scalar_t* a0 = a + static_cast<int64_t>(pair) * 2 * padded;
    const scalar_t* a1 = a0 + padded;
    float square = 0.0f;
    for (int d = lane; d < vdim; d += 32) {
        const float o = pl_load(a0 + d) - lambda * pl_load(a1 + d);
        square += o * o;
    }
    square = pl_warp_sum(square);
    const float factor = mult / sqrtf(square / static_cast<float>(vdim) + eps);
    for (int d = lane; d < vdim; d += 32) {
        const float o = pl_load(a0 + d) - lambda * pl_load(a1 + d);
        pl_store(out + static_cast<int64_t>(pair) * vdim + d, o * factor);
    }
}

}  // namespace

// q [T, n_heads * maps * dim], k [T, n_kv_heads * maps * dim], v [T, n_kv_heads * vdim], all with
// row_stride elements between tokens; q_out [T, n_heads * maps, padded] contiguous; pools
// [pages, n_kv_heads, page_size, padded] with page_stride / head_stride elements between
// pages / heads; inv_freq fp64 [rotary / 2] (rotary even, <= dim; 0: no rotation).
PL_API int pl_rope_maps_write(const void* q, const void* k, const void* v, int64_t row_stride, const int32_t* pos,
                              const int32_t* entry, const int32_t* table, int table_width, void* k_pool, void* v_pool,
                              int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                              const double* inv_freq, int rotary, int n_tokens, int n_heads, int n_kv_heads, int maps,
                              int dim, int vdim, int padded, void* q_out, int dtype, int32_t* status,
                              cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && maps > 0 && dim > 0 && vdim > 0,
               "rope_maps_write: bad sizes tokens=%d heads=%d kv_heads=%d maps=%d dim=%d vdim=%d", n_tokens, n_heads,
               n_kv_heads, maps, dim, vdim);
    PL_REQUIRE(padded >= maps * dim && padded >= vdim, "rope_maps_write: rows of %d cannot hold %d maps of %d or %d "
               "values", padded, maps, dim, vdim);
    PL_REQUIRE(rotary >= 0 && rotary % 2 == 0 && rotary <= dim && (rotary == 0 || inv_freq != nullptr),
               "rope_maps_write: rotary width %d must be even and at most dim %d", rotary, dim);
    if (n_tokens == 0) {
        return 0;
    }
    const int all_rows = n_heads * maps + n_kv_heads;
    const int rows_per_block = n_tokens >= 256 ? all_rows : 4;
    const int threads = rows_per_block * padded >= 1024 ? 256 : 128;
    PL_DISPATCH_DTYPE(dtype, "rope_maps_write", {
        pl_launch_overlapped(rope_maps_write_kernel<scalar_t>, dim3(n_tokens, (all_rows + rows_per_block - 1) / rows_per_block),
                             dim3(threads),
                             static_cast<size_t>(rotary > 0 ? rotary : 1) * sizeof(float), stream,
                             static_cast<const scalar_t*>(q), static_cast<const scalar_t*>(k),
                             static_cast<const scalar_t*>(v), row_stride, pos, entry, table, table_width,
                             static_cast<scalar_t*>(k_pool), static_cast<scalar_t*>(v_pool), page_stride, head_stride,
                             page_size, n_pages, inv_freq, rotary, n_heads, n_kv_heads, maps, dim, vdim, padded,
                             rows_per_block, static_cast<scalar_t*>(q_out), status);
    });
    PL_CHECK_LAUNCH("rope_maps_write");
    return 0;
}

// a [T, n_heads, 2, padded] (the two maps' attention outputs, the first vdim columns of each
// row), out [T, n_heads * vdim]: out = (a_0 - lambda a_1) / sqrt(mean((a_0 - lambda a_1)^2) + eps) * mult.
PL_API int pl_diff_combine(const void* a, void* out, int n_tokens, int n_heads, int vdim, int padded, float lambda,
                           float eps, float mult, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && n_heads > 0 && vdim > 0 && padded >= vdim, "diff_combine: bad sizes tokens=%d heads=%d "
               "vdim=%d rows of %d", n_tokens, n_heads, vdim, padded);
    if (n_tokens == 0) {
        return 0;
    }
    const int n_pairs = n_tokens * n_heads;
    const int warps = 4;
    PL_DISPATCH_DTYPE(dtype, "diff_combine", {
        pl_launch_overlapped(diff_combine_kernel<scalar_t>, dim3((n_pairs + warps - 1) / warps), dim3(warps * 32), 0,
                             stream, static_cast<const scalar_t*>(a), static_cast<scalar_t*>(out), n_pairs, vdim,
                             padded, lambda, eps, mult);
    });
    PL_CHECK_LAUNCH("diff_combine");
    return 0;
}
