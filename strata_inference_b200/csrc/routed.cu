// A feed-forward of many small experts of which each row uses a few.
//
//   router_topk      from 32-bit router logits [rows, experts] (+ bias): the `top` largest per
//                    row (ties: the lower index) and the softmax over those `top` logits only.
//   expert_activate  y = g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit),
//                    u = clamp(up, -limit, limit), from rows [gate (ff) | up (ff)];
//                    optionally every row times one weight.
//   routed_rows_*    few rows: each (row, chosen expert) pair streams ITS expert's matrices
//                    only.  gate_up makes the activated middle of every pair, down the rows'
//                    outputs: the pairs' results times their weights, summed in 32-bit in
//                    the order of the choice, on top of an optional base row.
//   routed_combine   many rows (experts run as products over sorted rows): the same sum
//                    from the pairs' outputs, found through the sort's inverse.
//
// Plain counterpart: tests/plain_gegorax.py routed_ff(), expert().
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_r(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float expert_act(float g, float u, float limit, float alpha) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoid_r(alpha * g) * (u + 1.0f);
}

// One warp per row.
__global__ void __launch_bounds__(128)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                   int* __restrict__ ids, float* __restrict__ weights, int rows, int experts, int top) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float* z = logits + (size_t)r * experts;
    float first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= ids[(size_t)r * top + j] == e;
            const float v = z[e] + (bias ? bias[e] : 0.f);
            if (!taken && (v > best || (v == best && e < at))) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (k == 0) first = best;
        const float w = expf(best - first);      // the first chosen logit is the largest
        sum += w;
        if (lane == 0) {
            ids[(size_t)r * top + k] = at;
            weights[(size_t)r * top + k] = w;
        }
        __syncwarp();
    }
    if (lane < top) weights[(size_t)r * top + lane] /= sum;
}

template <typename T>
__global__ void expert_activate_kernel(const T* __restrict__ gu, long long stride, T* __restrict__ y,
                                       const float* __restrict__ row_weight, int ff, float limit,
                                       float alpha, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / ff;
        const int j = (int)(i - r * ff);
        float v = expert_act(to_f32(gu[r * stride + j]), to_f32(gu[r * stride + ff + j]), limit, alpha);
        if (row_weight) v *= row_weight[r];
        y[i] = from_f32<T>(v);
    }
}

// <w_row, x> over `width` columns, x 32-bit in shared memory; the lanes of a warp share it.
template <typename T>
__device__ __forceinline__ float row_dot(const T* __restrict__ w, const float* x, int width, int lane) {
    float acc = 0.f;
    for (int c = lane; c < width; c += 32) acc += to_f32(w[c]) * x[c];
    return warp_sum(acc);
}

// grid (tiles of 8 middle columns per warp ..., pairs); a block: 4 warps, one pair's x row.
template <typename T>
__global__ void __launch_bounds__(128)
routed_rows_gate_up_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ w_gu,
                           const int* __restrict__ ids, T* __restrict__ mid, int width, int ff,
                           int top, float limit, float alpha) {
    extern __shared__ float xs[];
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pair = blockIdx.y;
    pdl_wait();
    const int e = ids[pair];
    const T* row = x + (size_t)(pair / top) * x_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32(row[c]);
    __syncthreads();
    const T* w = w_gu + (size_t)e * 2 * ff * width;
    for (int j = blockIdx.x * 4 + warp; j < ff; j += gridDim.x * 4) {
        const float g = row_dot(w + (size_t)j * width, xs, width, lane);
        const float u = row_dot(w + (size_t)(ff + j) * width, xs, width, lane);
        if (lane == 0) mid[(size_t)pair * ff + j] = from_f32<T>(expert_act(g, u, limit, alpha));
    }
}

// grid (tiles of output columns, rows); a block: 4 warps, the row's `top` middles.
template <typename T>
__global__ void __launch_bounds__(128)
routed_rows_down_kernel(const T* __restrict__ mid, const T* __restrict__ w_down,
                        const int* __restrict__ ids, const float* __restrict__ weights,
                        const T* __restrict__ base, T* __restrict__ out, int width, int ff, int top) {
    extern __shared__ float ms[];      // [top][ff]
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.y;
    pdl_wait();
    for (int c = threadIdx.x; c < top * ff; c += blockDim.x) ms[c] = to_f32(mid[(size_t)r * top * ff + c]);
    __syncthreads();
    for (int n = blockIdx.x * 4 + warp; n < width; n += gridDim.x * 4) {
        float acc = base ? to_f32(base[(size_t)r * width + n]) : 0.f;
        for (int k = 0; k < top; ++k) {
            const int e = ids[(size_t)r * top + k];
            const float v = row_dot(w_down + ((size_t)e * width + n) * ff, ms + k * ff, ff, lane);
            acc += weights[(size_t)r * top + k] * v;
        }
        if (lane == 0) out[(size_t)r * width + n] = from_f32<T>(acc);
    }
}

template <typename T>
__global__ void routed_combine_kernel(const T* __restrict__ ys, const int* __restrict__ where,
                                      const float* __restrict__ weights, const T* __restrict__ base,
                                      T* __restrict__ out, int width, int top, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / width;
        const int n = (int)(i - r * width);
        float acc = base ? to_f32(base[i]) : 0.f;
        for (int k = 0; k < top; ++k)
            acc += weights[r * top + k] * to_f32(ys[(size_t)where[r * top + k] * width + n]);
        out[i] = from_f32<T>(acc);
    }
}

int grid_for(size_t total) {
    const size_t want = (total + 255) / 256;
    return (int)(want < 148 * 16 ? (want ? want : 1) : 148 * 16);
}

}  // namespace

SIB_EXPORT int sib_router_topk(const float* logits, const float* bias, int* ids, float* weights,
                               int rows, int experts, int top, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && experts > 0 && top > 0 && top <= experts && top <= 32,
                "router_topk: rows=%d experts=%d top=%d (at most 32 and the number of experts)",
                rows, experts, top);
    sib_launch_chained(router_topk_kernel, dim3((rows + 3) / 4), dim3(128), 0, (cudaStream_t)stream,
                       logits, bias, ids, weights, rows, experts, top);
    return sib_check_launch("router_topk");
}

SIB_EXPORT int sib_expert_activate(const void* gu, long long stride, void* y, const float* row_weight,
                                   int dtype, int rows, int ff, float limit, float alpha,
                                   void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && ff > 0 && stride >= 2 * ff, "expert_activate: rows=%d ff=%d", rows, ff);
    const size_t total = (size_t)rows * ff;
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(expert_activate_kernel<T>, dim3(grid_for(total)),
                                                 dim3(256), 0, (cudaStream_t)stream, (const T*)gu,
                                                 stride, (T*)y, row_weight, ff, limit, alpha, total));
    return sib_check_launch("expert_activate");
}

SIB_EXPORT int sib_routed_rows(const void* x, long long x_stride, const void* w_gu, const void* w_down,
                               const int* ids, const float* weights, const void* base, void* mid,
                               void* out, int dtype, int rows, int width, int ff, int top,
                               float limit, float alpha, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && rows * (long long)top < 65536 && width > 0 && ff > 0 && top > 0,
                "routed_rows: rows=%d top=%d width=%d ff=%d", rows, top, width, ff);
    SIB_REQUIRE((size_t)width * 4 <= 48 * 1024 && (size_t)top * ff * 4 <= 48 * 1024,
                "routed_rows: rows of %d and %d x %d do not fit shared memory", width, top, ff);
    cudaStream_t s = (cudaStream_t)stream;
    const int pairs = rows * top;
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(routed_rows_gate_up_kernel<T>,
                                                 dim3(min((ff + 3) / 4, 64), pairs), dim3(128),
                                                 (size_t)width * 4, s, (const T*)x, x_stride,
                                                 (const T*)w_gu, ids, (T*)mid, width, ff, top, limit,
                                                 alpha));
    int rc = sib_check_launch("routed_rows_gate_up");
    if (rc) return rc;
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(routed_rows_down_kernel<T>,
                                                 dim3(min((width + 3) / 4, 64), rows), dim3(128),
                                                 (size_t)top * ff * 4, s, (const T*)mid,
                                                 (const T*)w_down, ids, weights, (const T*)base,
                                                 (T*)out, width, ff, top));
    return sib_check_launch("routed_rows_down");
}

SIB_EXPORT int sib_routed_combine(const void* ys, const int* where, const float* weights,
                                  const void* base, void* out, int dtype, int rows, int width,
                                  int top, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && width > 0 && top > 0, "routed_combine: rows=%d width=%d top=%d", rows,
                width, top);
    const size_t total = (size_t)rows * width;
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(routed_combine_kernel<T>, dim3(grid_for(total)),
                                                 dim3(256), 0, (cudaStream_t)stream, (const T*)ys,
                                                 where, weights, (const T*)base, (T*)out, width, top,
                                                 total));
    return sib_check_launch("routed_combine");
}
