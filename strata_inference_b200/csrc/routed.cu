// A feed-forward of many small experts of which each row uses a few.
//
//   router_rows      few rows: the router's 32-bit product and the choice below in one launch.
//   router_topk      from 32-bit router logits [rows, experts] (+ bias): the `top` largest per
//                    row (ties: the lower index) and the softmax over those `top` logits only.
//   expert_activate  y = g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit),
//                    u = clamp(up, -limit, limit), from rows [gate (ff) | up (ff)];
//                    optionally every row times one weight.
//   routed_rows_*    few rows: each (row, chosen expert) pair streams ITS expert's matrices
//                    only.  gate_up makes the activated middle of every pair, down the rows'
//                    outputs: the pairs' results times their weights, summed in 32-bit in
//                    the order of the choice, on top of an optional base row.
//   routed_expert_*  many pairs in a recorded step: expert-major, each expert's matrices read
//                    from memory once for all the pairs that chose it, then routed_combine.
//   routed_combine   many rows (experts run as products over sorted rows): the same sum
//                    from the pairs' outputs, found through the sort's inverse.
//
// Two things are parameters of every entry.  `score`: what a chosen expert's weight is,
// SCORE_SOFTMAX_TOP (the softmax over the chosen logits alone) or SCORE_SIGMOID (the sigmoid of
// the expert's own logit, not normalized).  `form`: what an expert computes, FORM_CLIPPED_GATED
// (above; matrices [2 ff, width]) or FORM_PLAIN_GELU, down(gelu(w * up x)) with the exact gelu,
// matrices [ff, width], where the pair's weight w multiplies what ENTERS the expert (it has no
// bias, so w * (up x) = up (w x)) and the pairs' outputs are summed as they are.
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
__device__ __forceinline__ float gelu_erf(float z) { return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f)); }
constexpr int SCORE_SOFTMAX_TOP = 0, SCORE_SIGMOID = 1;
constexpr int FORM_CLIPPED_GATED = 0, FORM_PLAIN_GELU = 1;

// One warp: the `top` largest of z[e] + bias[e] in order (ties: the lower index) and their
// weights: the softmax over them alone, or each one's own sigmoid.
__device__ __forceinline__ void choose_top(const float* z, const float* __restrict__ bias,
                                           int* __restrict__ ids, float* __restrict__ weights,
                                           int experts, int top, int lane, int score) {
    float first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= ids[j] == e;
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
        // (the first chosen logit is the largest)
        const float w = score == SCORE_SIGMOID ? sigmoid_r(best) : expf(best - first);
        sum += w;
        if (lane == 0) {
            ids[k] = at;
            weights[k] = w;
        }
        __syncwarp();
    }
    if (score == SCORE_SOFTMAX_TOP && lane < top) weights[lane] /= sum;
}

// One warp per row.
__global__ void __launch_bounds__(128)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                   int* __restrict__ ids, float* __restrict__ weights, int rows, int experts, int top,
                   int score) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= rows) return;
    choose_top(logits + (size_t)r * experts, bias, ids + (size_t)r * top, weights + (size_t)r * top,
               experts, top, lane, score);
}

// Few rows: the router's product and the choice in one launch.  One block per row: the row in
// shared memory as 32-bit numbers, a warp per expert's 32-bit matrix row in turn, then the
// first warp chooses.
template <typename T>
__global__ void __launch_bounds__(256)
router_rows_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ w,
                   const float* __restrict__ bias, int* __restrict__ ids, float* __restrict__ weights,
                   int width, int experts, int top, int score) {
    extern __shared__ __align__(16) float sh[];      // [width] the row, [experts] its logits
    float* xs = sh;
    float* z = sh + ((width + 3) & ~3);
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x;
    pdl_wait();
    for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32(x[(size_t)r * x_stride + c]);
    __syncthreads();
    const bool wide = width % 4 == 0 && ((uintptr_t)w % 16) == 0;
    for (int e = warp; e < experts; e += blockDim.x >> 5) {
        const float* row = w + (size_t)e * width;
        float acc = 0.f;
        if (wide) {
            for (int c = lane * 4; c < width; c += 128) {
                const float4 a = *(const float4*)(row + c), b = *(const float4*)(xs + c);
                acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
            }
        } else {
            for (int c = lane; c < width; c += 32) acc += row[c] * xs[c];
        }
        acc = warp_sum(acc);
        if (lane == 0) z[e] = acc;
    }
    __syncthreads();
    if (warp == 0)
        choose_top(z, bias, ids + (size_t)r * top, weights + (size_t)r * top, experts, top, lane, score);
}

// `group` 8: gate and up columns lie interleaved in eights (8 gates, then their 8 ups), as the
// products with a gated epilogue keep their matrices; 0: all gates, then all ups.
// Few rows and many experts: the logits alone, a warp per (row, expert) and 4 experts a block, so
// that the router's matrix is read by many blocks at once; router_topk_kernel then chooses.
template <typename T>
__global__ void __launch_bounds__(128)
router_logits_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ w,
                     float* __restrict__ z, int width, int experts) {
    extern __shared__ __align__(16) float xs[];      // [width] the row
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.y;
    pdl_wait();
    for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32(x[(size_t)r * x_stride + c]);
    __syncthreads();
    const int e = blockIdx.x * 4 + warp;
    if (e >= experts) return;
    const float* row = w + (size_t)e * width;
    float acc = 0.f;
    if (width % 4 == 0 && ((uintptr_t)w % 16) == 0) {
        for (int c = lane * 4; c < width; c += 128) {
            const float4 a = *(const float4*)(row + c), b = *(const float4*)(xs + c);
            acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
        }
    } else {
        for (int c = lane; c < width; c += 32) acc += row[c] * xs[c];
    }
    acc = warp_sum(acc);
    if (lane == 0) z[(size_t)r * experts + e] = acc;
}

template <typename T>
__global__ void expert_activate_kernel(const T* __restrict__ gu, long long stride, T* __restrict__ y,
                                       const float* __restrict__ row_weight, int ff, float limit,
                                       float alpha, size_t total, int form, int group) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / ff;
        const int j = (int)(i - r * ff);
        float v;
        if (form == FORM_PLAIN_GELU) {       // rows [up (ff)]; the row's weight on what enters the gelu
            v = gelu_erf(to_f32(gu[r * stride + j]) * (row_weight ? row_weight[r] : 1.0f));
        } else {
            const size_t g = group ? (size_t)(j / group) * 2 * group + j % group : (size_t)j;
            v = expert_act(to_f32(gu[r * stride + g]), to_f32(gu[r * stride + g + (group ? group : ff)]), limit, alpha);
            if (row_weight) v *= row_weight[r];
        }
        y[i] = from_f32<T>(v);
    }
}

// The same for bfloat16 rows whose widths are multiples of 8 and start on 16-byte boundaries: a
// thread takes 8 neighbouring outputs, whose gates and ups are 16 bytes each in either layout.
__global__ void expert_activate8_kernel(const __nv_bfloat16* __restrict__ gu, long long stride,
                                        __nv_bfloat16* __restrict__ y, const float* __restrict__ row_weight,
                                        int ff, float limit, float alpha, size_t total8, int form, int group) {
    pdl_trigger();
    pdl_wait();
    const int per_row = ff / 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / per_row;
        const int j = (int)(i - r * per_row) * 8;
        const float rw = row_weight ? row_weight[r] : 1.0f;
        float o[8];
        if (form == FORM_PLAIN_GELU) {
            const uint4 a = *reinterpret_cast<const uint4*>(gu + r * stride + j);
            const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[2 * e] = gelu_erf(__uint_as_float(w[e] << 16) * rw);
                o[2 * e + 1] = gelu_erf(__uint_as_float(w[e] & 0xffff0000u) * rw);
            }
        } else {
            const size_t g = group ? (size_t)2 * j : (size_t)j;
            const uint4 a = *reinterpret_cast<const uint4*>(gu + r * stride + g);
            const uint4 b = *reinterpret_cast<const uint4*>(gu + r * stride + g + (group ? 8 : ff));
            const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[2 * e] = expert_act(__uint_as_float(wa[e] << 16), __uint_as_float(wb[e] << 16), limit, alpha) * rw;
                o[2 * e + 1] = expert_act(__uint_as_float(wa[e] & 0xffff0000u), __uint_as_float(wb[e] & 0xffff0000u),
                                          limit, alpha) * rw;
            }
        }
        uint4 out;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 pr = __floats2bfloat162_rn(o[2 * e], o[2 * e + 1]);
            ow[e] = *reinterpret_cast<const uint32_t*>(&pr);
        }
        *reinterpret_cast<uint4*>(y + r * ff + j) = out;
    }
}

// Dot products of N matrix rows with one 32-bit vector x in shared memory, the lanes of a warp
// sharing the columns.  Rows that start on a 16-byte boundary and have a multiple of 8 (bfloat16)
// or 4 (32-bit) columns are read 16 bytes a lane at a time, all N rows' loads issued before
// the first is used; the matrices are read once and not kept in the first-level cache.
__device__ __forceinline__ uint4 load_stream16(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}
__device__ __forceinline__ float dot16(uint4 w, const float* x, __nv_bfloat16) {
    const float4 a = *(const float4*)x, b = *(const float4*)(x + 4);
    float acc = 0.f;
    acc += __uint_as_float(w.x << 16) * a.x + __uint_as_float(w.x & 0xffff0000u) * a.y;
    acc += __uint_as_float(w.y << 16) * a.z + __uint_as_float(w.y & 0xffff0000u) * a.w;
    acc += __uint_as_float(w.z << 16) * b.x + __uint_as_float(w.z & 0xffff0000u) * b.y;
    acc += __uint_as_float(w.w << 16) * b.z + __uint_as_float(w.w & 0xffff0000u) * b.w;
    return acc;
}
__device__ __forceinline__ float dot16(uint4 w, const float* x, float) {
    const float4 a = *(const float4*)x;
    return __uint_as_float(w.x) * a.x + __uint_as_float(w.y) * a.y + __uint_as_float(w.z) * a.z +
           __uint_as_float(w.w) * a.w;
}

// (read again soon by the same block: through the first-level cache)
__device__ __forceinline__ uint4 load_keep16(const void* ptr) { return __ldg((const uint4*)ptr); }

template <typename T, int N, bool KEEP = false>
__device__ __forceinline__ void rows_dot(const T* const (&w)[N], const float* const (&x)[N], int width,
                                         int lane, bool wide, float (&out)[N]) {
    constexpr int PER = 16 / (int)sizeof(T);
    float acc[N];
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = 0.f;
    if (wide) {
        for (int c = lane * PER; c < width; c += 32 * PER) {
            uint4 v[N];
#pragma unroll
            for (int i = 0; i < N; ++i) v[i] = KEEP ? load_keep16(w[i] + c) : load_stream16(w[i] + c);
#pragma unroll
            for (int i = 0; i < N; ++i) acc[i] += dot16(v[i], x[i] + c, T());
        }
    } else {
        for (int c = lane; c < width; c += 32) {
#pragma unroll
            for (int i = 0; i < N; ++i) acc[i] += to_f32(w[i][c]) * x[i][c];
        }
    }
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = warp_sum(acc[i]);
}

template <typename T>
__device__ __forceinline__ bool reads_wide(const T* base, int width) {
    return width % (16 / (int)sizeof(T)) == 0 && ((uintptr_t)base % 16) == 0;
}

// grid (tiles of middle columns, pairs); a block: 4 warps, one pair's x row; a warp takes two
// middle columns at a time: four matrix rows (two gates, two ups) in flight.  PLAIN (experts
// without a gate): four middle columns at a time, the pair's weight on what enters the gelu.
template <typename T, bool PLAIN>
__global__ void __launch_bounds__(128)
routed_rows_gate_up_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ w_gu,
                           const int* __restrict__ ids, const float* __restrict__ pair_weight,
                           T* __restrict__ mid, int width, int ff, int top, float limit, float alpha) {
    extern __shared__ __align__(16) float xs[];
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pair = blockIdx.y;
    pdl_wait();
    const int e = ids[pair];
    const T* row = x + (size_t)(pair / top) * x_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32(row[c]);
    __syncthreads();
    const T* w = w_gu + (size_t)e * (PLAIN ? 1 : 2) * ff * width;
    const bool wide = reads_wide(w_gu, width);
    const float* const xv[4] = {xs, xs, xs, xs};
    if constexpr (PLAIN) {
        const float pw = pair_weight ? pair_weight[pair] : 1.0f;
        for (int j = (blockIdx.x * 4 + warp) * 4; j < ff; j += gridDim.x * 16) {
            const T* const rows[4] = {w + (size_t)j * width, w + (size_t)min(j + 1, ff - 1) * width,
                                      w + (size_t)min(j + 2, ff - 1) * width,
                                      w + (size_t)min(j + 3, ff - 1) * width};
            float d[4];
            rows_dot<T, 4>(rows, xv, width, lane, wide, d);
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (j + i < ff) mid[(size_t)pair * ff + j + i] = from_f32<T>(gelu_erf(d[i] * pw));
            }
        }
        return;
    }
    for (int j = (blockIdx.x * 4 + warp) * 2; j < ff; j += gridDim.x * 8) {
        const int j1 = min(j + 1, ff - 1);
        const T* const rows[4] = {w + (size_t)j * width, w + (size_t)(ff + j) * width,
                                  w + (size_t)j1 * width, w + (size_t)(ff + j1) * width};
        float d[4];
        rows_dot<T, 4>(rows, xv, width, lane, wide, d);
        if (lane == 0) {
            mid[(size_t)pair * ff + j] = from_f32<T>(expert_act(d[0], d[1], limit, alpha));
            if (j1 != j) mid[(size_t)pair * ff + j1] = from_f32<T>(expert_act(d[2], d[3], limit, alpha));
        }
    }
}

// grid (tiles of output columns, rows); a block: 4 warps, the row's `top` middles; a warp takes
// one output column of up to 4 of the row's experts at a time.
template <typename T>
__global__ void __launch_bounds__(128)
routed_rows_down_kernel(const T* __restrict__ mid, const T* __restrict__ w_down,
                        const int* __restrict__ ids, const float* __restrict__ weights,
                        const T* __restrict__ base, T* __restrict__ out, int width, int ff, int top) {
    extern __shared__ __align__(16) float ms[];      // [top][ff]
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.y;
    pdl_wait();
    for (int c = threadIdx.x; c < top * ff; c += blockDim.x) ms[c] = to_f32(mid[(size_t)r * top * ff + c]);
    __syncthreads();
    const bool wide = reads_wide(w_down, ff) && ff % 4 == 0;
    for (int n = blockIdx.x * 4 + warp; n < width; n += gridDim.x * 4) {
        float acc = base ? to_f32(base[(size_t)r * width + n]) : 0.f;
        for (int k0 = 0; k0 < top; k0 += 4) {
            const T* rows[4];
            const float* mv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int k = min(k0 + i, top - 1);
                rows[i] = w_down + ((size_t)ids[(size_t)r * top + k] * width + n) * ff;
                mv[i] = ms + k * ff;
            }
            float d[4];
            rows_dot<T, 4>(rows, mv, ff, lane, wide, d);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (k0 + i < top) acc += (weights ? weights[(size_t)r * top + k0 + i] : 1.0f) * d[i];
        }
        if (lane == 0) out[(size_t)r * width + n] = from_f32<T>(acc);
    }
}

// Many pairs (a recorded step of many rows): expert-major.  grid (tiles of columns, experts); a
// block gathers the pairs that chose its expert (none: it returns without touching the
// expert's matrices) and runs its few matrix rows against each of them in turn, so that an
// expert's matrices come from memory once however many rows chose it (the rows after the
// first find them in the first-level cache).
__device__ __forceinline__ int pairs_of_expert(const int* __restrict__ ids, int pairs, int e, int* list,
                                               int* count) {
    if (threadIdx.x == 0) *count = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x)
        if (ids[i] == e) list[atomicAdd(count, 1)] = i;
    __syncthreads();
    return *count;
}

template <typename T, bool PLAIN>
__global__ void __launch_bounds__(128)
routed_expert_gate_up_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ w_gu,
                             const int* __restrict__ ids, const float* __restrict__ pair_weight,
                             T* __restrict__ mid, int width, int ff, int top, int pairs, float limit,
                             float alpha) {
    extern __shared__ __align__(16) float sh[];      // [width] a row, then the list of pairs
    __shared__ int count;
    float* xs = sh;
    int* list = (int*)(sh + ((width + 3) & ~3));
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.y;
    pdl_wait();
    const int n = pairs_of_expert(ids, pairs, e, list, &count);
    if (n == 0) return;
    const T* w = w_gu + (size_t)e * (PLAIN ? 1 : 2) * ff * width;
    const bool wide = reads_wide(w_gu, width);
    const int j = (blockIdx.x * 4 + warp) * (PLAIN ? 4 : 2), j1 = min(j + 1, ff - 1);
    const float* const xv[4] = {xs, xs, xs, xs};
    for (int q = 0; q < n; ++q) {
        const int pair = list[q];
        const T* row = x + (size_t)(pair / top) * x_stride;
        __syncthreads();
        for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32(row[c]);
        __syncthreads();
        if constexpr (PLAIN) {
            if (j < ff) {
                const T* const rows[4] = {w + (size_t)j * width, w + (size_t)j1 * width,
                                          w + (size_t)min(j + 2, ff - 1) * width,
                                          w + (size_t)min(j + 3, ff - 1) * width};
                float d[4];
                rows_dot<T, 4, true>(rows, xv, width, lane, wide, d);
                const float pw = pair_weight ? pair_weight[pair] : 1.0f;
                if (lane == 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (j + i < ff) mid[(size_t)pair * ff + j + i] = from_f32<T>(gelu_erf(d[i] * pw));
                }
            }
        } else if (j < ff) {
            const T* const rows[4] = {w + (size_t)j * width, w + (size_t)(ff + j) * width,
                                      w + (size_t)j1 * width, w + (size_t)(ff + j1) * width};
            float d[4];
            rows_dot<T, 4, true>(rows, xv, width, lane, wide, d);
            if (lane == 0) {
                mid[(size_t)pair * ff + j] = from_f32<T>(expert_act(d[0], d[1], limit, alpha));
                if (j1 != j) mid[(size_t)pair * ff + j1] = from_f32<T>(expert_act(d[2], d[3], limit, alpha));
            }
        }
    }
}

// ys[pair] = down_e(mid[pair]) for the pairs of expert e; a warp takes four output columns.
template <typename T>
__global__ void __launch_bounds__(128)
routed_expert_down_kernel(const T* __restrict__ mid, const T* __restrict__ w_down,
                          const int* __restrict__ ids, T* __restrict__ ys, int width, int ff, int pairs) {
    extern __shared__ __align__(16) float sh[];      // [ff] a pair's middle, then the list of pairs
    __shared__ int count;
    float* ms = sh;
    int* list = (int*)(sh + ((ff + 3) & ~3));
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.y;
    pdl_wait();
    const int n = pairs_of_expert(ids, pairs, e, list, &count);
    if (n == 0) return;
    const bool wide = reads_wide(w_down, ff);
    const int n0 = (blockIdx.x * 4 + warp) * 4;
    const float* const mv[4] = {ms, ms, ms, ms};
    for (int q = 0; q < n; ++q) {
        const int pair = list[q];
        __syncthreads();
        for (int c = threadIdx.x; c < ff; c += blockDim.x) ms[c] = to_f32(mid[(size_t)pair * ff + c]);
        __syncthreads();
        if (n0 < width) {
            const T* rows[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) rows[i] = w_down + ((size_t)e * width + min(n0 + i, width - 1)) * ff;
            float d[4];
            rows_dot<T, 4, true>(rows, mv, ff, lane, wide, d);
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (n0 + i < width) ys[(size_t)pair * width + n0 + i] = from_f32<T>(d[i]);
            }
        }
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
            acc += (weights ? weights[r * top + k] : 1.0f) * to_f32(ys[(size_t)where[r * top + k] * width + n]);
        out[i] = from_f32<T>(acc);
    }
}

int grid_for(size_t total) {
    const size_t want = (total + 255) / 256;
    return (int)(want < 148 * 16 ? (want ? want : 1) : 148 * 16);
}

}  // namespace

SIB_EXPORT int sib_router_topk(const float* logits, const float* bias, int* ids, float* weights,
                               int rows, int experts, int top, int score, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && experts > 0 && top > 0 && top <= experts && top <= 32,
                "router_topk: rows=%d experts=%d top=%d (at most 32 and the number of experts)",
                rows, experts, top);
    sib_launch_chained(router_topk_kernel, dim3((rows + 3) / 4), dim3(128), 0, (cudaStream_t)stream,
                       logits, bias, ids, weights, rows, experts, top, score);
    return sib_check_launch("router_topk");
}

SIB_EXPORT int sib_router_rows(const void* x, long long x_stride, int dtype, const float* w,
                               const float* bias, int* ids, float* weights, int rows, int width,
                               int experts, int top, int score, float* logits, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && width > 0 && experts > 0 && top > 0 && top <= experts && top <= 32,
                "router_rows: rows=%d width=%d experts=%d top=%d", rows, width, experts, top);
    if (logits != nullptr && experts >= 16 && rows < 65536 && (size_t)width * 4 <= 48 * 1024) {
        // (one block a row walked 32 experts' rows of 2 048 in 23 us; spread over the device the
        // product and the choice are two launches of a few us)
        SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(router_logits_kernel<T>, dim3((experts + 3) / 4, rows),
                                                     dim3(128), (size_t)width * 4, (cudaStream_t)stream,
                                                     (const T*)x, x_stride, w, logits, width, experts));
        int rc = sib_check_launch("router_logits");
        if (rc) return rc;
        sib_launch_chained(router_topk_kernel, dim3((rows + 3) / 4), dim3(128), 0, (cudaStream_t)stream,
                           (const float*)logits, bias, ids, weights, rows, experts, top, score);
        return sib_check_launch("router_topk");
    }
    const size_t shared = ((size_t)((width + 3) & ~3) + experts) * 4;
    SIB_REQUIRE(shared <= 48 * 1024, "router_rows: a row of %d and %d logits do not fit shared memory",
                width, experts);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(router_rows_kernel<T>, dim3(rows), dim3(256), shared,
                                                 (cudaStream_t)stream, (const T*)x, x_stride, w, bias,
                                                 ids, weights, width, experts, top, score));
    return sib_check_launch("router_rows");
}

SIB_EXPORT int sib_expert_activate(const void* gu, long long stride, void* y, const float* row_weight,
                                   int dtype, int rows, int ff, float limit, float alpha, int form,
                                   int group, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && ff > 0 && stride >= (form == FORM_PLAIN_GELU ? 1 : 2) * ff,
                "expert_activate: rows=%d ff=%d", rows, ff);
    SIB_REQUIRE(group == 0 || (group == 8 && ff % 8 == 0 && form != FORM_PLAIN_GELU),
                "expert_activate: columns interleaved in groups of %d (0 or 8, ff a multiple of 8)", group);
    const size_t total = (size_t)rows * ff;
    if (dtype == SIB_BF16 && ff % 8 == 0 && stride % 8 == 0 && ((uintptr_t)gu % 16) == 0 &&
        ((uintptr_t)y % 16) == 0) {
        sib_launch_chained(expert_activate8_kernel, dim3(grid_for(total / 8)), dim3(256), 0,
                           (cudaStream_t)stream, (const __nv_bfloat16*)gu, stride, (__nv_bfloat16*)y, row_weight,
                           ff, limit, alpha, total / 8, form, group);
        return sib_check_launch("expert_activate");
    }
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(expert_activate_kernel<T>, dim3(grid_for(total)),
                                                 dim3(256), 0, (cudaStream_t)stream, (const T*)gu,
                                                 stride, (T*)y, row_weight, ff, limit, alpha, total, form, group));
    return sib_check_launch("expert_activate");
}

SIB_EXPORT int sib_routed_rows(const void* x, long long x_stride, const void* w_gu, const void* w_down,
                               const int* ids, const float* weights, const void* base, void* mid,
                               void* out, int dtype, int rows, int width, int ff, int top,
                               float limit, float alpha, int form, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && rows * (long long)top < 65536 && width > 0 && ff > 0 && top > 0,
                "routed_rows: rows=%d top=%d width=%d ff=%d", rows, top, width, ff);
    SIB_REQUIRE((size_t)width * 4 <= 48 * 1024 && (size_t)top * ff * 4 <= 48 * 1024,
                "routed_rows: rows of %d and %d x %d do not fit shared memory", width, top, ff);
    cudaStream_t s = (cudaStream_t)stream;
    const int pairs = rows * top;
    const bool plain = form == FORM_PLAIN_GELU;
    // (experts without a gate weigh what enters them: the pairs' outputs are summed as they are)
    const float* out_weights = plain ? nullptr : weights;
    if (plain) {
        SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(routed_rows_gate_up_kernel<T, true>,
                                                     dim3(min((ff + 15) / 16, 64), pairs), dim3(128),
                                                     (size_t)width * 4, s, (const T*)x, x_stride,
                                                     (const T*)w_gu, ids, weights, (T*)mid, width, ff,
                                                     top, limit, alpha));
    } else {
        SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(routed_rows_gate_up_kernel<T, false>,
                                                     dim3(min((ff + 7) / 8, 64), pairs), dim3(128),
                                                     (size_t)width * 4, s, (const T*)x, x_stride,
                                                     (const T*)w_gu, ids, weights, (T*)mid, width, ff,
                                                     top, limit, alpha));
    }
    int rc = sib_check_launch("routed_rows_gate_up");
    if (rc) return rc;
    // (few rows: more blocks a row, so that the device is filled twice over: with one row and 64
    // blocks a warp walked 8 output columns one after the other, 100 us a layer at width 2 048)
    const int down_tiles = min((width + 3) / 4, max(64, 1184 / rows));
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(routed_rows_down_kernel<T>,
                                                 dim3(down_tiles, rows), dim3(128),
                                                 (size_t)top * ff * 4, s, (const T*)mid,
                                                 (const T*)w_down, ids, out_weights, (const T*)base,
                                                 (T*)out, width, ff, top));
    return sib_check_launch("routed_rows_down");
}

// The same as routed_rows for many pairs: `ys` [rows * top, width] takes the pairs' outputs and
// `order` the numbers 0 .. rows * top - 1 (where pair (r, k)'s output lies: r * top + k).
SIB_EXPORT int sib_routed_by_expert(const void* x, long long x_stride, const void* w_gu,
                                    const void* w_down, const int* ids, const float* weights,
                                    const void* base, void* mid, void* ys, const int* order, void* out,
                                    int dtype, int rows, int width, int ff, int top, int experts,
                                    float limit, float alpha, int form, void* stream) {
    if (rows == 0) return 0;
    const long long pairs = (long long)rows * top;
    SIB_REQUIRE(rows > 0 && width > 0 && ff > 0 && top > 0 && experts > 0 && experts < 65536 &&
                    ((size_t)max(width, ff) + 4 + pairs) * 4 <= 48 * 1024,
                "routed_by_expert: rows=%d top=%d width=%d ff=%d experts=%d", rows, top, width, ff, experts);
    cudaStream_t s = (cudaStream_t)stream;
    const bool plain = form == FORM_PLAIN_GELU;
    const float* out_weights = plain ? nullptr : weights;
    if (plain) {
        SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(routed_expert_gate_up_kernel<T, true>,
                                                     dim3((ff + 15) / 16, experts), dim3(128),
                                                     ((size_t)((width + 3) & ~3) + pairs) * 4, s,
                                                     (const T*)x, x_stride, (const T*)w_gu, ids, weights,
                                                     (T*)mid, width, ff, top, (int)pairs, limit, alpha));
    } else {
        SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(routed_expert_gate_up_kernel<T, false>,
                                                     dim3((ff + 7) / 8, experts), dim3(128),
                                                     ((size_t)((width + 3) & ~3) + pairs) * 4, s,
                                                     (const T*)x, x_stride, (const T*)w_gu, ids, weights,
                                                     (T*)mid, width, ff, top, (int)pairs, limit, alpha));
    }
    int rc = sib_check_launch("routed_expert_gate_up");
    if (rc) return rc;
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(routed_expert_down_kernel<T>,
                                                 dim3((width + 15) / 16, experts), dim3(128),
                                                 ((size_t)((ff + 3) & ~3) + pairs) * 4, s,
                                                 (const T*)mid, (const T*)w_down, ids, (T*)ys, width, ff,
                                                 (int)pairs));
    rc = sib_check_launch("routed_expert_down");
    if (rc) return rc;
    const size_t total = (size_t)rows * width;
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(routed_combine_kernel<T>, dim3(grid_for(total)),
                                                 dim3(256), 0, s, (const T*)ys, order, out_weights,
                                                 (const T*)base, (T*)out, width, top, total));
    return sib_check_launch("routed_combine");
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
