// The generalized delta rule: per head a matrix S[kd, vd] that decays per key channel and
// from which, before a token's k v^T is added, what the state holds along the token's unit
// key is taken out at a rate per key channel:
//
//     u = k / sqrt(sum k^2 + 1e-6)
//     S <- diag(w) S - (a * u)(u^T S) + k v^T,     o = S^T r
//     w = exp(-e^-1/2 sigmoid(d)),  a = sigmoid(a_raw + bias)       (per head and key channel)
//
// Like the other recurrences (csrc/recurrent.cu) it works column by column of S: column j
// only ever meets v[j], so with c = <u, S_j> taken on the old column
//     S_j <- w * S_j - c (a * u) + v_j k,     o_j = <S_j, r>
// A column is held in the registers of L neighbouring lanes (16 rows each); the tokens'
// vectors come through shared memory, 8 tokens at a time, two buffers in turn, copied
// asynchronously while the chunk in hand is worked on.  State, decays, rates, unit keys and
// sums are 32-bit.
//
// State of a slot: [heads][columns][kd] floats (a column's rows together).
// Plain counterpart: tests/plain_gegorax.py general_delta_mixer().
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_g(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---------------------------------------------------------------------------
// Step 1: per row and head, six 32-bit vectors side by side: r | k | w | u | a u | v.
// ---------------------------------------------------------------------------
struct GDeltaPrepareArgs {
    const void* proj;        // [rows, stride]: r (H d) | k (H d) | v (H d) | ...   and a (H d) at a_col
    const void* decay_in;    // [rows, decay_stride]: what the decay's sigmoid is taken of, before w0
    const float* w0;         // [H d]
    const float* a_bias;     // [H d]
    float* prep;             // [rows, H, 6, d]
    long long stride, decay_stride, a_col;
    int rows, H, d;
};

template <typename T>
__global__ void __launch_bounds__(128) gdelta_prepare_kernel(GDeltaPrepareArgs p) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x;
    const int h = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (h >= p.H) return;
    const int d = p.d, n = p.H * d;
    const T* row = (const T*)p.proj + (size_t)r * p.stride;
    const T* dec = (const T*)p.decay_in + (size_t)r * p.decay_stride;
    float* out = p.prep + ((size_t)r * p.H + h) * 6 * d;
    float ss = 0.f;
    for (int e = lane; e < d; e += 32) {
        const float k = to_f32(row[n + h * d + e]);
        ss += k * k;
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
    const float rate = expf(-0.5f);
    for (int e = lane; e < d; e += 32) {
        const int c = h * d + e;
        const float k = to_f32(row[n + c]);
        const float u = k * inv;
        const float a = sigmoid_g(to_f32(row[p.a_col + c]) + p.a_bias[c]);
        out[e] = to_f32(row[c]);
        out[d + e] = k;
        out[2 * d + e] = expf(-rate * sigmoid_g(to_f32(dec[c]) + p.w0[c]));
        out[3 * d + e] = u;
        out[4 * d + e] = a * u;
        out[5 * d + e] = to_f32(row[2 * n + c]);
    }
}

// ---------------------------------------------------------------------------
// Step 2: the recurrence.
// ---------------------------------------------------------------------------
struct GDeltaScanArgs {
    const float* prep;       // [rows, H, 6, d]
    float* state;            // [slots, state_stride]
    float* out;              // [rows, H * d]
    const int* seq_slot;
    const int* seq_start;
    const int* seq_end;
    const int* seq_row0;
    long long state_stride;
    int H, d;
};

constexpr int kPerLane = 16;
constexpr int kThreads = 64;
constexpr int kChunkMany = 8;

template <int L> __device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(a), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// kThreads threads = kThreads / L columns side by side; grid (column tiles, heads, sequences).
// Lane s of a column owns the rows ((i * L + s) * 4 .. + 3), i = 0..3.
// kChunk tokens are staged at a time; a step of single tokens stages one (CH = 1: an eighth of
// the shared memory, so that many more blocks are resident while the states stream through).
template <int L, bool VEC, int CH>
__global__ void __launch_bounds__(kThreads) gdelta_scan_kernel(GDeltaScanArgs p) {
    constexpr int kChunk = CH;
    constexpr int KP = kPerLane * L;            // key width as staged (zeros behind d)
    constexpr int CB = kThreads / L;            // columns of a block
    constexpr int BUF = kChunk * 6 * KP;
    extern __shared__ __align__(16) float staged[];     // two buffers of [kChunk][6][KP]
    pdl_trigger();
    const int tid = threadIdx.x;
    const int s = tid % L, cl = tid / L;
    const int col = blockIdx.x * CB + cl;
    const int h = blockIdx.y, b = blockIdx.z;
    const int d = p.d;
    const int slot = p.seq_slot[b];
    const int row0 = p.seq_row0[b], n = p.seq_end[b] - p.seq_start[b];
    const int n_chunks = (n + kChunk - 1) / kChunk;
    if (d < KP)      // what lies behind the width stays zero: copies only ever write below d
        for (int i = tid; i < 2 * BUF; i += kThreads) staged[i] = 0.f;
    float* mine = slot >= 0 && col < d
        ? p.state + (size_t)slot * p.state_stride + ((size_t)h * d + col) * d : nullptr;
    pdl_wait();
    float S[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane / 4; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int at = (i * L + s) * 4 + e;
            S[4 * i + e] = mine && at < d ? mine[at] : 0.f;
        }
    __syncthreads();

    // the vectors of chunk c's tokens into a buffer, asynchronously
    auto fetch = [&](float* buf, int c) {
        const int count = min(kChunk, n - c * kChunk);
        const int per = VEC ? 6 * d / 4 : 6 * d;       // copies a token
        for (int i = tid; i < count * per; i += kThreads) {
            const int t = i / per, e = (i % per) * (VEC ? 4 : 1);
            const float* src = p.prep + ((size_t)(row0 + c * kChunk + t) * p.H + h) * 6 * d + e;
            float* dst = buf + t * 6 * KP + (e / d) * KP + e % d;
            if (VEC) copy_async16(dst, src);
            else copy_async4(dst, src);
        }
        copies_commit();
    };
    if (n_chunks > 0) fetch(staged, 0);
    for (int c = 0; c < n_chunks; ++c) {
        float* buf = staged + (c & 1) * BUF;
        copies_wait();
        __syncthreads();
        if (c + 1 < n_chunks) fetch(staged + ((c + 1) & 1) * BUF, c + 1);
        const int count = min(kChunk, n - c * kChunk);
        // <u, S_j> of a token is taken right after the token before it has changed the column,
        // together with that token's <S_j, r>: two sums over the same registers whose
        // exchanges between the lanes travel side by side (the same additions in the same
        // order as one after the other)
        auto along = [&](const float* v6) {
            float su[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < kPerLane / 4; ++i) {
                const float4 x = *reinterpret_cast<const float4*>(v6 + 3 * KP + (i * L + s) * 4);
                su[0] += S[4 * i] * x.x;
                su[1] += S[4 * i + 1] * x.y;
                su[2] += S[4 * i + 2] * x.z;
                su[3] += S[4 * i + 3] * x.w;
            }
            return (su[0] + su[1]) + (su[2] + su[3]);
        };
        float c1 = lanes_sum<L>(along(buf));
        auto token = [&](int t, bool more) {
            const float* v6 = buf + t * 6 * KP;
            const float vj = col < d ? v6[5 * KP + col] : 0.f;
            float so[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < kPerLane / 4; ++i) {
                const int at = (i * L + s) * 4;
                const float4 rr = *reinterpret_cast<const float4*>(v6 + at);
                const float4 kk = *reinterpret_cast<const float4*>(v6 + KP + at);
                const float4 ww = *reinterpret_cast<const float4*>(v6 + 2 * KP + at);
                const float4 au = *reinterpret_cast<const float4*>(v6 + 4 * KP + at);
                S[4 * i] = ww.x * S[4 * i] - c1 * au.x + vj * kk.x;
                S[4 * i + 1] = ww.y * S[4 * i + 1] - c1 * au.y + vj * kk.y;
                S[4 * i + 2] = ww.z * S[4 * i + 2] - c1 * au.z + vj * kk.z;
                S[4 * i + 3] = ww.w * S[4 * i + 3] - c1 * au.w + vj * kk.w;
                so[0] += S[4 * i] * rr.x;
                so[1] += S[4 * i + 1] * rr.y;
                so[2] += S[4 * i + 2] * rr.z;
                so[3] += S[4 * i + 3] * rr.w;
            }
            float o = (so[0] + so[1]) + (so[2] + so[3]);
            float next = more ? along(v6 + 6 * KP) : 0.f;
#pragma unroll
            for (int w = L / 2; w > 0; w >>= 1) {
                o += __shfl_xor_sync(0xffffffffu, o, w);
                next += __shfl_xor_sync(0xffffffffu, next, w);
            }
            c1 = next;
            if (s == 0 && col < d)
                p.out[((size_t)(row0 + c * kChunk + t) * p.H + h) * d + col] = o;
        };
        if (count == kChunk) {
#pragma unroll
            for (int t = 0; t < kChunk; ++t) token(t, t + 1 < kChunk);
        } else {
            for (int t = 0; t < count; ++t) token(t, t + 1 < count);
        }
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < kPerLane / 4; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int at = (i * L + s) * 4 + e;
                if (at < d) mine[at] = S[4 * i + e];
            }
    }
}

}  // namespace

SIB_EXPORT int sib_gdelta_prepare(const void* proj, long long stride, long long a_col,
                                  const void* decay_in, long long decay_stride, int dtype,
                                  const float* w0, const float* a_bias, float* prep, int rows, int H,
                                  int d, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && H > 0 && d > 0 && (H + 3) / 4 < 65536,
                "general_delta_prepare: rows=%d heads=%d width=%d", rows, H, d);
    GDeltaPrepareArgs p{proj, decay_in, w0, a_bias, prep, stride, decay_stride, a_col, rows, H, d};
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(gdelta_prepare_kernel<T>, dim3(rows, (H + 3) / 4),
                                                 dim3(128), 0, (cudaStream_t)stream, p));
    return sib_check_launch("general_delta_prepare");
}

SIB_EXPORT int sib_gdelta_scan(const float* prep, float* state, long long state_stride, float* out,
                               const int* seq_slot, const int* seq_start, const int* seq_end,
                               const int* seq_row0, int rows, int n_seqs, int H, int d,
                               void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && n_seqs > 0 && n_seqs < 65536 && H > 0 && H < 65536 && d > 0 && d <= 512,
                "general_delta_scan: rows=%d sequences=%d heads=%d width=%d (at most 512)", rows,
                n_seqs, H, d);
    GDeltaScanArgs p{prep, state, out, seq_slot, seq_start, seq_end, seq_row0, state_stride, H, d};
    const int L = d <= 16 ? 1 : d <= 32 ? 2 : d <= 64 ? 4 : d <= 128 ? 8 : d <= 256 ? 16 : 32;
    const int per_block = kThreads / L;
    const dim3 grid((d + per_block - 1) / per_block, H, n_seqs);
    const bool vec = d % 4 == 0 && ((uintptr_t)prep % 16) == 0;
    // no sequence of the step has more than one token if there are no more rows than sequences
    const bool single = rows <= n_seqs;
    const size_t smem = (size_t)2 * (single ? 1 : kChunkMany) * 6 * kPerLane * L * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
#define GO_ONE(LL, VV, CC)                                                                     \
    do {                                                                                       \
        if (smem > 48 * 1024) {                                                                \
            cudaError_t e = cudaFuncSetAttribute(gdelta_scan_kernel<LL, VV, CC>,               \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            SIB_REQUIRE(e == cudaSuccess, "general_delta_scan: %s", cudaGetErrorString(e));    \
        }                                                                                      \
        sib_launch_chained(gdelta_scan_kernel<LL, VV, CC>, grid, dim3(kThreads), smem, s, p);  \
    } while (0)
#define GO(LL)                                        \
    do {                                              \
        if (vec && single) GO_ONE(LL, true, 1);       \
        else if (vec) GO_ONE(LL, true, kChunkMany);   \
        else if (single) GO_ONE(LL, false, 1);        \
        else GO_ONE(LL, false, kChunkMany);           \
    } while (0)
    if (L == 1) GO(1);
    else if (L == 2) GO(2);
    else if (L == 4) GO(4);
    else if (L == 8) GO(8);
    else if (L == 16) GO(16);
    else GO(32);
#undef GO
#undef GO_ONE
    return sib_check_launch("general_delta_scan");
}
