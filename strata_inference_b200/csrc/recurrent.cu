// Mixers that carry a matrix per head from token to token instead of keys and values:
// the gated delta rule (with its short convolutions) and the matrix memory with
// exponential gates.  State, decays, gates, unit norms and the recurrences are 32-bit.
//
// Both recurrences work column by column of the head's matrix S[kd, vd]: column j only
// ever meets v[j], so (head, column) pairs are independent and a launch has
// sequences x heads x columns of parallel work; the tokens of a sequence go one after
// the other.  A column is held in the registers of L neighbouring lanes (16 rows each).
//
//   delta:   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//            as one pass:  u = beta (v_j - g <S_j, k>),  o_j = g <S_j, q> + u <k, q>,
//            S_j <- g S_j + u k
//   memory:  m' = max(f + m, i);  a = e^(f + m - m'),  b = e^(i - m');
//            S_j <- a S_j + b v_j k,  o_j = a <S_j, q> + b v_j <k, q>
//            with one more column whose v is 1: it holds n, and its output is <n, q>.
//   retention:  S <- d S + k v^T,  o = S^T q  with one fixed decay d per head:
//            S_j <- d S_j + v_j k,  o_j = d <S_j, q> + v_j <k, q>
//   gated:   S <- a S + b k v^T,  o = S^T q  with a and b given per row and head (the
//            state-space layer: k = B, q = C, v = x, a = exp(-exp(A_log) dt), b = dt)
//
// State of a slot: [heads][columns][kd] floats (a column's rows together), then for the
// memory [heads] running maxima.  The delta rule's convolution history lies behind its
// matrices: [taps - 1][channels] floats, oldest first.
//
// Plain counterparts: tests/plain_karupel.py short_conv(), delta_mixer(), mlstm_mixer().
#include "common.cuh"

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) {
    return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
}

// ---------------------------------------------------------------------------
// Delta rule, step 1: per row, the short causal convolutions of q | k | v with silu, then
// unit q (times kd^-1/2) and unit k per head, beta and the decay per head (kd <= 512).
// ---------------------------------------------------------------------------
struct DeltaPrepareArgs {
    const void* proj;        // [rows, stride]: q (G kd) | k (G kd) | v (H vd) | gate (H vd) | b (H) | a (H)
    const float* conv_w;     // [channels, taps], channels = 2 G kd + H vd, last tap the row's own
    const float* a_log;      // [H]
    const float* dt_bias;    // [H]
    float* state;            // [slots, state_stride]; the history starts at hist_offset
    float* qn;               // [rows, G kd]
    float* kn;               // [rows, G kd]
    float* vc;               // [rows, H vd]
    float* beta;             // [rows, H]
    float* decay;            // [rows, H]
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* seq_start;
    const int* seq_row0;
    long long stride, state_stride, hist_offset;
    int H, G, kd, vd, taps;
};

// One warp per (row, unit): the q heads, the k heads, the v heads, and one unit for beta
// and the decay; a block takes 4 units of one row.
template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(DeltaPrepareArgs p) {
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x;
    const int unit = blockIdx.y * 4 + (threadIdx.x >> 5);
    const int units = 2 * p.G + p.H + 1;
    if (unit >= units) return;
    const int nqk = p.G * p.kd, channels = 2 * nqk + p.H * p.vd;
    const int pos = p.row_pos[r];
    const int b = p.row_seq[r];
    const int slot = p.seq_slot[b];
    const int start = p.seq_start[b], row0 = p.seq_row0[b];
    const float* hist = slot >= 0 ? p.state + (size_t)slot * p.state_stride + p.hist_offset : nullptr;
    pdl_wait();
    const T* proj = (const T*)p.proj;
    if (unit == units - 1) {
        for (int h = lane; h < p.H; h += 32) {
            const size_t at = (size_t)r * p.stride + channels + (size_t)p.H * p.vd;
            p.beta[(size_t)r * p.H + h] = sigmoid_f(to_f32(proj[at + h]));
            const float dt = softplus_f(to_f32(proj[at + p.H + h]) + p.dt_bias[h]);
            p.decay[(size_t)r * p.H + h] = expf(-expf(p.a_log[h]) * dt);
        }
        return;
    }
    // the convolved, activated values of 8 channels c0 + lane + 32 i (those below c1): all
    // loads of a tap are asked for before any is used
    auto channels8 = [&](int c0, int c1, float (&y)[8]) {
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = 0.f;
        for (int j = 0; j < p.taps; ++j) {
            const int at = pos - (p.taps - 1) + j;      // position of the tap's input
            float x[8], w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = c0 + lane + 32 * i;
                x[i] = w[i] = 0.f;
                if (c < c1) {
                    w[i] = p.conv_w[(size_t)c * p.taps + j];
                    if (at >= start) x[i] = to_f32(proj[(size_t)(row0 + at - start) * p.stride + c]);
                    else if (hist) x[i] = hist[(size_t)(at - start + p.taps - 1) * channels + c];
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] += w[i] * x[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = silu_f(y[i]);
    };
    float x[8];
    if (unit >= 2 * p.G) {                                   // a v head
        const int c0 = 2 * nqk + (unit - 2 * p.G) * p.vd;
        for (int d0 = 0; d0 < p.vd; d0 += 256) {
            channels8(c0 + d0, c0 + p.vd, x);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (d0 + lane + 32 * i < p.vd)
                    p.vc[(size_t)r * p.H * p.vd + (c0 - 2 * nqk) + d0 + lane + 32 * i] = x[i];
        }
        return;
    }
    float x2[8];                                             // kd <= 512: two rounds of 256
    channels8(unit * p.kd, (unit + 1) * p.kd, x);
#pragma unroll
    for (int i = 0; i < 8; ++i) x2[i] = 0.f;
    if (p.kd > 256) channels8(unit * p.kd + 256, (unit + 1) * p.kd, x2);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += x[i] * x[i] + x2[i] * x2[i];   // (channels beyond kd gave silu(0) = 0)
    float inv = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
    if (unit < p.G) inv *= 1.0f / sqrtf((float)p.kd);
    float* dst = (unit < p.G ? p.qn : p.kn) + (size_t)r * nqk + (size_t)(unit % p.G) * p.kd;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (lane + 32 * i < p.kd) dst[lane + 32 * i] = x[i] * inv;
        if (256 + lane + 32 * i < p.kd) dst[256 + lane + 32 * i] = x2[i] * inv;
    }
}

// The history after the step: the last taps - 1 inputs of each sequence.  One thread per
// (sequence, channel) walks the cells oldest first; a cell that keeps an older input takes
// it from a later cell of the same history, which has not been rewritten yet.
template <typename T>
__global__ void conv_history_kernel(const T* __restrict__ proj, long long stride, float* state,
                                    long long state_stride, long long hist_offset,
                                    const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                                    const int* __restrict__ seq_end, const int* __restrict__ seq_row0,
                                    int channels, int taps) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.y;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int n = seq_end[b] - seq_start[b], row0 = seq_row0[b];
    float* hist = state + (size_t)slot * state_stride + hist_offset;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x)
        for (int i = 0; i < taps - 1; ++i) {
            const int back = taps - 1 - i;              // the input `back` positions before the end
            hist[(size_t)i * channels + c] =
                back <= n ? to_f32(proj[(size_t)(row0 + n - back) * stride + c])
                          : hist[(size_t)(i + n) * channels + c];
        }
}

// ---------------------------------------------------------------------------
// The recurrences.
// ---------------------------------------------------------------------------
// SCAN_GATED: S <- keep S + take k v^T with keep and take given per row and head (a state-space
// layer's discretised decay and step size): the memory's update with ready-made factors.
enum { SCAN_DELTA = 0, SCAN_MEMORY = 1, SCAN_RETENTION = 2, SCAN_GATED = 3 };

struct ScanArgs {
    const void* q;           // row r, key head g at q + r * q_stride + g * kd
    const void* k;
    const void* v;           // row r, head h at v + r * v_stride + h * vd
    const float* decay;      // delta: [rows, H]
    const float* beta;       // delta: [rows, H]
    const void* gate_i;      // memory: row r, head h at gate_i + r * gate_stride + h (before bias and cap)
    const void* gate_f;
    const float* bias_i;     // [H]
    const float* bias_f;     // [H]
    float* state;            // [slots, state_stride]
    float* out;              // [rows, H * cols]; cols = vd (delta) or vd + 1 (memory: <n, q> last)
    float* m_out;            // memory: [rows, H] the running maximum after the row
    const int* seq_slot;
    const int* seq_start;
    const int* seq_end;
    const int* seq_row0;
    long long q_stride, k_stride, v_stride, gate_stride, state_stride;
    int H, G, kd, vd;
    float q_scale, cap;
    const float* head_decay; // retention: [H]
};

constexpr int kPerLane = 16;     // rows of a column that one lane holds
constexpr int kMaxLanes = 32;    // lanes that share a column at most
constexpr int kScanThreads = 64;
constexpr int kColsPerThread = 1;   // independent columns a thread walks side by side (2: slower, see below)
constexpr int kChunk = 8;        // tokens staged in shared memory at a time

template <int L> __device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float log_sigmoid_f(float z) { return -softplus_f(-z); }

// kScanThreads threads = kScanThreads / L columns side by side, each held by L neighbouring lanes, and
// kColsPerThread such sets per block (a thread walks its columns of all sets.  Measured at 8 heads
// of 128 x 256 and one sequence of 2 048 tokens: two sets 840 us against 643 us with one; a warp
// then issues more per cycle, but half as many warps leave half of the schedulers idle);
// grid (column tiles, heads,
// sequences).  Lane s of a column owns the rows ((i * L + s) * 4 .. + 3), so that
// the lanes of a column read neighbouring 16-byte pieces of it (i = 0..kPerLane / 4 - 1).
//
// The tokens' q, k, v and gates come through shared memory, kChunk tokens at a time and two
// buffers in turn: the next chunk's values are asked for before the current chunk is worked
// on and put down after it, so the walk over the tokens waits for shared memory only.  For
// the memory the gates of a chunk (which depend on no matrix) are made once per chunk by
// kChunk threads, in closed form: with F_t = f_1 + .. + f_t inside the chunk and m_0 the
// maximum before it,  m_t = max(F_t + m_0, max_{s <= t} (i_s + F_t - F_s)).
template <int MODE, typename TQ, typename TG, int L, bool VEC>
__global__ void __launch_bounds__(kScanThreads) recurrent_scan_kernel(ScanArgs p) {
    constexpr int KP = kPerLane * L;                 // key width as staged (zeros behind kd)
    constexpr int NT = kScanThreads;
    constexpr int NC = kColsPerThread;
    constexpr int CW = NT / L;                       // columns side by side in a block
    constexpr int CB = NC * CW;                      // columns of a block
    constexpr int BUF = kChunk * (2 * KP + CB + 4);  // q | k | v | keep | take | i | f
    constexpr int NQ = kChunk * KP / NT > 0 ? kChunk * KP / NT : 1;
    constexpr int NV = kChunk * CB / NT > 0 ? kChunk * CB / NT : 1;
    extern __shared__ __align__(16) float staged[];
    __shared__ float m_carry;
    pdl_trigger();
    const int tid = threadIdx.x;
    const int s = tid % L, cl = tid / L;
    const int col0 = blockIdx.x * CB + cl;         // this thread's columns: col0 + j * CW
    const int h = blockIdx.y, b = blockIdx.z;
    const int cols = MODE == SCAN_MEMORY ? p.vd + 1 : p.vd;
    // (lanes without a column still take part in shuffles and barriers)
    const int g = h / (p.H / p.G);
    const int slot = p.seq_slot[b];
    const int row0 = p.seq_row0[b], n = p.seq_end[b] - p.seq_start[b];
    const int n_chunks = (n + kChunk - 1) / kChunk;
    float S[NC][kPerLane];
    float* mine[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j)
        mine[j] = slot >= 0 && col0 + j * CW < cols
            ? p.state + (size_t)slot * p.state_stride + ((size_t)h * cols + col0 + j * CW) * p.kd : nullptr;
    float* m_cell = MODE == SCAN_MEMORY && slot >= 0
        ? p.state + (size_t)slot * p.state_stride + (size_t)p.H * cols * p.kd + h : nullptr;
    pdl_wait();
#pragma unroll
    for (int j = 0; j < NC; ++j)
#pragma unroll
        for (int i = 0; i < kPerLane / 4; ++i) {
            const int d = (i * L + s) * 4;
            if (VEC) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (mine[j] && d < p.kd) v = *reinterpret_cast<const float4*>(mine[j] + d);
                S[j][4 * i] = v.x; S[j][4 * i + 1] = v.y; S[j][4 * i + 2] = v.z; S[j][4 * i + 3] = v.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    S[j][4 * i + e] = mine[j] && d + e < p.kd ? mine[j][d + e] : 0.f;
            }
        }
    if (tid == 0) m_carry = m_cell ? *m_cell : 0.f;

    const TQ* qp = (const TQ*)p.q + (size_t)g * p.kd;
    const TQ* kp = (const TQ*)p.k + (size_t)g * p.kd;
    const TQ* vp = (const TQ*)p.v + (size_t)h * p.vd;
    TQ rq[NQ], rk[NQ], rv[NV];
    TG rg = from_f32<TG>(0.f);

    // the chunk's values from global memory into registers, as they are stored: nothing is
    // computed from them here, so no instruction waits for them before the chunk in hand
    // has been worked on ...
    auto fetch = [&](int c) {
        const int t0 = c * kChunk;
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
            const int e = tid + NT * i, t = e / KP, d = e % KP;
            const bool in = e < kChunk * KP && t0 + t < n && d < p.kd;
            const size_t r = (size_t)(row0 + t0 + t);
            rq[i] = from_f32<TQ>(0.f);
            rk[i] = from_f32<TQ>(0.f);
            if (in) {
                rq[i] = qp[r * p.q_stride + d];
                rk[i] = kp[r * p.k_stride + d];
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int e = tid + NT * i, t = e / CB, c2 = blockIdx.x * CB + e % CB;
            rv[i] = from_f32<TQ>(0.f);
            if (e < kChunk * CB && t0 + t < n && c2 < p.vd)
                rv[i] = vp[(size_t)(row0 + t0 + t) * p.v_stride + c2];
        }
        if (MODE != SCAN_RETENTION && tid < 2 * kChunk) {
            const int t = tid % kChunk;
            rg = from_f32<TG>(0.f);
            if (t0 + t < n) {
                const size_t r = (size_t)(row0 + t0 + t);
                if (MODE == SCAN_DELTA || MODE == SCAN_GATED)
                    rg = ((const TG*)(tid < kChunk ? p.decay : p.beta))[r * p.H + h];
                else
                    rg = ((const TG*)(tid < kChunk ? p.gate_i : p.gate_f))[r * p.gate_stride + h];
            }
        }
    };
    // ... and from the registers into a buffer, as 32-bit values: q scaled, the memory's
    // gates capped (and the forget gate's log sigmoid taken)
    auto put = [&](float* buf, int c) {
        const int t0 = c * kChunk;
#pragma unroll
        for (int i = 0; i < NQ; ++i)
            if (tid + NT * i < kChunk * KP) {
                buf[tid + NT * i] = to_f32(rq[i]) * p.q_scale;
                buf[kChunk * KP + tid + NT * i] = to_f32(rk[i]);
            }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int e = tid + NT * i, t = e / CB, c2 = blockIdx.x * CB + e % CB;
            if (e < kChunk * CB)
                buf[2 * kChunk * KP + e] =
                    (MODE == SCAN_MEMORY && c2 == p.vd && t0 + t < n) ? 1.0f : to_f32(rv[i]);
        }
        // delta: keep = decay, take = beta; retention: keep = the head's decay, take = 1;
        // memory: the gates i and f, worked on below
        if (tid < 2 * kChunk) {
            float v = to_f32(rg);
            if (MODE == SCAN_RETENTION) v = tid < kChunk ? p.head_decay[h] : 1.0f;
            if (MODE == SCAN_MEMORY) {
                const float bias = (tid < kChunk ? p.bias_i : p.bias_f)[h];
                v = p.cap * tanhf((v + bias) / p.cap);
                if (tid >= kChunk) v = log_sigmoid_f(v);
            }
            buf[2 * kChunk * KP + kChunk * CB + (MODE == SCAN_MEMORY ? 2 * kChunk : 0) + tid] = v;
        }
    };
    // memory: keep and take of the chunk's tokens from its gates and the maximum so far
    auto gates = [&](float* buf, int c) {
        if (MODE != SCAN_MEMORY) return;
        float* keep = buf + 2 * kChunk * KP + kChunk * CB;
        const float* gi = keep + 2 * kChunk;
        const float* gf = gi + kChunk;
        const int t0 = c * kChunk;
        const int t = tid;
        if (t < kChunk && t0 + t < n) {
            const float m0 = m_carry;
            float F = 0.f, best = -INFINITY, before = m0, now = m0;
            // walking s = 0..t: F = F_s, best = max_{u <= s} (i_u - F_u)
            for (int u = 0; u <= t; ++u) {
                before = now;
                F += gf[u];
                best = fmaxf(best, gi[u] - F);
                now = fmaxf(F + m0, best + F);
            }
            keep[t] = expf(gf[t] + before - now);
            keep[kChunk + t] = expf(gi[t] - now);
            if (p.m_out && blockIdx.x == 0) p.m_out[(size_t)(row0 + t0 + t) * p.H + h] = now;
            if (t == kChunk - 1 || t0 + t == n - 1) staged[2 * BUF] = now;    // (read after the barrier)
        }
    };

    if (n_chunks > 0) {
        fetch(0);
        put(staged, 0);
    }
    __syncthreads();
    if (n_chunks > 0) gates(staged, 0);
    __syncthreads();
    if (MODE == SCAN_MEMORY && tid == 0 && n_chunks > 0) m_carry = staged[2 * BUF];
    __syncthreads();
    for (int c = 0; c < n_chunks; ++c) {
        float* buf = staged + (c & 1) * BUF;
        float* next = staged + ((c + 1) & 1) * BUF;
        const bool more = c + 1 < n_chunks;
        if (more) fetch(c + 1);
        const int count = min(kChunk, n - c * kChunk);
        const float* keep = buf + 2 * kChunk * KP + kChunk * CB;
        for (int t = 0; t < count; ++t) {
            float kk[kPerLane], qq[kPerLane];
#pragma unroll
            for (int i = 0; i < kPerLane / 4; ++i) {
                const int d = (i * L + s) * 4;
                const float4 a = *reinterpret_cast<const float4*>(buf + t * KP + d);
                const float4 c4 = *reinterpret_cast<const float4*>(buf + kChunk * KP + t * KP + d);
                qq[4 * i] = a.x; qq[4 * i + 1] = a.y; qq[4 * i + 2] = a.z; qq[4 * i + 3] = a.w;
                kk[4 * i] = c4.x; kk[4 * i + 1] = c4.y; kk[4 * i + 2] = c4.z; kk[4 * i + 3] = c4.w;
            }
            float kq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) kq[i & 3] += kk[i] * qq[i];
            const float kq1 = lanes_sum<L>((kq[0] + kq[1]) + (kq[2] + kq[3]));
            const float keep_t = keep[t], beta_t = keep[kChunk + t];
#pragma unroll
            for (int j = 0; j < NC; ++j) {         // (independent of one another: they overlap)
                const float vj = buf[2 * kChunk * KP + t * CB + cl + j * CW];
                float sk[4] = {0.f, 0.f, 0.f, 0.f}, sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < kPerLane; ++i) {
                    if (MODE == SCAN_DELTA) sk[i & 3] += S[j][i] * kk[i];
                    sq[i & 3] += S[j][i] * qq[i];
                }
                const float sq1 = lanes_sum<L>((sq[0] + sq[1]) + (sq[2] + sq[3]));
                float take;       // S <- keep S + take k
                if (MODE == SCAN_DELTA) {
                    const float sk1 = lanes_sum<L>((sk[0] + sk[1]) + (sk[2] + sk[3]));
                    take = beta_t * (vj - keep_t * sk1);
                } else {
                    take = beta_t * vj;
                }
#pragma unroll
                for (int i = 0; i < kPerLane; ++i) S[j][i] = keep_t * S[j][i] + take * kk[i];
                if (s == 0 && col0 + j * CW < cols)
                    p.out[((size_t)(row0 + c * kChunk + t) * p.H + h) * cols + col0 + j * CW] =
                        keep_t * sq1 + take * kq1;
            }
        }
        if (more) put(next, c + 1);
        __syncthreads();
        if (more) gates(next, c + 1);
        __syncthreads();
        if (MODE == SCAN_MEMORY && tid == 0 && more) m_carry = staged[2 * BUF];
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < NC; ++j) {
        if (!mine[j]) continue;
#pragma unroll
        for (int i = 0; i < kPerLane / 4; ++i) {
            const int d = (i * L + s) * 4;
            if (VEC) {
                if (d < p.kd)
                    *reinterpret_cast<float4*>(mine[j] + d) =
                        make_float4(S[j][4 * i], S[j][4 * i + 1], S[j][4 * i + 2], S[j][4 * i + 3]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (d + e < p.kd) mine[j][d + e] = S[j][4 * i + e];
            }
        }
    }
    if (m_cell && blockIdx.x == 0 && tid == 0) *m_cell = m_carry;
}

template <int MODE, typename TQ, typename TG>
static int launch_scan(const ScanArgs& p, int n_seqs, cudaStream_t s) {
    const int cols = MODE == SCAN_MEMORY ? p.vd + 1 : p.vd;
    const int L = p.kd <= 16 ? 1 : p.kd <= 32 ? 2 : p.kd <= 64 ? 4 : p.kd <= 128 ? 8 : p.kd <= 256 ? 16 : 32;
    const int threads = kScanThreads;
    const int per_block = kColsPerThread * threads / L;       // columns of a block
    const dim3 grid((cols + per_block - 1) / per_block, p.H, n_seqs);
    const bool vec = p.kd % 4 == 0 && p.state_stride % 4 == 0 && ((uintptr_t)p.state % 16) == 0;
    // two buffers and the word that hands the running maximum from chunk to chunk
    const size_t smem = (size_t)(2 * kChunk * (2 * kPerLane * L + kColsPerThread * kScanThreads / L + 4) + 4) * sizeof(float);
#define GO_ONE(LL, VV)                                                                            \
    do {                                                                                          \
        if (smem > 48 * 1024) {                                                                   \
            cudaError_t e = cudaFuncSetAttribute(recurrent_scan_kernel<MODE, TQ, TG, LL, VV>,     \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            SIB_REQUIRE(e == cudaSuccess, "recurrent_scan: %s", cudaGetErrorString(e));           \
        }                                                                                         \
        sib_launch_chained(recurrent_scan_kernel<MODE, TQ, TG, LL, VV>, grid, dim3(threads), smem, s, p); \
    } while (0)
#define GO(LL)                  \
    do {                        \
        if (vec) GO_ONE(LL, true); \
        else GO_ONE(LL, false); \
    } while (0)
    if (L == 1) GO(1);
    else if (L == 2) GO(2);
    else if (L == 4) GO(4);
    else if (L == 8) GO(8);
    else if (L == 16) GO(16);
    else GO(32);
#undef GO
#undef GO_ONE
    return sib_check_launch("recurrent_scan");
}

static int check_scan(const char* what, int rows, int n_seqs, int H, int G, int kd, int vd) {
    SIB_REQUIRE(rows > 0 && n_seqs > 0 && n_seqs < 65536 && H > 0 && H < 65536 && G > 0 && H % G == 0,
                "%s: rows=%d sequences=%d heads=%d key heads=%d", what, rows, n_seqs, H, G);
    SIB_REQUIRE(kd > 0 && kd <= kMaxLanes * kPerLane && vd > 0,
                "%s: key width %d (at most %d) and value width %d", what, kd, kMaxLanes * kPerLane, vd);
    return 0;
}

SIB_EXPORT int sib_delta_prepare(
    const void* proj, long long stride, int dtype, const float* conv_w, const float* a_log,
    const float* dt_bias, float* state, long long state_stride, long long hist_offset, float* qn,
    float* kn, float* vc, float* beta, float* decay, const int* row_pos, const int* row_seq,
    const int* seq_slot, const int* seq_start, const int* seq_end, const int* seq_row0, int rows,
    int n_seqs, int H, int G, int kd, int vd, int taps, void* stream) {
    if (rows == 0) return 0;
    if (check_scan("delta_prepare", rows, n_seqs, H, G, kd, vd)) return -1;
    SIB_REQUIRE(taps >= 1 && taps <= 64, "delta_prepare: %d taps", taps);
    const int channels = 2 * G * kd + H * vd;
    const int units = 2 * G + H + 1;
    SIB_REQUIRE((units + 3) / 4 < 65536, "delta_prepare: too many heads (%d)", H);
    DeltaPrepareArgs p{proj, conv_w, a_log, dt_bias, state, qn, kn, vc, beta, decay, row_pos,
                       row_seq, seq_slot, seq_start, seq_row0, stride, state_stride, hist_offset,
                       H, G, kd, vd, taps};
    cudaStream_t s = (cudaStream_t)stream;
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(delta_prepare_kernel<T>, dim3(rows, (units + 3) / 4),
                                                 dim3(128), 0, s, p));
    int rc = sib_check_launch("delta_prepare");
    if (rc || taps == 1) return rc;
    const dim3 grid((channels + 255) / 256, n_seqs);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(conv_history_kernel<T>, grid, dim3(256), 0, s,
                                                 (const T*)proj, stride, state, state_stride,
                                                 hist_offset, seq_slot, seq_start, seq_end, seq_row0,
                                                 channels, taps));
    return sib_check_launch("conv_history");
}

SIB_EXPORT int sib_delta_scan(const float* qn, const float* kn, const float* vc, const float* decay,
                              const float* beta, float* state, long long state_stride, float* out,
                              const int* seq_slot, const int* seq_start, const int* seq_end,
                              const int* seq_row0, int rows, int n_seqs, int H, int G, int kd, int vd,
                              void* stream) {
    if (rows == 0) return 0;
    if (check_scan("delta_scan", rows, n_seqs, H, G, kd, vd)) return -1;
    ScanArgs p{qn, kn, vc, decay, beta, nullptr, nullptr, nullptr, nullptr, state, out, nullptr,
               seq_slot, seq_start, seq_end, seq_row0, (long long)G * kd, (long long)G * kd,
               (long long)H * vd, 0, state_stride, H, G, kd, vd, 1.0f, 0.f};
    return launch_scan<SCAN_DELTA, float, float>(p, n_seqs, (cudaStream_t)stream);
}

// q | k | v and the two gates' inputs are columns of one projected row (of `dtype`).
SIB_EXPORT int sib_memory_scan(const void* proj, long long stride, int dtype, long long gate_i_col,
                               long long gate_f_col, const float* bias_i, const float* bias_f,
                               float cap, float* state, long long state_stride, float* out,
                               float* m_out, const int* seq_slot, const int* seq_start,
                               const int* seq_end, const int* seq_row0, int rows, int n_seqs, int H,
                               int kd, int vd, void* stream) {
    if (rows == 0) return 0;
    if (check_scan("memory_scan", rows, n_seqs, H, H, kd, vd)) return -1;
    SIB_REQUIRE(cap > 0.f && bias_i && bias_f, "memory_scan: the gates need a cap and biases");
    const size_t esz = dtype == SIB_F32 ? 4 : 2;
    const char* base = (const char*)proj;
    ScanArgs p{base, base + (size_t)H * kd * esz, base + (size_t)2 * H * kd * esz, nullptr, nullptr,
               base + (size_t)gate_i_col * esz, base + (size_t)gate_f_col * esz, bias_i, bias_f,
               state, out, m_out, seq_slot, seq_start, seq_end, seq_row0, stride, stride, stride,
               stride, state_stride, H, H, kd, vd, 1.0f / sqrtf((float)kd), cap};
    SIB_DISPATCH_DTYPE(dtype, return (launch_scan<SCAN_MEMORY, T, T>(p, n_seqs, (cudaStream_t)stream)));
    return 0;
}

// ---------------------------------------------------------------------------
// Retention, step 1: per row and head, q and k rotated by the row's position on their first
// `rot` dimensions in half-split pairs (i, i + rot/2; angle pos * inv_freq[i], taken in
// 32-bit), k then times k_scale; v as it is.  All three leave as 32-bit rows.  `act` 1: q, k
// and v pass SiLU first, value by value in 32-bit (linear attention whose inputs are
// activated projections and nothing else).
// One warp per (row, unit): the q heads, the k heads, the v heads.
// ---------------------------------------------------------------------------
struct RetentionPrepareArgs {
    const void* proj;        // [rows, stride]: q (H kd) | k (H kd) | v (H vd) | ...
    const float* inv_freq;   // [rot / 2] or null
    const int* row_pos;
    float* qn;               // [rows, H kd]
    float* kn;               // [rows, H kd]
    float* vc;               // [rows, H vd]
    long long stride;
    int rows, H, kd, vd, rot;
    float k_scale;
    int act;                 // 0: none, 1: SiLU on q, k and v
};

template <typename T>
__global__ void __launch_bounds__(128) retention_prepare_kernel(RetentionPrepareArgs p) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x;
    const int unit = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (unit >= 3 * p.H) return;
    const T* row = (const T*)p.proj + (size_t)r * p.stride;
    if (unit >= 2 * p.H) {
        const int h = unit - 2 * p.H;
        const T* src = row + (size_t)2 * p.H * p.kd + (size_t)h * p.vd;
        float* dst = p.vc + ((size_t)r * p.H + h) * p.vd;
        for (int d = lane; d < p.vd; d += 32) {
            const float x = to_f32(src[d]);
            dst[d] = p.act ? silu_f(x) : x;
        }
        return;
    }
    const bool is_q = unit < p.H;
    const int h = is_q ? unit : unit - p.H;
    const T* src = row + (size_t)unit * p.kd;
    float* dst = (is_q ? p.qn : p.kn) + ((size_t)r * p.H + h) * p.kd;
    const float pos = (float)p.row_pos[r];
    const int half = p.inv_freq ? p.rot / 2 : 0;
    const float post = is_q ? 1.0f : p.k_scale;
    for (int d = lane; d < p.kd; d += 32) {
        float x = to_f32(src[d]);
        if (p.act) x = silu_f(x);
        if (d < 2 * half) {
            const int i = d < half ? d : d - half;
            const float ang = pos * p.inv_freq[i];
            const float c = cosf(ang), s = sinf(ang);
            float other = to_f32(src[d < half ? d + half : d - half]);
            if (p.act) other = silu_f(other);
            x = d < half ? x * c - other * s : x * c + other * s;
        }
        dst[d] = x * post;
    }
}

SIB_EXPORT int sib_retention_prepare(const void* proj, long long stride, int dtype,
                                     const float* inv_freq, int rot, const int* row_pos, float* qn,
                                     float* kn, float* vc, int rows, int H, int kd, int vd,
                                     float k_scale, int act, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && H > 0 && kd > 0 && vd > 0 && row_pos, "retention_prepare: rows=%d heads=%d widths %d, %d",
                rows, H, kd, vd);
    SIB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= kd && (rot == 0 || inv_freq != nullptr),
                "retention_prepare: %d rotated dimensions of %d", rot, kd);
    SIB_REQUIRE((3 * H + 3) / 4 < 65536, "retention_prepare: too many heads (%d)", H);
    RetentionPrepareArgs p{proj, rot ? inv_freq : nullptr, row_pos, qn, kn, vc, stride, rows, H, kd, vd, rot, k_scale, act};
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(retention_prepare_kernel<T>, dim3(rows, (3 * H + 3) / 4),
                                                 dim3(128), 0, (cudaStream_t)stream, p));
    return sib_check_launch("retention_prepare");
}

// The retention recurrence over prepared 32-bit rows; decay: one value per head.
SIB_EXPORT int sib_retention_scan(const float* qn, const float* kn, const float* vc,
                                  const float* head_decay, float* state, long long state_stride,
                                  float* out, const int* seq_slot, const int* seq_start,
                                  const int* seq_end, const int* seq_row0, int rows, int n_seqs,
                                  int H, int kd, int vd, void* stream) {
    if (rows == 0) return 0;
    if (check_scan("retention_scan", rows, n_seqs, H, H, kd, vd)) return -1;
    SIB_REQUIRE(head_decay != nullptr, "retention_scan: the heads' decays are needed");
    ScanArgs p{qn, kn, vc, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, state, out, nullptr,
               seq_slot, seq_start, seq_end, seq_row0, (long long)H * kd, (long long)H * kd,
               (long long)H * vd, 0, state_stride, H, H, kd, vd, 1.0f, 0.f, head_decay};
    return launch_scan<SCAN_RETENTION, float, float>(p, n_seqs, (cudaStream_t)stream);
}

// The gated recurrence over 32-bit rows: q, k (key heads of kd, G of them) and v (H heads of vd)
// are given with their row strides (they may be columns of one buffer); keep, take: [rows, H].
SIB_EXPORT int sib_gated_scan(const float* q, const float* k, const float* v, long long q_stride,
                              long long k_stride, long long v_stride, const float* keep,
                              const float* take, float* state, long long state_stride, float* out,
                              const int* seq_slot, const int* seq_start, const int* seq_end,
                              const int* seq_row0, int rows, int n_seqs, int H, int G, int kd, int vd,
                              void* stream) {
    if (rows == 0) return 0;
    if (check_scan("gated_scan", rows, n_seqs, H, G, kd, vd)) return -1;
    SIB_REQUIRE(keep != nullptr && take != nullptr, "gated_scan: the rows' factors are needed");
    ScanArgs p{q, k, v, keep, take, nullptr, nullptr, nullptr, nullptr, state, out, nullptr,
               seq_slot, seq_start, seq_end, seq_row0, q_stride, k_stride, v_stride, 0, state_stride,
               H, G, kd, vd, 1.0f, 0.f};
    return launch_scan<SCAN_GATED, float, float>(p, n_seqs, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// The state-space layer around its recurrence.
//   ssm_prepare   per row: the causal convolution (with bias) and silu of the channels
//       x (H vd) | B (G N) | C (G N) of a projected row z | x | B | C | dt, the step size
//       dt = softplus(dt + dt_bias) and the decay exp(-exp(A_log) dt) per head, all 32-bit;
//       inputs before the step come from the slot's history [taps - 1][channels].
//   ssm_finish    y = (o + D_h x) * silu(z), divided by its root mean square in `parts`
//       equal parts of a row, times a weight.
// ---------------------------------------------------------------------------
struct SsmPrepareArgs {
    const void* proj;        // [rows, stride]: z (inner) | x (inner) | B | C | dt (H)
    const float* conv_w;     // [channels, taps], last tap the row's own
    const float* conv_b;     // [channels]
    const float* a_log;      // [H]
    const float* dt_bias;    // [H]
    const float* state;      // [slots, state_stride]; the history starts at hist_offset
    float* xbc;              // [rows, channels]
    float* keep;             // [rows, H]
    float* take;             // [rows, H]
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* seq_start;
    const int* seq_row0;
    long long stride, state_stride, hist_offset;
    int H, inner, channels, taps;
};

template <typename T>
__global__ void __launch_bounds__(256) ssm_prepare_kernel(SsmPrepareArgs p) {
    pdl_trigger();
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= p.channels + p.H) return;
    const int pos = p.row_pos[r];
    const int b = p.row_seq[r];
    const int slot = p.seq_slot[b];
    const int start = p.seq_start[b], row0 = p.seq_row0[b];
    pdl_wait();
    const T* proj = (const T*)p.proj;
    if (c >= p.channels) {
        const int h = c - p.channels;
        const float dt = softplus_f(to_f32(proj[(size_t)r * p.stride + p.inner + p.channels + h]) + p.dt_bias[h]);
        p.keep[(size_t)r * p.H + h] = expf(-expf(p.a_log[h]) * dt);
        p.take[(size_t)r * p.H + h] = dt;
        return;
    }
    const float* hist = slot >= 0 ? p.state + (size_t)slot * p.state_stride + p.hist_offset : nullptr;
    float y = p.conv_b[c];
    for (int j = 0; j < p.taps; ++j) {
        const int at = pos - (p.taps - 1) + j;
        float x = 0.f;
        if (at >= start) x = to_f32(proj[(size_t)(row0 + at - start) * p.stride + p.inner + c]);
        else if (hist) x = hist[(size_t)(at - start + p.taps - 1) * p.channels + c];
        y += p.conv_w[(size_t)c * p.taps + j] * x;
    }
    p.xbc[(size_t)r * p.channels + c] = silu_f(y);
}

SIB_EXPORT int sib_ssm_prepare(const void* proj, long long stride, int dtype, const float* conv_w,
                               const float* conv_b, const float* a_log, const float* dt_bias,
                               float* state, long long state_stride, long long hist_offset,
                               float* xbc, float* keep, float* take, const int* row_pos,
                               const int* row_seq, const int* seq_slot, const int* seq_start,
                               const int* seq_end, const int* seq_row0, int rows, int n_seqs, int H,
                               int inner, int channels, int taps, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && n_seqs > 0 && n_seqs < 65536 && H > 0 && inner > 0 && channels >= inner,
                "ssm_prepare: rows=%d sequences=%d heads=%d inner=%d channels=%d", rows, n_seqs, H,
                inner, channels);
    SIB_REQUIRE(taps >= 1 && taps <= 64, "ssm_prepare: %d taps", taps);
    SsmPrepareArgs p{proj, conv_w, conv_b, a_log, dt_bias, state, xbc, keep, take, row_pos, row_seq,
                     seq_slot, seq_start, seq_row0, stride, state_stride, hist_offset, H, inner,
                     channels, taps};
    cudaStream_t s = (cudaStream_t)stream;
    const int by = (channels + H + 255) / 256;
    SIB_REQUIRE(by < 65536, "ssm_prepare: too many channels (%d)", channels);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(ssm_prepare_kernel<T>, dim3(rows, by), dim3(256), 0, s, p));
    int rc = sib_check_launch("ssm_prepare");
    if (rc || taps == 1) return rc;
    // the history after the step: the channels begin `inner` columns into a projected row
    const size_t esz = dtype == SIB_F32 ? 4 : 2;
    const char* first = (const char*)proj + (size_t)inner * esz;
    const dim3 grid((channels + 255) / 256, n_seqs);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(conv_history_kernel<T>, grid, dim3(256), 0, s,
                                                 (const T*)first, stride, state, state_stride,
                                                 hist_offset, seq_slot, seq_start, seq_end, seq_row0,
                                                 channels, taps));
    return sib_check_launch("conv_history");
}

// One block per (row, part of the row).
template <typename T>
__global__ void __launch_bounds__(128)
ssm_finish_kernel(const float* __restrict__ o, const float* __restrict__ xbc, long long x_stride,
                  const T* __restrict__ z, long long z_stride, const float* __restrict__ skip,
                  const float* __restrict__ w, T* __restrict__ y, int rows, int inner, int vd,
                  int parts, float eps) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const size_t r = blockIdx.x / parts;
    const int part = (int)(blockIdx.x % parts), len = inner / parts, e0 = part * len;
    auto value = [&](int e) {
        const float zz = to_f32(z[r * z_stride + e]);
        return (o[r * inner + e] + skip[e / vd] * xbc[r * x_stride + e]) * silu_f(zz);
    };
    float ss = 0.f;
    for (int e = e0 + threadIdx.x; e < e0 + len; e += blockDim.x) {
        const float v = value(e);
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)len + eps);
    for (int e = e0 + threadIdx.x; e < e0 + len; e += blockDim.x)
        y[r * inner + e] = from_f32<T>(value(e) * inv * w[e]);
}

SIB_EXPORT int sib_ssm_finish(const float* o, const float* xbc, long long x_stride, const void* z,
                              long long z_stride, const float* skip, const float* w, void* y,
                              int dtype, int rows, int inner, int vd, int parts, float eps,
                              void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && inner > 0 && vd > 0 && inner % vd == 0 && parts > 0 && inner % parts == 0,
                "ssm_finish: rows=%d inner=%d head width=%d parts=%d", rows, inner, vd, parts);
    const long long blocks = (long long)rows * parts;
    SIB_REQUIRE(blocks < (1ll << 31), "ssm_finish: too many rows (%d)", rows);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(ssm_finish_kernel<T>, dim3((unsigned)blocks), dim3(128),
                                                 0, (cudaStream_t)stream, o, xbc, x_stride,
                                                 (const T*)z, z_stride, skip, w, (T*)y, rows, inner,
                                                 vd, parts, eps));
    return sib_check_launch("ssm_finish");
}

// ---------------------------------------------------------------------------
// After either recurrence: each head's output divided by its root mean square, times a
// weight, times an activated gate.
//   x = o[r, h, :vd]            (memory: divided by max(|o[r, h, vd]|, e^-m[r, h]) + 1e-6)
//   y[r, h, :] = x / sqrt(mean(x^2) + eps) * w[h * w_stride + :] * act(gate[r, h * vd + :])
// act: 0 silu, 1 sigmoid; w null: no weight.  One warp per (row, head).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ m, const float* __restrict__ w,
                      int w_stride, const T* __restrict__ gate, long long gate_stride,
                      T* __restrict__ y, int rows, int H, int vd, int cols, float eps, int act) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (unit >= (long long)rows * H) return;
    const size_t r = unit / H;
    const int h = (int)(unit % H);
    const float* x = o + (size_t)unit * cols;
    float scale = 1.f;
    if (m) scale = 1.0f / (fmaxf(fabsf(x[vd]), expf(-m[unit])) + 1e-6f);
    float ss = 0.f;
    for (int e = lane; e < vd; e += 32) {
        const float v = x[e] * scale;
        ss += v * v;
    }
    const float inv = scale / sqrtf(warp_sum(ss) / (float)vd + eps);
    for (int e = lane; e < vd; e += 32) {
        const float z = to_f32(gate[r * gate_stride + (size_t)h * vd + e]);
        const float a = act == 0 ? silu_f(z) : sigmoid_f(z);
        y[(size_t)unit * vd + e] = from_f32<T>(x[e] * inv * (w ? w[(size_t)h * w_stride + e] : 1.0f) * a);
    }
}

// The same for heads of many columns (all heads normed together count as one): a block per
// (row, head), its threads sharing the columns.
template <typename T>
__global__ void __launch_bounds__(256)
wide_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ m, const float* __restrict__ w,
                      int w_stride, const T* __restrict__ gate, long long gate_stride,
                      T* __restrict__ y, int H, int vd, int cols, float eps, int act) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const size_t unit = blockIdx.x;
    const size_t r = unit / H;
    const int h = (int)(unit % H);
    const float* x = o + unit * cols;
    float scale = 1.f;
    if (m) scale = 1.0f / (fmaxf(fabsf(x[vd]), expf(-m[unit])) + 1e-6f);
    float ss = 0.f;
    for (int e = threadIdx.x; e < vd; e += blockDim.x) {
        const float v = x[e] * scale;
        ss += v * v;
    }
    const float inv = scale / sqrtf(block_sum(ss, scratch) / (float)vd + eps);
    for (int e = threadIdx.x; e < vd; e += blockDim.x) {
        const float z = to_f32(gate[r * gate_stride + (size_t)h * vd + e]);
        const float a = act == 0 ? silu_f(z) : sigmoid_f(z);
        y[unit * vd + e] = from_f32<T>(x[e] * inv * (w ? w[(size_t)h * w_stride + e] : 1.0f) * a);
    }
}

SIB_EXPORT int sib_head_norm_gate(const float* o, const float* m, const float* w, int w_stride,
                                  const void* gate, long long gate_stride, void* y, int dtype,
                                  int rows, int H, int vd, int cols, float eps, int act,
                                  void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && H > 0 && vd > 0 && cols >= vd && (m == nullptr || cols > vd),
                "head_norm_gate: rows=%d heads=%d width=%d of %d", rows, H, vd, cols);
    const long long blocks = ((long long)rows * H + 3) / 4;
    SIB_REQUIRE(blocks < (1ll << 29), "head_norm_gate: too many rows (%d)", rows);
    if (vd >= 512) {
        SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(wide_norm_gate_kernel<T>, dim3((unsigned)((long long)rows * H)),
                                                     dim3(256), 0, (cudaStream_t)stream, o, m, w, w_stride,
                                                     (const T*)gate, gate_stride, (T*)y, H, vd, cols, eps, act));
        return sib_check_launch("head_norm_gate");
    }
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(head_norm_gate_kernel<T>, dim3((unsigned)blocks),
                                                 dim3(128), 0, (cudaStream_t)stream, o, m, w, w_stride,
                                                 (const T*)gate, gate_stride, (T*)y, rows, H, vd, cols,
                                                 eps, act));
    return sib_check_launch("head_norm_gate");
}
