// What lies between the q|k|v product and the attention kernel for mixers whose heads are
// worked on first, and what lies between the attention kernel and the output product:
//
//   head_prepare   per row and head, in 32-bit:
//       x  = proj + bias                                   (bias optional)
//       q, k: x <- x / sqrt(mean(x^2) + eps) * w           (w optional: no norm without it)
//       q, k: the first `rot` dimensions rotated in half-split pairs (i, i + rot/2), or in
//             neighbouring pairs (2i, 2i + 1), by the angle pos * inv_freq[i]; the rest pass
//       v:    v <- (1 - lambda) v + lambda v_first         (v_first optional)
//     q, k and v go to a packed buffer whose heads are all `pad` wide (key width and value
//     width may differ: the narrower one is filled up with zeros, which changes neither a
//     score nor a weighted sum), and k and v also into the paged cache of that width.
//
//   head_gate      y[r, h, :vd] = o[r, h, :vd] * sigmoid(gate[r, h])    (gate optional)
//     which also drops the filled-up columns again.
//
// Plain counterpart: tests/plain_karupel.py attention_mixer().
#include "common.cuh"

struct HeadPrepareArgs {
    const void* proj;          // [rows, proj_stride]: q heads | k heads | v heads | ...
    void* qkv;                 // [rows, (n_heads + 2 n_kv) * pad]
    const float* bias;         // [n_heads * kd + n_kv * kd + n_kv * vd] or null
    const float* q_gain;       // [kd] or null
    const float* k_gain;       // [kd] or null
    const float* inv_freq;     // [rot / 2] or null
    const void* v_first;       // row r, kv head g at v_first + r * v_first_stride + g * v_first_pad; or null
    const float* lambda;       // one value on the device (with v_first)
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* seq_end;
    void* k_pool;              // [pages, n_kv, page_tokens, pad]; null: nothing is stored
    void* v_pool;
    const int* page_table;
    long long proj_stride, v_first_stride;
    int n_heads, n_kv, kd, vd, pad, rot, v_first_pad;
    int max_pages, page_tokens, ring_tokens;
    float eps;
    int neighbours;            // 1: the rotated pairs are (2i, 2i + 1) instead of (i, i + rot/2)
};

// One warp per (row, head unit); a block takes 4 units of one row.
template <typename T>
__global__ void __launch_bounds__(128) head_prepare_kernel(HeadPrepareArgs p) {
    extern __shared__ float staged[];          // [4][pad]
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x;
    const int unit = blockIdx.y * 4 + warp;
    const int units = p.n_heads + 2 * p.n_kv;
    if (unit >= units) return;
    float* mine = staged + (size_t)warp * p.pad;
    const bool is_q = unit < p.n_heads;
    const bool is_v = unit >= p.n_heads + p.n_kv;
    const int width = is_v ? p.vd : p.kd;
    // where the unit's values start in a row of proj (and in bias)
    const int col = is_q ? unit * p.kd
                         : !is_v ? p.n_heads * p.kd + (unit - p.n_heads) * p.kd
                                 : (p.n_heads + p.n_kv) * p.kd + (unit - p.n_heads - p.n_kv) * p.vd;
    const int pos = p.row_pos[r];
    T* dst = nullptr;
    if (!is_q && p.k_pool) {
        const int b = p.row_seq[r];
        const int slot = p.seq_slot[b];
        bool keep = slot >= 0;               // (a filling row's sequence holds no slot)
        int cell = pos;
        if (keep && p.ring_tokens > 0) {
            keep = pos >= p.seq_end[b] - p.ring_tokens;
            cell = pos % p.ring_tokens;
        }
        if (keep) {
            const int page = p.page_table[(size_t)slot * p.max_pages + cell / p.page_tokens];
            const int g = is_v ? unit - p.n_heads - p.n_kv : unit - p.n_heads;
            T* pool = (T*)(is_v ? p.v_pool : p.k_pool);
            dst = pool + (((size_t)page * p.n_kv + g) * p.page_tokens + cell % p.page_tokens) * p.pad;
        }
    }
    pdl_wait();
    const T* src = (const T*)p.proj + (size_t)r * p.proj_stride + col;
    float ss = 0.f;
    for (int d = lane; d < width; d += 32) {
        float x = to_f32(src[d]);
        if (p.bias) x += p.bias[col + d];
        mine[d] = x;
        ss += x * x;
    }
    T* out = (T*)p.qkv + (size_t)r * units * p.pad + (size_t)unit * p.pad;
    if (is_v) {
        const T* first = p.v_first
            ? (const T*)p.v_first + (size_t)r * p.v_first_stride + (size_t)(unit - p.n_heads - p.n_kv) * p.v_first_pad
            : nullptr;
        const float lam = first ? *p.lambda : 0.f;
        for (int d = lane; d < p.pad; d += 32) {
            float x = 0.f;
            if (d < width) {
                x = mine[d];
                if (first) x = (1.f - lam) * x + lam * to_f32(first[d]);
            }
            const T y = from_f32<T>(x);
            out[d] = y;
            if (dst) dst[d] = y;
        }
        return;
    }
    const float* gain = is_q ? p.q_gain : p.k_gain;
    float inv = 1.f;
    if (gain) inv = 1.0f / sqrtf(warp_sum(ss) / (float)width + p.eps);
    __syncwarp();
    if (gain)
        for (int d = lane; d < width; d += 32) mine[d] = mine[d] * inv * gain[d];
    __syncwarp();
    const int half = p.inv_freq ? p.rot / 2 : 0;
    for (int d = lane; d < p.pad; d += 32) {
        float x = 0.f;
        if (d < width) {
            x = mine[d];
            if (d < 2 * half && p.neighbours) {
                const float ang = (float)pos * p.inv_freq[d >> 1];
                const float c = cosf(ang), s = sinf(ang);
                x = (d & 1) ? x * c + mine[d - 1] * s : x * c - mine[d + 1] * s;
            } else if (d < 2 * half) {
                const int i = d < half ? d : d - half;
                const float ang = (float)pos * p.inv_freq[i];
                const float c = cosf(ang), s = sinf(ang);
                x = d < half ? x * c - mine[d + half] * s : x * c + mine[d - half] * s;
            }
        }
        const T y = from_f32<T>(x);
        out[d] = y;
        if (dst) dst[d] = y;
    }
}

SIB_EXPORT int sib_head_prepare(
    const void* proj, long long proj_stride, void* qkv, int dtype, const float* bias,
    const float* q_gain, const float* k_gain, float eps, const float* inv_freq, int rot,
    const void* v_first, long long v_first_stride, int v_first_pad, const float* lambda, const int* row_pos,
    const int* row_seq, const int* seq_slot, const int* seq_end, void* k_pool, void* v_pool,
    const int* page_table, int max_pages, int page_tokens, int ring_tokens, int rows, int n_heads,
    int n_kv, int kd, int vd, int pad, int neighbours, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && n_heads > 0 && n_kv >= 0 && kd > 0 && vd > 0,
                "head_prepare: rows=%d heads=%d kv_heads=%d key width=%d value width=%d", rows,
                n_heads, n_kv, kd, vd);
    SIB_REQUIRE(pad >= kd && pad >= vd, "head_prepare: heads of %d and %d do not fit a width of %d",
                kd, vd, pad);
    SIB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= kd && (rot == 0 || inv_freq != nullptr),
                "head_prepare: %d rotated dimensions of %d", rot, kd);
    SIB_REQUIRE(row_pos != nullptr, "head_prepare: positions are needed");
    SIB_REQUIRE(k_pool == nullptr || (v_pool && page_table && row_seq && seq_slot && seq_end &&
                                      page_tokens > 0 && max_pages > 0),
                "head_prepare: incomplete cache description");
    SIB_REQUIRE(v_first == nullptr || (lambda != nullptr && v_first_pad >= vd),
                "head_prepare: mixing values needs lambda and heads of at least %d", vd);
    HeadPrepareArgs p{proj, qkv, bias, q_gain, k_gain, rot ? inv_freq : nullptr, v_first, lambda,
                      row_pos, row_seq, seq_slot, seq_end, k_pool, v_pool, page_table, proj_stride,
                      v_first_stride, n_heads, n_kv, kd, vd, pad, rot, v_first_pad, max_pages, page_tokens,
                      ring_tokens, eps, neighbours};
    const int units = n_heads + 2 * n_kv;
    const size_t smem = (size_t)4 * pad * sizeof(float);
    SIB_REQUIRE(smem <= 48 * 1024, "head_prepare: heads of %d are too wide", pad);
    SIB_REQUIRE(rows < 65536 * 32767ll && (units + 3) / 4 < 65536, "head_prepare: too many rows");
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(head_prepare_kernel<T>, dim3(rows, (units + 3) / 4),
                                                 dim3(128), smem, (cudaStream_t)stream, p));
    return sib_check_launch("head_prepare");
}

// ---------------------------------------------------------------------------
// pool_store: one more cell per block of `pool` positions for an attention that sees far
// tokens only as blocks: the mean of the block's keys and the mean of its values, as the
// packed rows and the cache hold them, written into a second paged cache whose cell b stands
// for the positions b pool .. b pool + pool - 1.  A block is written by the step that brings
// its last position; positions of the block that earlier steps brought are read from the
// (ring) cache, the step's own from its packed rows.
// grid (blocks a sequence can complete in this step, kv heads, sequences); thread d of pad.
// ---------------------------------------------------------------------------
struct PoolStoreArgs {
    const void* qkv;           // [rows, (n_heads + 2 n_kv) * pad]
    const void* k_pool;        // [pages, n_kv, page_tokens, pad]: earlier positions
    const void* v_pool;
    const int* page_table;
    void* pk_pool;             // [pages, n_kv, pool_page_tokens, pad]: the blocks' cells
    void* pv_pool;
    const int* pool_table;
    const int* seq_slot;
    const int* seq_start;
    const int* seq_end;
    const int* seq_row0;
    int n_heads, n_kv, pad, pool;
    int max_pages, page_tokens, ring_tokens, pool_max_pages, pool_page_tokens;
};

template <typename T>
__global__ void pool_store_kernel(PoolStoreArgs p) {
    pdl_trigger();
    const int b = blockIdx.z, g = blockIdx.y;
    const int slot = p.seq_slot[b];
    const int start = p.seq_start[b], end = p.seq_end[b], row0 = p.seq_row0[b];
    const int block = start / p.pool + blockIdx.x;
    if (slot < 0 || block >= end / p.pool) return;
    pdl_wait();
    const int units = p.n_heads + 2 * p.n_kv;
    const int page = p.pool_table[(size_t)slot * p.pool_max_pages + block / p.pool_page_tokens];
    const size_t cell = (((size_t)page * p.n_kv + g) * p.pool_page_tokens + block % p.pool_page_tokens) * p.pad;
    for (int d = threadIdx.x; d < 2 * p.pad; d += blockDim.x) {
        const bool is_v = d >= p.pad;
        const int e = is_v ? d - p.pad : d;
        float sum = 0.f;
        for (int j = block * p.pool; j < (block + 1) * p.pool; ++j) {
            if (j >= start) {
                const int unit = p.n_heads + (is_v ? p.n_kv : 0) + g;
                sum += to_f32(((const T*)p.qkv)[((size_t)(row0 + j - start) * units + unit) * p.pad + e]);
            } else {
                const int at = p.ring_tokens > 0 ? j % p.ring_tokens : j;
                const int pg = p.page_table[(size_t)slot * p.max_pages + at / p.page_tokens];
                const T* src = (const T*)(is_v ? p.v_pool : p.k_pool);
                sum += to_f32(src[(((size_t)pg * p.n_kv + g) * p.page_tokens + at % p.page_tokens) * p.pad + e]);
            }
        }
        ((T*)(is_v ? p.pv_pool : p.pk_pool))[cell + e] = from_f32<T>(sum / (float)p.pool);
    }
}

SIB_EXPORT int sib_pool_store(const void* qkv, const void* k_pool, const void* v_pool,
                              const int* page_table, int max_pages, int page_tokens, int ring_tokens,
                              void* pk_pool, void* pv_pool, const int* pool_table, int pool_max_pages,
                              int pool_page_tokens, const int* seq_slot, const int* seq_start,
                              const int* seq_end, const int* seq_row0, int dtype, int n_seqs,
                              int max_count, int n_heads, int n_kv, int pad, int pool, void* stream) {
    if (n_seqs == 0 || max_count == 0) return 0;
    SIB_REQUIRE(n_seqs > 0 && n_seqs < 65536 && n_kv > 0 && n_kv < 65536 && pad > 0 && pool > 0 && max_count > 0,
                "pool_store: sequences=%d kv_heads=%d width=%d pool=%d", n_seqs, n_kv, pad, pool);
    SIB_REQUIRE(qkv && k_pool && v_pool && page_table && pk_pool && pv_pool && pool_table &&
                    page_tokens > 0 && max_pages > 0 && pool_page_tokens > 0 && pool_max_pages > 0,
                "pool_store: incomplete cache description");
    PoolStoreArgs p{qkv, k_pool, v_pool, page_table, pk_pool, pv_pool, pool_table, seq_slot, seq_start,
                    seq_end, seq_row0, n_heads, n_kv, pad, pool, max_pages, page_tokens, ring_tokens,
                    pool_max_pages, pool_page_tokens};
    // a step of c positions completes at most (c + pool - 1) / pool blocks of a sequence
    const dim3 grid((max_count + pool - 1) / pool, n_kv, n_seqs);
    const int threads = 2 * pad < 256 ? (2 * pad + 31) / 32 * 32 : 256;
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(pool_store_kernel<T>, grid, dim3(threads), 0,
                                                 (cudaStream_t)stream, p));
    return sib_check_launch("pool_store");
}

// y[r, h * vd + e] = o[r, h * pad + e] * sigmoid(gate[r * gate_stride + h])
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ o, const T* __restrict__ gate,
                                 long long gate_stride, T* __restrict__ y, int n_heads, int vd,
                                 int pad, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / ((size_t)n_heads * vd);
        const int rest = (int)(idx - r * (size_t)n_heads * vd);
        const int h = rest / vd, e = rest - h * vd;
        float x = to_f32(o[(r * n_heads + h) * (size_t)pad + e]);
        if (gate) x *= 1.0f / (1.0f + expf(-to_f32(gate[r * gate_stride + h])));
        y[idx] = from_f32<T>(x);
    }
}

SIB_EXPORT int sib_head_gate(const void* o, const void* gate, long long gate_stride, void* y,
                             int dtype, int rows, int n_heads, int vd, int pad, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && n_heads > 0 && vd > 0 && pad >= vd,
                "head_gate: rows=%d heads=%d width=%d of %d", rows, n_heads, vd, pad);
    const size_t total = (size_t)rows * n_heads * vd;
    const size_t want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(head_gate_kernel<T>, dim3(blocks), dim3(256), 0,
                                                 (cudaStream_t)stream, (const T*)o, (const T*)gate,
                                                 gate_stride, (T*)y, n_heads, vd, pad, total));
    return sib_check_launch("head_gate");
}

// ---------------------------------------------------------------------------
// latent_prepare: what lies between the projections and the attention kernel of an
// attention whose keys and values of all heads are made from ONE low-rank row per position
// (the latent c, width `rank`) plus ONE rotated key part shared by the heads (width `rd`).
// The scores are taken against the latent itself: with k_h = U_h c,
//     <q_h, k_h> = <U_h^T q_h, c>,
// so a query head becomes [U_h^T q_h | rotated part of q_h] (the product with U_h is the
// caller's, its result `q_lat`), a position's key row becomes [c | rotated shared part], both
// `pad` wide with zeros behind, and a value is the key row's first `rank` columns.
//
// Per row, in 32-bit:
//   key unit:   c = x / sqrt(mean(x^2) + eps) * w   over x = down[:rank];   the shared part
//               down[rank : rank + rd] rotated;  the row goes to `k_rows` and to the cache
//   query unit: [q_lat[h, r, :] | q_h's last rd columns rotated | 0]  ->  q_rows[r, h, :]
// Rotation: the first `rot` (<= rd) columns in neighbouring pairs (2i, 2i + 1) by the angle
// pos * inv_freq[i].
// Plain counterpart: tests/plain_vavupel.py latent_attention().
// ---------------------------------------------------------------------------
struct LatentPrepareArgs {
    const void* proj;          // [rows, proj_stride]: query heads of (qd + rd) | down (rank + rd) | ...
    const void* q_lat;         // [n_heads, rows, rank]
    void* q_rows;              // [rows, n_heads * pad]
    void* k_rows;              // [rows, pad]
    const float* c_gain;       // [rank]
    const float* inv_freq;     // [rot / 2] or null
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* seq_end;
    void* k_pool;              // [pages, 1, page_tokens, pad]; null: nothing is stored
    const int* page_table;
    long long proj_stride;
    int rows, n_heads, qd, rd, rank, pad, rot;
    int max_pages, page_tokens, ring_tokens;
    float eps;
    // the down projection's rows (rank + rd) where they do not follow the query heads in `proj`
    // (queries that come from a product of their own); null: they do
    const void* down;
    long long down_stride;
};

template <typename T>
__device__ __forceinline__ float rotated_pair(const T* part, int d, int rot, const float* inv_freq,
                                              float pos) {
    float x = to_f32(part[d]);
    if (d < rot) {
        const float ang = pos * inv_freq[d >> 1];
        const float c = cosf(ang), s = sinf(ang);
        x = (d & 1) ? x * c + to_f32(part[d - 1]) * s : x * c - to_f32(part[d + 1]) * s;
    }
    return x;
}

// One warp per (row, unit): n_heads query units, then the key unit.
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(LatentPrepareArgs p) {
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x;
    const int unit = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (unit > p.n_heads) return;
    const float pos = (float)p.row_pos[r];
    const int rot = p.inv_freq ? p.rot : 0;
    pdl_wait();
    const T* row = (const T*)p.proj + (size_t)r * p.proj_stride;
    if (unit < p.n_heads) {
        if (p.q_lat == nullptr) return;      // (the caller wants the key rows only)
        const T* lat = (const T*)p.q_lat + ((size_t)unit * p.rows + r) * p.rank;
        const T* part = row + (size_t)unit * (p.qd + p.rd) + p.qd;
        T* out = (T*)p.q_rows + ((size_t)r * p.n_heads + unit) * p.pad;
        for (int d = lane; d < p.pad; d += 32) {
            T y = from_f32<T>(0.f);
            if (d < p.rank) y = lat[d];
            else if (d < p.rank + p.rd) y = from_f32<T>(rotated_pair<T>(part, d - p.rank, rot, p.inv_freq, pos));
            out[d] = y;
        }
        return;
    }
    T* dst = nullptr;
    if (p.k_pool) {
        const int b = p.row_seq[r];
        const int slot = p.seq_slot[b];
        const int at = p.row_pos[r];
        bool keep = slot >= 0;               // (a filling row's sequence holds no slot)
        int cell = at;
        if (keep && p.ring_tokens > 0) {
            keep = at >= p.seq_end[b] - p.ring_tokens;
            cell = at % p.ring_tokens;
        }
        if (keep) {
            const int page = p.page_table[(size_t)slot * p.max_pages + cell / p.page_tokens];
            dst = (T*)p.k_pool + ((size_t)page * p.page_tokens + cell % p.page_tokens) * p.pad;
        }
    }
    const T* down = p.down ? (const T*)p.down + (size_t)r * p.down_stride
                           : row + (size_t)p.n_heads * (p.qd + p.rd);
    float ss = 0.f;
    for (int d = lane; d < p.rank; d += 32) {
        const float x = to_f32(down[d]);
        ss += x * x;
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)p.rank + p.eps);
    T* out = (T*)p.k_rows + (size_t)r * p.pad;
    for (int d = lane; d < p.pad; d += 32) {
        float x = 0.f;
        if (d < p.rank) x = to_f32(down[d]) * inv * p.c_gain[d];
        else if (d < p.rank + p.rd) x = rotated_pair<T>(down + p.rank, d - p.rank, rot, p.inv_freq, pos);
        const T y = from_f32<T>(x);
        out[d] = y;
        if (dst) dst[d] = y;
    }
}

SIB_EXPORT int sib_latent_prepare(
    const void* proj, long long proj_stride, const void* q_lat, void* q_rows, void* k_rows, int dtype,
    const float* c_gain, float eps, const float* inv_freq, int rot, const int* row_pos,
    const int* row_seq, const int* seq_slot, const int* seq_end, void* k_pool, const int* page_table,
    int max_pages, int page_tokens, int ring_tokens, int rows, int n_heads, int qd, int rd, int rank,
    int pad, const void* down, long long down_stride, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && n_heads > 0 && qd > 0 && rd >= 0 && rank > 0 && pad >= rank + rd,
                "latent_prepare: rows=%d heads=%d widths %d + %d, rank %d in rows of %d", rows, n_heads,
                qd, rd, rank, pad);
    SIB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= rd && (rot == 0 || inv_freq != nullptr),
                "latent_prepare: %d rotated dimensions of %d", rot, rd);
    SIB_REQUIRE(row_pos && c_gain && k_rows && (q_lat != nullptr) == (q_rows != nullptr),
                "latent_prepare: an argument is missing");
    SIB_REQUIRE(k_pool == nullptr || (page_table && row_seq && seq_slot && seq_end && page_tokens > 0 &&
                                      max_pages > 0),
                "latent_prepare: incomplete cache description");
    SIB_REQUIRE((n_heads + 4) / 4 < 65536, "latent_prepare: too many heads (%d)", n_heads);
    LatentPrepareArgs p{proj, q_lat, q_rows, k_rows, c_gain, rot ? inv_freq : nullptr, row_pos, row_seq,
                        seq_slot, seq_end, k_pool, page_table, proj_stride, rows, n_heads, qd, rd, rank,
                        pad, rot, max_pages, page_tokens, ring_tokens, eps, down, down_stride};
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(latent_prepare_kernel<T>, dim3(rows, (n_heads + 4) / 4),
                                                 dim3(128), 0, (cudaStream_t)stream, p));
    return sib_check_launch("latent_prepare");
}

// ---------------------------------------------------------------------------
// latent_expand: packed rows for the prompt attention kernels when keys and values are
// made per head from the latent (k_h = U_h c and v_h = V_h c, the caller's products):
//   query head h:  [a_h (qd) | its last rd columns rotated | 0]
//   key head h:    [k_h (qd) | the row's shared rotated part, as latent_prepare left it in
//                   k_rows[r, rank : rank + rd] | 0]
//   value head h:  [v_h (vd) | 0]
// every head `hw` wide: qkv[r] = queries | keys | values.  One warp per (row, unit).
// ---------------------------------------------------------------------------
struct LatentExpandArgs {
    const void* proj;          // [rows, proj_stride]: query heads of (qd + rd) | ...
    const void* k_rows;        // [rows, pad]
    const void* k_heads;       // [rows, n_heads * qd]
    const void* v_heads;       // [rows, n_heads * vd]
    void* qkv;                 // [rows, 3 * n_heads * hw]
    const float* inv_freq;
    const int* row_pos;
    long long proj_stride;
    int rows, n_heads, qd, rd, vd, rank, pad, hw, rot;
};

template <typename T>
__global__ void __launch_bounds__(128) latent_expand_kernel(LatentExpandArgs p) {
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x;
    const int unit = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (unit >= 3 * p.n_heads) return;
    const float pos = (float)p.row_pos[r];
    const int rot = p.inv_freq ? p.rot : 0;
    pdl_wait();
    const int kind = unit / p.n_heads, h = unit % p.n_heads;
    T* out = (T*)p.qkv + ((size_t)r * 3 * p.n_heads + unit) * p.hw;
    const T zero = from_f32<T>(0.f);
    if (kind == 0) {
        const T* head = (const T*)p.proj + (size_t)r * p.proj_stride + (size_t)h * (p.qd + p.rd);
        for (int d = lane; d < p.hw; d += 32) {
            T y = zero;
            if (d < p.qd) y = head[d];
            else if (d < p.qd + p.rd) y = from_f32<T>(rotated_pair<T>(head + p.qd, d - p.qd, rot, p.inv_freq, pos));
            out[d] = y;
        }
    } else if (kind == 1) {
        const T* kh = (const T*)p.k_heads + ((size_t)r * p.n_heads + h) * p.qd;
        const T* shared = (const T*)p.k_rows + (size_t)r * p.pad + p.rank;
        for (int d = lane; d < p.hw; d += 32)
            out[d] = d < p.qd ? kh[d] : (d < p.qd + p.rd ? shared[d - p.qd] : zero);
    } else {
        const T* vh = (const T*)p.v_heads + ((size_t)r * p.n_heads + h) * p.vd;
        for (int d = lane; d < p.hw; d += 32) out[d] = d < p.vd ? vh[d] : zero;
    }
}

SIB_EXPORT int sib_latent_expand(const void* proj, long long proj_stride, const void* k_rows,
                                 const void* k_heads, const void* v_heads, void* qkv, int dtype,
                                 const float* inv_freq, int rot, const int* row_pos, int rows,
                                 int n_heads, int qd, int rd, int vd, int rank, int pad, int hw,
                                 void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && n_heads > 0 && qd > 0 && rd >= 0 && vd > 0 && hw >= qd + rd && hw >= vd &&
                    pad >= rank + rd,
                "latent_expand: rows=%d heads=%d widths %d + %d and %d in heads of %d", rows, n_heads, qd,
                rd, vd, hw);
    SIB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= rd && (rot == 0 || inv_freq != nullptr),
                "latent_expand: %d rotated dimensions of %d", rot, rd);
    SIB_REQUIRE(proj && k_rows && k_heads && v_heads && qkv && row_pos, "latent_expand: an argument is missing");
    SIB_REQUIRE((3 * n_heads + 3) / 4 < 65536, "latent_expand: too many heads (%d)", n_heads);
    LatentExpandArgs p{proj, k_rows, k_heads, v_heads, qkv, rot ? inv_freq : nullptr, row_pos, proj_stride,
                       rows, n_heads, qd, rd, vd, rank, pad, hw, rot};
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(latent_expand_kernel<T>, dim3(rows, (3 * n_heads + 3) / 4),
                                                 dim3(128), 0, (cudaStream_t)stream, p));
    return sib_check_launch("latent_expand");
}
