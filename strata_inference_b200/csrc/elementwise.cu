// Embedding gather with scale, gated activations (tanh-GELU, SiLU), soft cap, row copies.
//
// Plain counterparts: tests/plain_gemma2.py embed(), gelu_tanh(), lm_head().
// Reference formulas: src/backend/cpu.rs:1086-1136 (row gather),
// src/model/layer.rs:1285-1288 (scale), src/backend/cpu.rs:1190-1199 (GeGLU).
#include "common.cuh"

// out[r, :] = scale * table[tokens[r], :], accumulated stream in f32.
template <typename T>
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                  float* __restrict__ out, int hidden, float scale) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const T* src = table + (size_t)tokens[r] * hidden;
    float* dst = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(src[i]) * scale;
}

SIB_EXPORT int sib_embed_rows(const int* tokens, const void* table, int table_dtype, float* out,
                              int rows, int hidden, float scale, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && hidden > 0, "embed_rows: rows=%d hidden=%d", rows, hidden);
    SIB_DISPATCH_DTYPE(table_dtype,
                       sib_launch_chained(embed_rows_kernel<T>, dim3(rows), dim3(256), 0,
                                          (cudaStream_t)stream, tokens, (const T*)table, out, hidden,
                                          scale));
    return sib_check_launch("embed_rows");
}

__device__ __forceinline__ float gelu_tanh(float g) {
    const float c = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
}

__device__ __forceinline__ float silu_act(float g) { return g / (1.0f + expf(-g)); }

enum { ACT_GELU_TANH = 0, ACT_SILU = 1 };
__device__ __forceinline__ float gate_act(float g, int act) {
    return act == ACT_SILU ? silu_act(g) : gelu_tanh(g);
}

// out[r, i] = act(gate(r, i)) * up(r, i).  The two halves of gate_up[r, :]
// are laid out either as [all gates | all ups] (group == 0) or in groups of
// `group` gates followed by the `group` matching ups.
template <typename T>
__global__ void gelu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter,
                                int group, size_t total, int act) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / inter;
        const int i = (int)(idx - r * inter);
        const T* row = gate_up + r * 2 * (size_t)inter;
        const int gi = group ? (i / group) * 2 * group + i % group : i;
        const int ui = group ? gi + group : inter + i;
        const float g = to_f32(row[gi]), u = to_f32(row[ui]);
        out[idx] = from_f32<T>(gate_act(g, act) * u);
    }
}

// The bfloat16 case with groups of 8: a group is 32 contiguous bytes (8 gates,
// 8 ups) and gives 16 contiguous bytes of output; one thread per group, every
// access 16 bytes wide.
__global__ void gelu_mul_group8_bf16_kernel(const uint4* __restrict__ gate_up,
                                            uint4* __restrict__ out, size_t groups, int act) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint4 gv = gate_up[2 * i], uv = gate_up[2 * i + 1];
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xffff0000u);
            const float u0 = __uint_as_float(uw[k] << 16), u1 = __uint_as_float(uw[k] & 0xffff0000u);
            const __nv_bfloat162 o = __floats2bfloat162_rn(gate_act(g0, act) * u0, gate_act(g1, act) * u1);
            ow[k] = *reinterpret_cast<const uint32_t*>(&o);
        }
        out[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

SIB_EXPORT int sib_gated_mul(const void* gate_up, void* out, int dtype, int rows, int inter,
                             int group, int act, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && inter > 0, "gelu_mul: rows=%d inter=%d", rows, inter);
    SIB_REQUIRE(act == ACT_GELU_TANH || act == ACT_SILU, "gelu_mul: unknown activation %d", act);
    SIB_REQUIRE(group >= 0 && (group == 0 || inter % group == 0),
                "gelu_mul: %d columns do not come in groups of %d", inter, group);
    const size_t total = (size_t)rows * inter;
    if (dtype == SIB_BF16 && group == 8 && ((uintptr_t)gate_up % 16) == 0 &&
        ((uintptr_t)out % 16) == 0) {
        const size_t groups = total / 8;
        const size_t want = (groups + 255) / 256;
        const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
        gelu_mul_group8_bf16_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
            (const uint4*)gate_up, (uint4*)out, groups, act);
        return sib_check_launch("gelu_mul");
    }
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    SIB_DISPATCH_DTYPE(dtype, (gelu_mul_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>(
                                  (const T*)gate_up, (T*)out, inter, group, total, act)));
    return sib_check_launch("gelu_mul");
}

SIB_EXPORT int sib_gelu_mul(const void* gate_up, void* out, int dtype, int rows, int inter,
                            int group, void* stream) {
    return sib_gated_mul(gate_up, out, dtype, rows, inter, group, ACT_GELU_TANH, stream);
}

// out = x in another element type (the 32-bit stream as activations).
template <typename Tin, typename Tout>
__global__ void cast_rows_kernel(const Tin* __restrict__ x, Tout* __restrict__ out, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x)
        out[idx] = from_f32<Tout>(to_f32(x[idx]));
}

SIB_EXPORT int sib_cast_rows(const void* x, int in_dtype, void* out, int out_dtype, long long total,
                             void* stream) {
    if (total == 0) return 0;
    SIB_REQUIRE(total > 0, "cast_rows: %lld elements", total);
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
#define GO(TIN, TOUT) \
    sib_launch_chained(cast_rows_kernel<TIN, TOUT>, dim3(blocks), dim3(256), 0, s, (const TIN*)x, \
                       (TOUT*)out, (size_t)total)
    if (in_dtype == SIB_F32 && out_dtype == SIB_F32) GO(float, float);
    else if (in_dtype == SIB_F32 && out_dtype == SIB_BF16) GO(float, __nv_bfloat16);
    else if (in_dtype == SIB_BF16 && out_dtype == SIB_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else if (in_dtype == SIB_BF16 && out_dtype == SIB_F32) GO(__nv_bfloat16, float);
    else SIB_REQUIRE(false, "cast_rows: unknown element types %d -> %d", in_dtype, out_dtype);
#undef GO
    return sib_check_launch("cast_rows");
}

// x = cap * tanh(x / cap), in place, 32-bit.
__global__ void softcap_kernel(float* x, size_t total, float cap) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x)
        x[idx] = cap * tanhf(x[idx] / cap);
}

SIB_EXPORT int sib_softcap(float* x, long long total, float cap, void* stream) {
    if (total == 0 || cap <= 0.f) return 0;
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    softcap_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, (size_t)total, cap);
    return sib_check_launch("softcap");
}

// ---------------------------------------------------------------------------
// Embedding with a hashed bigram table beside the token table:
//     out[r, :] = scale * table[tok_r, :] + bigram[(prev_r * mul_prev + tok_r * mul_cur) mod buckets, :]
// and bigram[buckets, :] (the table's last row) for a sequence's first token.  prev_r is
// the token of the row before in the same sequence; for the first row of a step that
// continues a sequence it is what the slot's state holds (last_token[slot]), which a second
// small kernel brings up to the step's end afterwards.  Rows of a sequence without a slot
// (fillers of a recorded step) store nothing.
// Plain counterpart: tests/plain_vavupel.py bigram_embedding().
// ---------------------------------------------------------------------------
template <typename T>
__global__ void bigram_embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                    const T* __restrict__ bigram, const int* __restrict__ row_pos,
                                    const int* __restrict__ row_seq, const int* __restrict__ seq_slot,
                                    const int* __restrict__ seq_row0, const int* __restrict__ last_token,
                                    float* __restrict__ out, int hidden, float scale, int buckets,
                                    long long mul_prev, long long mul_cur) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int tok = tokens[r];
    long long pick = buckets;
    if (row_pos[r] > 0) {
        const int b = row_seq[r];
        const int slot = seq_slot[b];
        const long long prev = r > seq_row0[b] ? tokens[r - 1] : (slot >= 0 ? last_token[slot] : 0);
        pick = (prev * mul_prev + (long long)tok * mul_cur) % buckets;
        if (pick < 0) pick += buckets;
    }
    const T* src = table + (size_t)tok * hidden;
    const T* two = bigram + (size_t)pick * hidden;
    float* dst = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        dst[i] = to_f32(src[i]) * scale + to_f32(two[i]);
}

__global__ void last_token_kernel(const int* __restrict__ tokens, const int* __restrict__ seq_slot,
                                  const int* __restrict__ seq_start, const int* __restrict__ seq_end,
                                  const int* __restrict__ seq_row0, int* __restrict__ last_token,
                                  int n_seqs) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_seqs) return;
    const int slot = seq_slot[b];
    const int n = seq_end[b] - seq_start[b];
    if (slot >= 0 && n > 0) last_token[slot] = tokens[seq_row0[b] + n - 1];
}

SIB_EXPORT int sib_bigram_embed(const int* tokens, const void* table, const void* bigram,
                                int table_dtype, const int* row_pos, const int* row_seq,
                                const int* seq_slot, const int* seq_start, const int* seq_end,
                                const int* seq_row0, int* last_token, float* out, int rows,
                                int n_seqs, int hidden, float scale, int buckets, long long mul_prev,
                                long long mul_cur, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && n_seqs > 0 && hidden > 0 && buckets > 0,
                "bigram_embed: rows=%d sequences=%d hidden=%d buckets=%d", rows, n_seqs, hidden, buckets);
    SIB_REQUIRE(row_pos && row_seq && seq_slot && seq_start && seq_end && seq_row0 && last_token,
                "bigram_embed: the step's tables and the slots' last tokens are needed");
    cudaStream_t s = (cudaStream_t)stream;
    SIB_DISPATCH_DTYPE(table_dtype,
                       sib_launch_chained(bigram_embed_kernel<T>, dim3(rows), dim3(256), 0, s, tokens,
                                          (const T*)table, (const T*)bigram, row_pos, row_seq, seq_slot,
                                          seq_row0, (const int*)last_token, out, hidden, scale, buckets,
                                          mul_prev, mul_cur));
    int rc = sib_check_launch("bigram_embed");
    if (rc) return rc;
    sib_launch_chained(last_token_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, s, tokens, seq_slot,
                       seq_start, seq_end, seq_row0, last_token, n_seqs);
    return sib_check_launch("last_token");
}

// out = act(x), one value per value: the activation of a feed-forward without a gate.
// act 2: the square of max(x, 0); act 3: tanh(x).
enum { ACT_RELU_SQUARED = 2, ACT_TANH = 3 };
template <typename T>
__global__ void activate_kernel(const T* __restrict__ x, T* __restrict__ out, size_t total, int act) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const float v = to_f32(x[idx]);
        float y;
        if (act == ACT_RELU_SQUARED) { const float p = fmaxf(v, 0.f); y = p * p; }
        else if (act == ACT_TANH) y = tanhf(v);
        else y = gate_act(v, act);
        out[idx] = from_f32<T>(y);
    }
}

SIB_EXPORT int sib_activate(const void* x, void* out, int dtype, long long total, int act, void* stream) {
    if (total == 0) return 0;
    SIB_REQUIRE(total > 0 && act >= 0 && act <= ACT_TANH, "activate: %lld values, activation %d", total, act);
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(activate_kernel<T>, dim3(blocks), dim3(256), 0,
                                                 (cudaStream_t)stream, (const T*)x, (T*)out, (size_t)total, act));
    return sib_check_launch("activate");
}

// out[r, :] = [a[r, :] | b[r, :]] in out's element type: two 32-bit streams side by side
// as the input of one product.
template <typename T>
__global__ void pair_rows_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                 T* __restrict__ out, int hidden, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / (2 * (size_t)hidden);
        const int c = (int)(idx - r * 2 * (size_t)hidden);
        out[idx] = from_f32<T>(c < hidden ? a[r * hidden + c] : b[r * hidden + c - hidden]);
    }
}

SIB_EXPORT int sib_pair_rows(const float* a, const float* b, void* out, int out_dtype, int rows,
                             int hidden, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && hidden > 0 && a && b && out, "pair_rows: rows=%d hidden=%d", rows, hidden);
    const size_t total = (size_t)rows * hidden * 2;
    const size_t want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    SIB_DISPATCH_DTYPE(out_dtype, sib_launch_chained(pair_rows_kernel<T>, dim3(blocks), dim3(256), 0,
                                                     (cudaStream_t)stream, a, b, (T*)out, hidden, total));
    return sib_check_launch("pair_rows");
}

// ---------------------------------------------------------------------------
// gelu_gate_rows: y[r, j] = gelu_tanh(t[r, j]) * e[r, col0 + j]: a gate made from the stream
// times a slice of a 32-bit row that was gathered for the row's token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gelu_gate_rows_kernel(const T* __restrict__ t, const float* __restrict__ e,
                                      long long e_stride, int col0, T* __restrict__ y, int width,
                                      size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / width;
        const int j = (int)(i - r * width);
        const float z = to_f32(t[i]);
        const float g = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        y[i] = from_f32<T>(g * e[r * e_stride + col0 + j]);
    }
}

SIB_EXPORT int sib_gelu_gate_rows(const void* t, const float* e, long long e_stride, int col0, void* y,
                                  int dtype, int rows, int width, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && width > 0 && col0 >= 0 && e_stride >= col0 + width,
                "gelu_gate_rows: rows=%d width=%d from column %d of %lld", rows, width, col0, e_stride);
    const size_t total = (size_t)rows * width;
    const size_t want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(gelu_gate_rows_kernel<T>, dim3(blocks), dim3(256), 0,
                                                 (cudaStream_t)stream, (const T*)t, e, e_stride, col0,
                                                 (T*)y, width, total));
    return sib_check_launch("gelu_gate_rows");
}
