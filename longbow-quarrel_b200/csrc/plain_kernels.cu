// Plain kernels for every operation of the decoder, in 32-bit and in bfloat16 storage.
//
// These are the kernels of the true 32-bit path (every product and sum in IEEE
// float, FFMA on the CUDA cores, no tensor-core mode of reduced precision), and the
// twins beside which each tuned bfloat16 kernel is checked.  Every reduction runs in
// an order that depends only on the row's own sizes, never on what else is in the
// batch, so a position's result does not change with the way the work is cut.
//
// Counterparts in the reference (23skdu/longbow-quarrel), by formula:
//   embedding     internal/device/kernels.metal:465   embedding_f16
//   rmsnorm       internal/device/kernels.metal:905   rmsnorm_f32_to_f16_v4
//   linear        internal/device/kernels.metal:105   linear_f16 (y = x W^T, F32 accumulate)
//   rope          internal/device/kernels.metal:430   rope_f16 (half-split pairs)
//   store K/V     internal/device/kernels.metal:1221  store_kv_f16
//   attention     internal/device/kernels.metal:657   att_fused_f16
//   swiglu        internal/device/cpu_ref.go:133      CPUSwiGLU (no clamp)
#include "common.cuh"
#include <math_constants.h>

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                 float* __restrict__ out, int D, int V) {
    pdl_launch_dependents();
    pdl_wait();
    int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 || tok >= V) tok = 0;  // range is checked on the host before launch
    const TW* row = table + (size_t)tok * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) out[(size_t)t * D + i] = to_f32(row[i]);
}

LQ_EXPORT int lq_embedding(const void* table, int table_dtype, const int* tokens, float* out,
                           int T, int D, int V, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (table_dtype == LQ_F32)
        return launch_pdl(embedding_kernel<float>, dim3(T), dim3(256), 0, stream, (const float*)table, tokens, out, D, V);
    else if (table_dtype == LQ_BF16)
        return launch_pdl(embedding_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16*)table, tokens, out, D, V);
    else
        return LQ_BAD_DTYPE;
    return lq_launch_status();
}

// Embedding of a token plus a row of a second table chosen by the pair (token before it, token):
//   out[t] = table[tok] + pairs[(prev * mul_prev + tok * mul_cur) mod buckets],   pairs[buckets] at a sequence's first token.
// The token before a step's first row is the sequence's state (last[slot], written by last_tokens_kernel after the
// step's rows have been read); sums in float32.
template <typename TW>
__global__ void embedding_pairs_kernel(const TW* __restrict__ table, const TW* __restrict__ pairs, const int* __restrict__ tokens,
                                       const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                       const int* __restrict__ slots, const int* __restrict__ cu_rows,
                                       const int* __restrict__ last, float* __restrict__ out, int D, int V, int buckets,
                                       long long mul_prev, long long mul_cur) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, b = tok_seq[t];
    int tok = tokens[t];
    if (tok < 0 || tok >= V) tok = 0;  // range is checked on the host before launch
    long long at = buckets;
    if (tok_pos[t] > 0) {
        int prev = t > cu_rows[b] ? tokens[t - 1] : last[slots[b]];
        if (prev < 0 || prev >= V) prev = 0;
        at = (prev * mul_prev + tok * mul_cur) % buckets;
        if (at < 0) at += buckets;
    }
    const TW* row = table + (size_t)tok * D;
    const TW* pr = pairs + (size_t)at * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) out[(size_t)t * D + i] = to_f32(row[i]) + to_f32(pr[i]);
}

__global__ void last_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ cu_rows, const int* __restrict__ slots,
                                   int* __restrict__ last, int B) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) last[slots[b]] = tokens[cu_rows[b + 1] - 1];
}

LQ_EXPORT int lq_embedding_pairs(const void* table, const void* pairs, int table_dtype, const int* tokens, const int* tok_pos,
                                 const int* tok_seq, const int* slots, const int* cu_rows, int* last, float* out, int T, int B,
                                 int D, int V, int buckets, long long mul_prev, long long mul_cur, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (buckets < 1) return LQ_BAD_SIZE;
    int rc;
    if (table_dtype == LQ_F32)
        rc = launch_pdl(embedding_pairs_kernel<float>, dim3(T), dim3(256), 0, stream, (const float*)table, (const float*)pairs, tokens,
                        tok_pos, tok_seq, slots, cu_rows, (const int*)last, out, D, V, buckets, mul_prev, mul_cur);
    else if (table_dtype == LQ_BF16)
        rc = launch_pdl(embedding_pairs_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16*)table,
                        (const __nv_bfloat16*)pairs, tokens, tok_pos, tok_seq, slots, cu_rows, (const int*)last, out, D, V, buckets,
                        mul_prev, mul_cur);
    else
        return LQ_BAD_DTYPE;
    if (rc != LQ_OK) return rc;
    return launch_pdl(last_tokens_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, tokens, cu_rows, slots, last, B);
}

// ------------------------------------------------------------------ short causal convolution over time, per channel
//   out[t] = h[t] + sum_j w[:, j] * h[t - taps + 1 + j]      (j = 0 .. taps - 1; rows before the sequence's start are zero)
// The taps - 1 rows ahead of a step's first row are the sequence's state [slot][taps - 1][D] (float32, oldest first,
// zero when the sequence starts); conv_state_kernel moves it on once the step's rows have been read.  Sums in float32.
template <typename T>
__global__ void __launch_bounds__(256) causal_conv_kernel(const T* __restrict__ h, T* __restrict__ out, const float* __restrict__ w,
                                                          const float* __restrict__ state, const int* __restrict__ tok_seq,
                                                          const int* __restrict__ slots, const int* __restrict__ cu_rows, int D,
                                                          int taps, int add_input) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, b = tok_seq[t], first = cu_rows[b], i = t - first, keep = taps - 1;
    const float* st = state + (size_t)slots[b] * keep * D;
    for (int d = blockIdx.y * 256 + threadIdx.x; d < D; d += gridDim.y * 256) {
        const float own = to_f32(h[(size_t)t * D + d]);
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int k = i - keep + j;        // the step's row that tap j reads; below 0: the state's row keep + k
            const float v = j == keep ? own : (k >= 0 ? to_f32(h[(size_t)(first + k) * D + d]) : st[(size_t)(keep + k) * D + d]);
            acc = fmaf(w[(size_t)d * taps + j], v, acc);
        }
        out[(size_t)t * D + d] = from_f32<T>(add_input ? own + acc : acc);
    }
}

// The same sums for rows whose channels come in whole 16-byte pieces: a thread makes 16 / sizeof(T) neighbouring channels,
// every tap's piece one load, the taps added in the same order as above.  wt: the weight by taps, [taps, D], so that a
// thread's weights of one tap are neighbours too.
template <typename T>
__global__ void __launch_bounds__(256) causal_conv_vec_kernel(const T* __restrict__ h, T* __restrict__ out, const float* __restrict__ wt,
                                                              const float* __restrict__ state, const int* __restrict__ tok_seq,
                                                              const int* __restrict__ slots, const int* __restrict__ cu_rows, int D,
                                                              int taps, int add_input) {
    constexpr int V = 16 / sizeof(T);
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, b = tok_seq[t], first = cu_rows[b], i = t - first, keep = taps - 1;
    const int d = (blockIdx.y * 256 + threadIdx.x) * V;
    if (d >= D) return;
    const float* st = state + (size_t)slots[b] * keep * D;
    auto piece = [&](const T* p, float (&v)[V]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int c = 0; c < V; ++c) v[c] = to_f32(e[c]);
    };
    float own[V], acc[V];
    piece(h + (size_t)t * D + d, own);
#pragma unroll
    for (int c = 0; c < V; ++c) acc[c] = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int k = i - keep + j;
        float v[V];
        if (j == keep) {
#pragma unroll
            for (int c = 0; c < V; ++c) v[c] = own[c];
        } else if (k >= 0) {
            piece(h + (size_t)(first + k) * D + d, v);
        } else {
            const float4* sp = reinterpret_cast<const float4*>(st + (size_t)(keep + k) * D + d);
#pragma unroll
            for (int c = 0; c < V / 4; ++c) {
                const float4 f = sp[c];
                v[4 * c] = f.x; v[4 * c + 1] = f.y; v[4 * c + 2] = f.z; v[4 * c + 3] = f.w;
            }
        }
        const float4* wp = reinterpret_cast<const float4*>(wt + (size_t)j * D + d);
#pragma unroll
        for (int c = 0; c < V / 4; ++c) {
            const float4 f = wp[c];
            acc[4 * c] = fmaf(f.x, v[4 * c], acc[4 * c]);
            acc[4 * c + 1] = fmaf(f.y, v[4 * c + 1], acc[4 * c + 1]);
            acc[4 * c + 2] = fmaf(f.z, v[4 * c + 2], acc[4 * c + 2]);
            acc[4 * c + 3] = fmaf(f.w, v[4 * c + 3], acc[4 * c + 3]);
        }
    }
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int c = 0; c < V; ++c) e[c] = from_f32<T>(add_input ? own[c] + acc[c] : acc[c]);
    *reinterpret_cast<uint4*>(out + (size_t)t * D + d) = raw;
}

template <typename T>
__global__ void __launch_bounds__(256) conv_state_kernel(const T* __restrict__ h, float* __restrict__ state,
                                                         const int* __restrict__ slots, const int* __restrict__ cu_rows, int D,
                                                         int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, first = cu_rows[b], n = cu_rows[b + 1] - first, keep = taps - 1;
    float* st = state + (size_t)slots[b] * keep * D;
    for (int d = blockIdx.y * 256 + threadIdx.x; d < D; d += gridDim.y * 256)
        for (int k = 0; k < keep; ++k) {       // rising k: a row that moves down is read before it is overwritten
            const int i = n - keep + k;
            st[(size_t)k * D + d] = i >= 0 ? to_f32(h[(size_t)(first + i) * D + d]) : st[(size_t)(k + n) * D + d];
        }
}

// wt (or null): the same weight laid out [taps, D]; with it, rows whose channels come in whole 16-byte pieces take the
// kernel that makes 16 bytes of channels a thread.
LQ_EXPORT int lq_causal_conv_by_taps(const void* h, void* out, int dtype, const float* w, const float* wt, float* state,
                                     const int* tok_seq, const int* slots, const int* cu_rows, int T, int B, int D, int taps,
                                     int add_input, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (taps < 1 || (taps > 1 && !state)) return LQ_BAD_SIZE;
    const int ny = (D + 1023) / 1024;
    int rc;
    typedef __nv_bfloat16 bf;
    const bool pieces = wt != nullptr && (((uintptr_t)h | (uintptr_t)out | (uintptr_t)state | (uintptr_t)wt) & 15) == 0;
    if (dtype == LQ_F32 && pieces && D % 4 == 0)
        rc = launch_pdl(causal_conv_vec_kernel<float>, dim3(T, (D / 4 + 255) / 256), dim3(256), 0, stream, (const float*)h, (float*)out,
                        wt, (const float*)state, tok_seq, slots, cu_rows, D, taps, add_input);
    else if (dtype == LQ_BF16 && pieces && D % 8 == 0)
        rc = launch_pdl(causal_conv_vec_kernel<bf>, dim3(T, (D / 8 + 255) / 256), dim3(256), 0, stream, (const bf*)h, (bf*)out, wt,
                        (const float*)state, tok_seq, slots, cu_rows, D, taps, add_input);
    else if (dtype == LQ_F32)
        rc = launch_pdl(causal_conv_kernel<float>, dim3(T, ny), dim3(256), 0, stream, (const float*)h, (float*)out, w, (const float*)state,
                        tok_seq, slots, cu_rows, D, taps, add_input);
    else if (dtype == LQ_BF16)
        rc = launch_pdl(causal_conv_kernel<bf>, dim3(T, ny), dim3(256), 0, stream, (const bf*)h, (bf*)out, w, (const float*)state, tok_seq,
                        slots, cu_rows, D, taps, add_input);
    else
        return LQ_BAD_DTYPE;
    if (rc != LQ_OK || taps == 1) return rc;
    if (dtype == LQ_F32)
        return launch_pdl(conv_state_kernel<float>, dim3(B, ny), dim3(256), 0, stream, (const float*)h, state, slots, cu_rows, D, taps);
    return launch_pdl(conv_state_kernel<bf>, dim3(B, ny), dim3(256), 0, stream, (const bf*)h, state, slots, cu_rows, D, taps);
}

LQ_EXPORT int lq_causal_conv(const void* h, void* out, int dtype, const float* w, float* state, const int* tok_seq, const int* slots,
                             const int* cu_rows, int T, int B, int D, int taps, int add_input, cudaStream_t stream) {
    return lq_causal_conv_by_taps(h, out, dtype, w, nullptr, state, tok_seq, slots, cu_rows, T, B, D, taps, add_input, stream);
}

// ------------------------------------------------------------------ x += m * y (a branch that joins the stream with a multiplier)
__global__ void add_scaled_kernel(float* __restrict__ x, const float* __restrict__ y, float m, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = fmaf(m, y[i], x[i]);
}

__global__ void add_scaled4_kernel(float4* __restrict__ x, const float4* __restrict__ y, float m, size_t total4) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    float4 a = x[i];
    const float4 b = y[i];
    a.x = fmaf(m, b.x, a.x); a.y = fmaf(m, b.y, a.y); a.z = fmaf(m, b.z, a.z); a.w = fmaf(m, b.w, a.w);
    x[i] = a;
}

LQ_EXPORT int lq_add_scaled(float* x, const float* y, float m, long long total, cudaStream_t stream) {
    if (total <= 0) return LQ_OK;
    if (total % 4 == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0)
        return launch_pdl(add_scaled4_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream, (float4*)x, (const float4*)y, m,
                          (size_t)(total / 4));
    return launch_pdl(add_scaled_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, y, m, (size_t)total);
}

// ------------------------------------------------------------------ rmsnorm
// x is the 32-bit residual stream.  rows (optional) picks the rows to normalise.
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                               const int* __restrict__ rows, TO* __restrict__ out, int D, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float partial[32];
    __shared__ float scale_s;
    int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = xr[i];
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += partial[w];
        scale_s = 1.0f / sqrtf(t / (float)D + eps);
    }
    __syncthreads();
    float scale = scale_s;
    for (int i = threadIdx.x; i < D; i += blockDim.x)
        out[(size_t)r * D + i] = from_f32<TO>(xr[i] * scale * gain[i]);
}

// Rows whose length is a multiple of 4 and at most 256 * 4 * RMS_VEC: each thread keeps its
// part of the row in registers (one read of x), float4 loads, packed stores.  The sum of squares
// runs in an order fixed by the row length alone.
constexpr int RMS_VEC = 8;   // float4 pieces per thread

template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ gain, const int* __restrict__ rows,
                   TO* __restrict__ out, int D, float eps) {
    __shared__ float partial[8];
    __shared__ float scale_s;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, n4 = D >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * D);
    float4 v[RMS_VEC];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        int c = threadIdx.x + i * 256;
        v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        s = fmaf(v[i].x, v[i].x, s); s = fmaf(v[i].y, v[i].y, s);
        s = fmaf(v[i].z, v[i].z, s); s = fmaf(v[i].w, v[i].w, s);
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += partial[w];
        scale_s = 1.0f / sqrtf(t / (float)D + eps);
    }
    __syncthreads();
    const float scale = scale_s;
    const float4* g4 = reinterpret_cast<const float4*>(gain);
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        int c = threadIdx.x + i * 256;
        if (c >= n4) break;
        float4 g = g4[c];
        float o0 = v[i].x * scale * g.x, o1 = v[i].y * scale * g.y, o2 = v[i].z * scale * g.z, o3 = v[i].w * scale * g.w;
        if (sizeof(TO) == 4) {
            reinterpret_cast<float4*>(out + (size_t)r * D)[c] = make_float4(o0, o1, o2, o3);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
            uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            reinterpret_cast<uint2*>(out + (size_t)r * D)[c] = packed;
        }
    }
}

LQ_EXPORT int lq_rmsnorm(const float* x, const float* gain, const int* rows, void* out, int out_dtype,
                         int n_rows, int D, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return LQ_OK;
    if (out_dtype != LQ_F32 && out_dtype != LQ_BF16) return LQ_BAD_DTYPE;
    const bool vec = D % 4 == 0 && D <= 256 * 4 * RMS_VEC && (((uintptr_t)x | (uintptr_t)gain | (uintptr_t)out) & 15) == 0;
    if (out_dtype == LQ_F32)
        return vec ? launch_pdl(rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, gain, rows, (float*)out, D, eps)
                   : launch_pdl(rmsnorm_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, gain, rows, (float*)out, D, eps);
    return vec ? launch_pdl(rmsnorm_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, x, gain, rows, (__nv_bfloat16*)out, D, eps)
               : launch_pdl(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, x, gain, rows, (__nv_bfloat16*)out, D, eps);
}

// ------------------------------------------------------------------ layer norm
// out = (x - mean) / sqrt(var + eps) * gain + bias over rows of the 32-bit stream, var the mean of the squared
// deviations from the mean (two passes: the mean first, then the deviations), all in float32.  Optionally the
// rows first take up to two branches, x += m1 * y1 + m2 * y2 (in place; a mixer of two sides joining the stream),
// so that the addition and the norm that reads the stream next are one pass.  rows (optional) picks rows (then
// nothing is added).  A block per row; sums run in an order that depends on D alone.
template <typename TO>
__global__ void __launch_bounds__(256)
layernorm_kernel(float* __restrict__ x, const float* __restrict__ y1, float m1, const float* __restrict__ y2, float m2,
                 const float* __restrict__ gain, const float* __restrict__ bias, const int* __restrict__ rows,
                 TO* __restrict__ out, int D, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float partial[8];
    __shared__ float stat;
    const int r = blockIdx.x, tid = threadIdx.x;
    const size_t at = (size_t)(rows ? rows[r] : r) * D;
    float* xr = x + at;
    float s = 0.f;
    for (int i = tid; i < D; i += 256) {
        float v = xr[i];
        if (y1) {
            v = fmaf(m1, y1[at + i], v);
            if (y2) v = fmaf(m2, y2[at + i], v);
            xr[i] = v;
        }
        s += v;
    }
    s = warp_sum(s);
    if ((tid & 31) == 0) partial[tid >> 5] = s;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += partial[w];
        stat = t / (float)D;
    }
    __syncthreads();
    const float mean = stat;
    float q = 0.f;
    for (int i = tid; i < D; i += 256) {
        const float d = xr[i] - mean;
        q = fmaf(d, d, q);
    }
    q = warp_sum(q);
    __syncthreads();
    if ((tid & 31) == 0) partial[tid >> 5] = q;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += partial[w];
        stat = 1.0f / sqrtf(t / (float)D + eps);
    }
    __syncthreads();
    const float inv = stat;
    for (int i = tid; i < D; i += 256)
        out[(size_t)r * D + i] = from_f32<TO>((xr[i] - mean) * inv * gain[i] + (bias ? bias[i] : 0.f));
}

// Rows whose length is a multiple of 4 and at most 256 * 4 * RMS_VEC: each thread keeps its part of the row in registers
// (one read of the stream and of the branches), float4 loads, packed stores; the same two passes over the registers.
template <typename TO>
__global__ void __launch_bounds__(256)
layernorm_vec_kernel(float* __restrict__ x, const float* __restrict__ y1, float m1, const float* __restrict__ y2, float m2,
                     const float* __restrict__ gain, const float* __restrict__ bias, const int* __restrict__ rows,
                     TO* __restrict__ out, int D, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float partial[8];
    __shared__ float stat;
    const int r = blockIdx.x, tid = threadIdx.x, n4 = D >> 2;
    const size_t at = (size_t)(rows ? rows[r] : r) * D;
    float4* xr = reinterpret_cast<float4*>(x + at);
    float4 v[RMS_VEC];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        const int c = tid + i * 256;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < n4) {
            v[i] = xr[c];
            if (y1) {
                const float4 a = reinterpret_cast<const float4*>(y1 + at)[c];
                v[i].x = fmaf(m1, a.x, v[i].x); v[i].y = fmaf(m1, a.y, v[i].y); v[i].z = fmaf(m1, a.z, v[i].z); v[i].w = fmaf(m1, a.w, v[i].w);
                if (y2) {
                    const float4 b = reinterpret_cast<const float4*>(y2 + at)[c];
                    v[i].x = fmaf(m2, b.x, v[i].x); v[i].y = fmaf(m2, b.y, v[i].y); v[i].z = fmaf(m2, b.z, v[i].z); v[i].w = fmaf(m2, b.w, v[i].w);
                }
                xr[c] = v[i];
            }
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    }
    s = warp_sum(s);
    if ((tid & 31) == 0) partial[tid >> 5] = s;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += partial[w];
        stat = t / (float)D;
    }
    __syncthreads();
    const float mean = stat;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        if (tid + i * 256 < n4) {
            v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
            q = fmaf(v[i].x, v[i].x, q); q = fmaf(v[i].y, v[i].y, q); q = fmaf(v[i].z, v[i].z, q); q = fmaf(v[i].w, v[i].w, q);
        }
    }
    q = warp_sum(q);
    __syncthreads();
    if ((tid & 31) == 0) partial[tid >> 5] = q;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += partial[w];
        stat = 1.0f / sqrtf(t / (float)D + eps);
    }
    __syncthreads();
    const float inv = stat;
    const float4* g4 = reinterpret_cast<const float4*>(gain);
    const float4* b4 = reinterpret_cast<const float4*>(bias);
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        const int c = tid + i * 256;
        if (c >= n4) break;
        const float4 g = g4[c], b = bias ? b4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        const float o0 = fmaf(v[i].x * inv, g.x, b.x), o1 = fmaf(v[i].y * inv, g.y, b.y);
        const float o2 = fmaf(v[i].z * inv, g.z, b.z), o3 = fmaf(v[i].w * inv, g.w, b.w);
        if (sizeof(TO) == 4) {
            reinterpret_cast<float4*>(out + (size_t)r * D)[c] = make_float4(o0, o1, o2, o3);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
            reinterpret_cast<uint2*>(out + (size_t)r * D)[c] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
    }
}

LQ_EXPORT int lq_layernorm(float* x, const float* y1, float m1, const float* y2, float m2, const float* gain, const float* bias,
                           const int* rows, void* out, int out_dtype, int n_rows, int D, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return LQ_OK;
    if ((rows && y1) || (y2 && !y1)) return LQ_BAD_SIZE;
    const bool vec = D % 4 == 0 && D <= 256 * 4 * RMS_VEC &&
        (((uintptr_t)x | (uintptr_t)y1 | (uintptr_t)y2 | (uintptr_t)gain | (uintptr_t)bias | (uintptr_t)out) & 15) == 0;
    if (vec && out_dtype == LQ_F32)
        return launch_pdl(layernorm_vec_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, y1, m1, y2, m2, gain, bias, rows,
                          (float*)out, D, eps);
    if (vec && out_dtype == LQ_BF16)
        return launch_pdl(layernorm_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, x, y1, m1, y2, m2, gain, bias, rows,
                          (__nv_bfloat16*)out, D, eps);
    if (out_dtype == LQ_F32)
        return launch_pdl(layernorm_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, y1, m1, y2, m2, gain, bias, rows,
                          (float*)out, D, eps);
    if (out_dtype == LQ_BF16)
        return launch_pdl(layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, x, y1, m1, y2, m2, gain, bias, rows,
                          (__nv_bfloat16*)out, D, eps);
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ two streams side by side, as a product's input
// out[t] = [a[t], b[t]] in the activation dtype from two float32 [T, D] (the stream and the embedding's rows ahead of
// the product that mixes them at the start of a pass over repeated layers).
template <typename TO>
__global__ void side_by_side_kernel(const float* __restrict__ a, const float* __restrict__ b, TO* __restrict__ out, int D,
                                    size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / (2 * D);
    const int c = (int)(i % (2 * D));
    out[i] = from_f32<TO>(c < D ? a[t * D + c] : b[t * D + c - D]);
}

// Four columns a thread (D a multiple of 4, 16-byte aligned tensors).
template <typename TO>
__global__ void side_by_side_vec_kernel(const float4* __restrict__ a, const float4* __restrict__ b, TO* __restrict__ out, int D4,
                                        size_t total4) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const size_t t = i / (2 * D4);
    const int c = (int)(i % (2 * D4));
    const float4 v = c < D4 ? a[t * D4 + c] : b[t * D4 + c - D4];
    if (sizeof(TO) == 4) {
        reinterpret_cast<float4*>(out)[i] = v;
    } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        reinterpret_cast<uint2*>(out)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
}

LQ_EXPORT int lq_side_by_side(const float* a, const float* b, void* out, int out_dtype, int T, int D, cudaStream_t stream) {
    const size_t total = (size_t)T * 2 * D;
    if (total == 0) return LQ_OK;
    if (D % 4 == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0 && (out_dtype == LQ_F32 || out_dtype == LQ_BF16)) {
        const unsigned blocks4 = (unsigned)((total / 4 + 255) / 256);
        if (out_dtype == LQ_F32)
            return launch_pdl(side_by_side_vec_kernel<float>, dim3(blocks4), dim3(256), 0, stream, (const float4*)a, (const float4*)b,
                              (float*)out, D / 4, total / 4);
        return launch_pdl(side_by_side_vec_kernel<__nv_bfloat16>, dim3(blocks4), dim3(256), 0, stream, (const float4*)a, (const float4*)b,
                          (__nv_bfloat16*)out, D / 4, total / 4);
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == LQ_F32)
        return launch_pdl(side_by_side_kernel<float>, dim3(blocks), dim3(256), 0, stream, a, b, (float*)out, D, total);
    if (out_dtype == LQ_BF16)
        return launch_pdl(side_by_side_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, a, b, (__nv_bfloat16*)out, D, total);
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ a branch joins the stream with a multiplier, and the next norm
// x += m * y for rows of a branch's output y [T, D] (float32), then h = x / rms(x) * gain in the activation dtype: what
// add_scaled and rmsnorm do one after the other, with one pass over the stream.  Sums run in rmsnorm's order.
template <typename TO>
__global__ void __launch_bounds__(256)
add_scaled_norm_kernel(float* __restrict__ x, const float* __restrict__ y, float m, const float* __restrict__ gain,
                       TO* __restrict__ out, int D, float eps) {
    __shared__ float partial[8];
    __shared__ float scale_s;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * D;
    const float* yr = y + (size_t)r * D;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += 256) {
        const float v = fmaf(m, yr[i], xr[i]);
        xr[i] = v;
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += partial[w];
        scale_s = 1.0f / sqrtf(t / (float)D + eps);
    }
    __syncthreads();
    const float scale = scale_s;
    for (int i = threadIdx.x; i < D; i += 256) out[(size_t)r * D + i] = from_f32<TO>(xr[i] * scale * gain[i]);
}

template <typename TO>
__global__ void __launch_bounds__(256)
add_scaled_norm_vec_kernel(float* __restrict__ x, const float* __restrict__ y, float m, const float* __restrict__ gain,
                           TO* __restrict__ out, int D, float eps) {
    __shared__ float partial[8];
    __shared__ float scale_s;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, n4 = D >> 2;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)r * D);
    const float4* yr = reinterpret_cast<const float4*>(y + (size_t)r * D);
    float4 v[RMS_VEC];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        int c = threadIdx.x + i * 256;
        if (c < n4) {
            const float4 a = xr[c], b = yr[c];
            v[i] = make_float4(fmaf(m, b.x, a.x), fmaf(m, b.y, a.y), fmaf(m, b.z, a.z), fmaf(m, b.w, a.w));
            xr[c] = v[i];
        } else {
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        s = fmaf(v[i].x, v[i].x, s); s = fmaf(v[i].y, v[i].y, s);
        s = fmaf(v[i].z, v[i].z, s); s = fmaf(v[i].w, v[i].w, s);
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += partial[w];
        scale_s = 1.0f / sqrtf(t / (float)D + eps);
    }
    __syncthreads();
    const float scale = scale_s;
    const float4* g4 = reinterpret_cast<const float4*>(gain);
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        int c = threadIdx.x + i * 256;
        if (c >= n4) break;
        float4 g = g4[c];
        float o0 = v[i].x * scale * g.x, o1 = v[i].y * scale * g.y, o2 = v[i].z * scale * g.z, o3 = v[i].w * scale * g.w;
        if (sizeof(TO) == 4) {
            reinterpret_cast<float4*>(out + (size_t)r * D)[c] = make_float4(o0, o1, o2, o3);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
            uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            reinterpret_cast<uint2*>(out + (size_t)r * D)[c] = packed;
        }
    }
}

LQ_EXPORT int lq_add_scaled_norm(float* x, const float* y, float m, const float* gain, void* out, int out_dtype, int n_rows, int D,
                                 float eps, cudaStream_t stream) {
    if (n_rows <= 0) return LQ_OK;
    if (out_dtype != LQ_F32 && out_dtype != LQ_BF16) return LQ_BAD_DTYPE;
    const bool vec = D % 4 == 0 && D <= 256 * 4 * RMS_VEC && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)gain | (uintptr_t)out) & 15) == 0;
    typedef __nv_bfloat16 bf;
    if (out_dtype == LQ_F32)
        return vec ? launch_pdl(add_scaled_norm_vec_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, y, m, gain, (float*)out, D, eps)
                   : launch_pdl(add_scaled_norm_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, y, m, gain, (float*)out, D, eps);
    return vec ? launch_pdl(add_scaled_norm_vec_kernel<bf>, dim3(n_rows), dim3(256), 0, stream, x, y, m, gain, (bf*)out, D, eps)
               : launch_pdl(add_scaled_norm_kernel<bf>, dim3(n_rows), dim3(256), 0, stream, x, y, m, gain, (bf*)out, D, eps);
}

// ------------------------------------------------------------------ norm of a branch, added to the stream
// x += y / rms(y) * gain for rows of a branch's output y [T, D] (float32): the stream takes the branch after
// the branch's own norm.  With next_gain, the rows of the norm that reads the stream next are made on the way:
// h = x / rms(x) * next_gain, in the activation dtype.  Sums run in an order fixed by D alone.
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_add_kernel(const float* __restrict__ y, const float* __restrict__ gain, float* __restrict__ x,
                   const float* __restrict__ next_gain, TO* __restrict__ h, int D, float eps, float next_eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float partial[8];
    __shared__ float scale_s;
    const int r = blockIdx.x;
    const float* yr = y + (size_t)r * D;
    float* xr = x + (size_t)r * D;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += 256) s = fmaf(yr[i], yr[i], s);
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += partial[w];
        scale_s = 1.0f / sqrtf(t / (float)D + eps);
    }
    __syncthreads();
    const float scale = scale_s;
    s = 0.f;
    for (int i = threadIdx.x; i < D; i += 256) {
        const float v = xr[i] + yr[i] * scale * gain[i];
        xr[i] = v;
        s = fmaf(v, v, s);
    }
    if (!next_gain) return;
    s = warp_sum(s);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += partial[w];
        scale_s = 1.0f / sqrtf(t / (float)D + next_eps);
    }
    __syncthreads();
    const float scale2 = scale_s;
    for (int i = threadIdx.x; i < D; i += 256) h[(size_t)r * D + i] = from_f32<TO>(xr[i] * scale2 * next_gain[i]);
}

LQ_EXPORT int lq_rmsnorm_add(const float* y, const float* gain, float* x, const float* next_gain, void* h, int h_dtype,
                             int n_rows, int D, float eps, float next_eps, cudaStream_t stream) {
    if (n_rows <= 0) return LQ_OK;
    if (h_dtype == LQ_F32)
        return launch_pdl(rmsnorm_add_kernel<float>, dim3(n_rows), dim3(256), 0, stream, y, gain, x, next_gain, (float*)h, D, eps, next_eps);
    if (h_dtype == LQ_BF16)
        return launch_pdl(rmsnorm_add_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, y, gain, x, next_gain,
                          (__nv_bfloat16*)h, D, eps, next_eps);
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ linear (FFMA)
// C[M,N] = A[M,K] . W[N,K]^T (+ residual[M,N]).  Each output is one chain of fused
// multiply-adds over k = 0..K-1 in rising order, whatever M is.
constexpr int GT = 64;   // tile of C
constexpr int GK = 16;   // k step

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C,
                  const float* __restrict__ residual, int M, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float As[GK][GT + 1];
    __shared__ float Ws[GK][GT + 1];
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += GK) {
        for (int i = threadIdx.x; i < GT * GK; i += 256) {
            int r = i / GK, c = i % GK;
            int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * K + gk]) : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (residual) v += residual[(size_t)gm * N + gn];
            C[(size_t)gm * N + gn] = from_f32<TC>(v);
        }
    }
}

template <typename TA, typename TW>
static int gemm_plain_c(const void* A, const void* W, void* C, int c_dtype, const float* residual,
                        int M, int N, int K, cudaStream_t stream) {
    dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
    if (c_dtype == LQ_F32)
        return launch_pdl(gemm_plain_kernel<TA, TW, float>, grid, dim3(256), 0, stream, (const TA*)A, (const TW*)W, (float*)C, residual, M, N, K);
    else if (c_dtype == LQ_BF16)
        return launch_pdl(gemm_plain_kernel<TA, TW, __nv_bfloat16>, grid, dim3(256), 0, stream, (const TA*)A, (const TW*)W, (__nv_bfloat16*)C, residual, M, N, K);
    else
        return LQ_BAD_DTYPE;
    return lq_launch_status();
}

LQ_EXPORT int lq_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                            const float* residual, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LQ_OK;
    if (a_dtype == LQ_F32 && w_dtype == LQ_F32) return gemm_plain_c<float, float>(A, W, C, c_dtype, residual, M, N, K, stream);
    if (a_dtype == LQ_F32 && w_dtype == LQ_BF16) return gemm_plain_c<float, __nv_bfloat16>(A, W, C, c_dtype, residual, M, N, K, stream);
    if (a_dtype == LQ_BF16 && w_dtype == LQ_F32) return gemm_plain_c<__nv_bfloat16, float>(A, W, C, c_dtype, residual, M, N, K, stream);
    if (a_dtype == LQ_BF16 && w_dtype == LQ_BF16) return gemm_plain_c<__nv_bfloat16, __nv_bfloat16>(A, W, C, c_dtype, residual, M, N, K, stream);
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ rope + cache write
// qkv [T, (H + 2 Hkv) hd] holds q, k, v of each token side by side.  q and k are
// rotated in place (pairs i, i + hd/2; angle = position * f_i from the cos/sin
// tables, which may be null for no rotation); k and v are then stored into the
// token's cache page.  A page holds [Hkv][page_size][hd] of one layer.
// With has_kv == 0 the rows hold q only (a layer that reads another layer's cache).
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_seq, const int* __restrict__ slots,
                                     const int* __restrict__ page_table, int pt_stride,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     int H, int Hkv, int hd, int page_size, int has_kv) {
    pdl_launch_dependents();
    pdl_wait();
    int t = blockIdx.x;
    int pos = tok_pos[t];
    int half = hd >> 1;
    int row_w = (H + (has_kv ? 2 * Hkv : 0)) * hd;
    T* row = qkv + (size_t)t * row_w;
    const float* cs = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)pos * half : nullptr;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (has_kv) {
        int slot = slots[tok_seq[t]];
        int page = page_table[(size_t)slot * pt_stride + pos / page_size];
        size_t base = ((size_t)page * Hkv * page_size + (pos % page_size)) * hd;
        kdst = k_pages + base;
        vdst = v_pages + base;
    }
    int n_rot = (H + (has_kv ? Hkv : 0)) * half;
    for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
        int head = i / half, j = i % half;
        T* p = row + (size_t)head * hd;
        float x0 = to_f32(p[j]), x1 = to_f32(p[j + half]);
        float y0 = x0, y1 = x1;
        if (cs) {
            float c = cs[j], s = sn[j];
            y0 = x0 * c - x1 * s;
            y1 = x0 * s + x1 * c;
        }
        T o0 = from_f32<T>(y0), o1 = from_f32<T>(y1);
        p[j] = o0;
        p[j + half] = o1;
        if (head >= H) {
            T* d = kdst + (size_t)(head - H) * page_size * hd;
            d[j] = o0;
            d[j + half] = o1;
        }
    }
    if (has_kv) {
        const T* vsrc = row + (size_t)(H + Hkv) * hd;
        for (int i = threadIdx.x; i < Hkv * hd; i += blockDim.x) {
            int head = i / hd, j = i % hd;
            vdst[(size_t)head * page_size * hd + j] = vsrc[i];
        }
    }
}

// The same work with 16-byte accesses, for half head sizes that are a multiple of the vector
// length (8 bfloat16 or 4 float32): a thread rotates VEC pairs of one head at a time.
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_write_vec_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                         const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ slots,
                         const int* __restrict__ page_table, int pt_stride, T* __restrict__ k_pages,
                         T* __restrict__ v_pages, int H, int Hkv, int hd, int page_size, int has_kv) {
    constexpr int VEC = Vec16<T>::N;
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int half = hd >> 1, pieces = half / VEC;
    const int row_w = (H + (has_kv ? 2 * Hkv : 0)) * hd;
    T* row = qkv + (size_t)t * row_w;
    const float* cs = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)pos * half : nullptr;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (has_kv) {
        int slot = slots[tok_seq[t]];
        int page = page_table[(size_t)slot * pt_stride + pos / page_size];
        size_t base = ((size_t)page * Hkv * page_size + (pos % page_size)) * hd;
        kdst = k_pages + base;
        vdst = v_pages + base;
    }
    const int n_rot = (H + (has_kv ? Hkv : 0)) * pieces;
    for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
        const int head = i / pieces, j = (i % pieces) * VEC;
        T* p = row + (size_t)head * hd;
        uint4 a = *reinterpret_cast<const uint4*>(p + j), b = *reinterpret_cast<const uint4*>(p + j + half);
        const T* x0 = reinterpret_cast<const T*>(&a);
        const T* x1 = reinterpret_cast<const T*>(&b);
        uint4 oa, ob;
        T* y0 = reinterpret_cast<T*>(&oa);
        T* y1 = reinterpret_cast<T*>(&ob);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            float u = to_f32(x0[e]), w = to_f32(x1[e]);
            float c = cs ? cs[j + e] : 1.f, s = sn ? sn[j + e] : 0.f;
            y0[e] = from_f32<T>(u * c - w * s);
            y1[e] = from_f32<T>(u * s + w * c);
        }
        *reinterpret_cast<uint4*>(p + j) = oa;
        *reinterpret_cast<uint4*>(p + j + half) = ob;
        if (head >= H) {
            T* d = kdst + (size_t)(head - H) * page_size * hd;
            *reinterpret_cast<uint4*>(d + j) = oa;
            *reinterpret_cast<uint4*>(d + j + half) = ob;
        }
    }
    if (has_kv) {
        const T* vsrc = row + (size_t)(H + Hkv) * hd;
        const int per_head = hd / VEC;
        for (int i = threadIdx.x; i < Hkv * per_head; i += blockDim.x) {
            int head = i / per_head, j = (i % per_head) * VEC;
            *reinterpret_cast<uint4*>(vdst + (size_t)head * page_size * hd + j) =
                *reinterpret_cast<const uint4*>(vsrc + (size_t)head * hd + j);
        }
    }
}

template <typename T>
static int rope_launch(void* qkv, const float* cos_t, const float* sin_t, const int* tok_pos, const int* tok_seq,
                       const int* slots, const int* page_table, int pt_stride, void* k_pages, void* v_pages, int Tn,
                       int H, int Hkv, int hd, int page_size, int has_kv, cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    const bool vec = (hd / 2) % VEC == 0 && (((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0;
    auto kernel = vec ? rope_kv_write_vec_kernel<T> : rope_kv_write_kernel<T>;
    return launch_pdl(kernel, dim3(Tn), dim3(256), 0, stream, (T*)qkv, cos_t, sin_t, tok_pos, tok_seq, slots, page_table,
                      pt_stride, (T*)k_pages, (T*)v_pages, H, Hkv, hd, page_size, has_kv);
}

LQ_EXPORT int lq_rope_kv_write(void* qkv, int dtype, const float* cos_t, const float* sin_t,
                               const int* tok_pos, const int* tok_seq, const int* slots,
                               const int* page_table, int pt_stride, void* k_pages, void* v_pages,
                               int T, int H, int Hkv, int hd, int page_size, int has_kv,
                               cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (hd % 2) return LQ_BAD_SIZE;
    if (dtype == LQ_F32)
        return rope_launch<float>(qkv, cos_t, sin_t, tok_pos, tok_seq, slots, page_table, pt_stride, k_pages, v_pages,
                                  T, H, Hkv, hd, page_size, has_kv, stream);
    if (dtype == LQ_BF16)
        return rope_launch<__nv_bfloat16>(qkv, cos_t, sin_t, tok_pos, tok_seq, slots, page_table, pt_stride, k_pages,
                                          v_pages, T, H, Hkv, hd, page_size, has_kv, stream);
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ biases, partial rotation, cache write
// Rows of `buf` [T, stride] hold n_rot heads of size hd side by side from column 0 (queries, then keys where
// the layer has keys of its own), and from column v_off Hkv value heads of size vd.  Each of the n_rot heads
// gets its bias (bias[column], optional) and has its first `rot` dimensions rotated in pairs (i, i + rot/2)
// by the angle of its row's position (cos/sin tables [positions, rot/2]); the rest of the head passes.
// Heads below k_first (the queries) go to qout [T, qout_stride], which may be buf itself; with a cache, heads
// k_first.. go into the row's page of k_pages [page][Hkv][page_size][hd], and the values (with their bias)
// into v_pages [..][vd] (with v_unit: each value head first divided by its root mean square, sqrt(mean(v^2) + v_eps)).
// The rows may be float32 while queries and cache are bfloat16: a product's 32-bit sums
// then meet their biases and angles before anything is rounded.
// unit_norm (after the bias, ahead of the rotation; 32-bit, eps inside the root): 1, each of the n_rot heads is divided by
// its own root mean square; 2, the queries (heads below k_first) are divided by the root mean square of all of them
// together and the keys likewise, and each dimension is multiplied by norm_w[column] (the queries' weights, then the keys').
// q_temp_every > 0: the queries are then multiplied by 1 + q_temp_coef * ln(floor((p + 1) / q_temp_every) + 1) at position p.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
rope_partial_kernel(const TI* buf, int stride, TO* qout, int qout_stride, const float* __restrict__ bias,
                    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                    const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ slots,
                    const int* __restrict__ page_table, int pt_stride, TO* __restrict__ k_pages, TO* __restrict__ v_pages,
                    int n_rot, int k_first, int Hkv, int hd, int vd, int v_off, int page_size, int v_unit, float v_eps,
                    int unit_norm, const float* __restrict__ norm_w, float norm_eps, float q_temp_coef, int q_temp_every) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float head_mul[];             // [n_rot] what each head is multiplied by (unit norm, query temperature)
    const int t = blockIdx.x, pos = tok_pos[t], half = rot >> 1;
    const TI* row = buf + (size_t)t * stride;
    const bool scaled = unit_norm || q_temp_every > 0;
    if (scaled) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (unit_norm) {
            // Sums of squares, a warp per head, in an order that depends on hd alone.
            for (int head = warp; head < n_rot; head += 8) {
                const TI* p = row + (size_t)head * hd;
                float ss = 0.f;
                for (int j = lane; j < hd; j += 32) {
                    const float v = to_f32(p[j]) + (bias ? bias[(size_t)head * hd + j] : 0.f);
                    ss = fmaf(v, v, ss);
                }
                ss = warp_sum(ss);
                if (lane == 0) head_mul[head] = ss;
            }
            __syncthreads();
            if (unit_norm == 2) {
                // One norm over all queries and one over all keys: the heads' sums added in the order of the heads.
                float sq = 0.f, sk = 0.f;
                for (int head = 0; head < k_first; ++head) sq += head_mul[head];
                for (int head = k_first; head < n_rot; ++head) sk += head_mul[head];
                __syncthreads();
                const float iq = 1.f / sqrtf(sq / (float)(k_first * hd) + norm_eps);
                const float ik = n_rot > k_first ? 1.f / sqrtf(sk / (float)((n_rot - k_first) * hd) + norm_eps) : 0.f;
                for (int head = threadIdx.x; head < n_rot; head += 256) head_mul[head] = head < k_first ? iq : ik;
            } else {
                for (int head = threadIdx.x; head < n_rot; head += 256)
                    head_mul[head] = 1.f / sqrtf(head_mul[head] / (float)hd + norm_eps);
            }
        } else {
            for (int head = threadIdx.x; head < n_rot; head += 256) head_mul[head] = 1.f;
        }
        __syncthreads();
        if (q_temp_every > 0) {
            const float qt = 1.f + q_temp_coef * logf((float)((pos + 1) / q_temp_every) + 1.f);
            for (int head = threadIdx.x; head < k_first; head += 256) head_mul[head] *= qt;
            __syncthreads();
        }
    }
    TO* qrow = qout + (size_t)t * qout_stride;
    const float* cs = rot ? cos_t + (size_t)pos * half : nullptr;
    const float* sn = rot ? sin_t + (size_t)pos * half : nullptr;
    size_t at = 0;
    if (k_pages) {
        const int page = page_table[(size_t)slots[tok_seq[t]] * pt_stride + pos / page_size];
        at = (size_t)page * Hkv * page_size + (pos % page_size);
    }
    const int per_head = hd - half;                 // a rotated pair is one piece of work, every other dimension one
    for (int i = threadIdx.x; i < n_rot * per_head; i += 256) {
        const int head = i / per_head, j = i % per_head;
        const TI* p = row + (size_t)head * hd;
        const float* b = bias ? bias + (size_t)head * hd : nullptr;
        TO* qd = head < k_first ? qrow + (size_t)head * hd : nullptr;
        TO* kd = (k_pages && head >= k_first) ? k_pages + (at + (size_t)(head - k_first) * page_size) * hd : nullptr;
        const float mul = scaled ? head_mul[head] : 1.f;
        const float* nw = (unit_norm == 2 && norm_w) ? norm_w + (size_t)head * hd : nullptr;
        if (j < half) {
            float u = to_f32(p[j]) + (b ? b[j] : 0.f), w = to_f32(p[j + half]) + (b ? b[j + half] : 0.f);
            if (scaled) {
                u *= mul;
                w *= mul;
                if (nw) { u *= nw[j]; w *= nw[j + half]; }
            }
            const float c = cs[j], s = sn[j];
            const TO o0 = from_f32<TO>(u * c - w * s), o1 = from_f32<TO>(w * c + u * s);
            if (qd) { qd[j] = o0; qd[j + half] = o1; }
            if (kd) { kd[j] = o0; kd[j + half] = o1; }
        } else {
            const int d = j + half;
            float v = to_f32(p[d]) + (b ? b[d] : 0.f);
            if (scaled) v = nw ? v * mul * nw[d] : v * mul;
            const TO o = from_f32<TO>(v);
            if (qd) qd[d] = o;
            if (kd) kd[d] = o;
        }
    }
    if (v_pages && v_unit) {
        // Each value head divided by its root mean square (32-bit; eps inside the root): a warp per head.
        const TI* vsrc = row + v_off;
        const float* b = bias ? bias + v_off : nullptr;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int head = warp; head < Hkv; head += 8) {
            float ss = 0.f;
            for (int j = lane; j < vd; j += 32) {
                const float v = to_f32(vsrc[head * vd + j]) + (b ? b[head * vd + j] : 0.f);
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
            const float inv = 1.f / sqrtf(ss / (float)vd + v_eps);
            for (int j = lane; j < vd; j += 32) {
                const float v = to_f32(vsrc[head * vd + j]) + (b ? b[head * vd + j] : 0.f);
                v_pages[(at + (size_t)head * page_size) * vd + j] = from_f32<TO>(v * inv);
            }
        }
    } else if (v_pages) {
        const TI* vsrc = row + v_off;
        const float* b = bias ? bias + v_off : nullptr;
        for (int i = threadIdx.x; i < Hkv * vd; i += 256) {
            const int head = i / vd, j = i % vd;
            v_pages[(at + (size_t)head * page_size) * vd + j] = from_f32<TO>(to_f32(vsrc[i]) + (b ? b[i] : 0.f));
        }
    }
}

LQ_EXPORT int lq_rope_partial(const void* buf, int in_dtype, int stride, void* qout, int out_dtype, int qout_stride,
                              const float* bias, const float* cos_t, const float* sin_t, int rot, const int* tok_pos,
                              const int* tok_seq, const int* slots, const int* page_table, int pt_stride, void* k_pages,
                              void* v_pages, int T, int n_rot, int k_first, int Hkv, int hd, int vd, int v_off,
                              int page_size, int v_unit, float v_eps, int unit_norm, const float* norm_w, float norm_eps,
                              float q_temp_coef, int q_temp_every, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (rot % 2 || rot > hd || (rot && (!cos_t || !sin_t)) || (!k_pages) != (!v_pages)) return LQ_BAD_SIZE;
    if (unit_norm < 0 || unit_norm > 2 || n_rot > 8192) return LQ_BAD_SIZE;
    const size_t smem = (size_t)n_rot * sizeof(float);
    typedef __nv_bfloat16 bf;
#define LQ_GO(TI, TO) return launch_pdl(rope_partial_kernel<TI, TO>, dim3(T), dim3(256), smem, stream, (const TI*)buf, stride, \
        (TO*)qout, qout_stride, bias, cos_t, sin_t, rot, tok_pos, tok_seq, slots, page_table, pt_stride, (TO*)k_pages, \
        (TO*)v_pages, n_rot, k_first, Hkv, hd, vd, v_off, page_size, v_unit, v_eps, unit_norm, norm_w, norm_eps, q_temp_coef, \
        q_temp_every)
    if (in_dtype == LQ_F32 && out_dtype == LQ_F32) LQ_GO(float, float);
    if (in_dtype == LQ_BF16 && out_dtype == LQ_BF16) LQ_GO(bf, bf);
    if (in_dtype == LQ_F32 && out_dtype == LQ_BF16) LQ_GO(float, bf);
#undef LQ_GO
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ activations, soft cap
// out = act(x), element by element, in float32: 0 relu(x)^2, 1 gelu (tanh form), 2 silu, 3 relu, 4 gelu (erf form).
__device__ __forceinline__ float activation(float v, int act) {
    switch (act) {
        case 0: { float r = fmaxf(v, 0.f); return r * r; }
        case 1: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case 2: return v / (1.f + expf(-v));
        case 4: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
        default: return fmaxf(v, 0.f);
    }
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, T* __restrict__ out, size_t total, int act) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_f32<T>(activation(to_f32(x[i]), act));
}

// Sixteen bytes per thread, where the sizes and addresses allow it.
template <typename T>
__global__ void activation_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, size_t pieces, int act) {
    constexpr int VEC = 16 / sizeof(T);
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pieces) return;
    uint4 v = x[i];
    T* e = reinterpret_cast<T*>(&v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) e[j] = from_f32<T>(activation(to_f32(e[j]), act));
    out[i] = v;
}

LQ_EXPORT int lq_activation(const void* x, void* out, int dtype, long long total, int act, cudaStream_t stream) {
    if (total <= 0) return LQ_OK;
    if (act < 0 || act > 4) return LQ_BAD_SIZE;
    const int vec = dtype == LQ_F32 ? 4 : 8;
    if ((dtype == LQ_F32 || dtype == LQ_BF16) && total % vec == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
        const size_t pieces = (size_t)total / vec;
        const unsigned vblocks = (unsigned)((pieces + 255) / 256);
        if (dtype == LQ_F32)
            return launch_pdl(activation_vec_kernel<float>, dim3(vblocks), dim3(256), 0, stream, (const uint4*)x, (uint4*)out, pieces, act);
        return launch_pdl(activation_vec_kernel<__nv_bfloat16>, dim3(vblocks), dim3(256), 0, stream, (const uint4*)x, (uint4*)out, pieces, act);
    }
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == LQ_F32)
        return launch_pdl(activation_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, (float*)out, (size_t)total, act);
    if (dtype == LQ_BF16)
        return launch_pdl(activation_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x,
                          (__nv_bfloat16*)out, (size_t)total, act);
    return LQ_BAD_DTYPE;
}

// out[t, f] = act(gu[t, f] + b[f]) * (gu[t, F + f] + b[F + f]): a gated feed-forward's two halves (gate columns, then up
// columns) with their biases (float32 [2F], or none), the activation in float32.
template <typename TI, typename TO>
__global__ void gated_act_kernel(const TI* __restrict__ gu, const float* __restrict__ bias, TO* __restrict__ out, size_t total,
                                 int F, int act) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / F;
    const int f = i % F;
    float g = to_f32(gu[t * 2 * F + f]), u = to_f32(gu[t * 2 * F + F + f]);
    if (bias) { g += bias[f]; u += bias[F + f]; }
    out[i] = from_f32<TO>(activation(g, act) * u);
}

// bfloat16 in and out, F a multiple of 8: eight outputs a thread from two 16-byte loads, the same arithmetic.
__global__ void gated_act_vec_kernel(const uint4* __restrict__ gu, const float* __restrict__ bias, uint4* __restrict__ out,
                                     size_t total8, int F8, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const size_t t = i / F8;
    const int f8 = (int)(i % F8);
    uint4 g = gu[t * 2 * F8 + f8], u = gu[t * 2 * F8 + F8 + f8], o;
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float2 gv = __bfloat1622float2(gp[j]), uv = __bfloat1622float2(up[j]);
        if (bias) {
            const int f = f8 * 8 + 2 * j;
            gv.x += bias[f]; gv.y += bias[f + 1];
            uv.x += bias[8 * F8 + f]; uv.y += bias[8 * F8 + f + 1];
        }
        op[j] = __floats2bfloat162_rn(activation(gv.x, act) * uv.x, activation(gv.y, act) * uv.y);
    }
    out[i] = o;
}

LQ_EXPORT int lq_gated_act(const void* gu, int in_dtype, const float* bias, void* out, int out_dtype, int T, int F, int act,
                           cudaStream_t stream) {
    const size_t total = (size_t)T * F;
    if (total == 0) return LQ_OK;
    if (act < 0 || act > 4) return LQ_BAD_SIZE;
    if (in_dtype == LQ_BF16 && out_dtype == LQ_BF16 && F % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0)
        return launch_pdl(gated_act_vec_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, stream, (const uint4*)gu, bias,
                          (uint4*)out, total / 8, F / 8, act);
    const unsigned blocks = (unsigned)((total + 255) / 256);
    typedef __nv_bfloat16 bf;
    if (in_dtype == LQ_F32 && out_dtype == LQ_F32)
        return launch_pdl(gated_act_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, bias, (float*)out, total, F, act);
    if (in_dtype == LQ_F32 && out_dtype == LQ_BF16)
        return launch_pdl(gated_act_kernel<float, bf>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, bias, (bf*)out, total, F, act);
    if (in_dtype == LQ_BF16 && out_dtype == LQ_BF16)
        return launch_pdl(gated_act_kernel<bf, bf>, dim3(blocks), dim3(256), 0, stream, (const bf*)gu, bias, (bf*)out, total, F, act);
    return LQ_BAD_DTYPE;
}

// x[t, d] += bias[d] (float32 rows of the stream; a projection's bias that its residual epilogue does not add).
__global__ void add_bias_kernel(float* __restrict__ x, const float* __restrict__ bias, size_t total, int D) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] += bias[i % D];
}

LQ_EXPORT int lq_add_bias(float* x, const float* bias, int T, int D, cudaStream_t stream) {
    const size_t total = (size_t)T * D;
    if (total == 0) return LQ_OK;
    return launch_pdl(add_bias_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, bias, total, D);
}

// x[r, c] *= sigmoid(gate[r, c / group]) (act 1) or silu(...) (act 2), in place; gate rows may be strided.  group 1: a gate
// for every value; group n: one gate for n neighbouring columns (a head's values behind one number).
template <typename T, typename TG>
__global__ void gate_mul_kernel(T* __restrict__ x, const TG* __restrict__ gate, int gate_stride, int cols, size_t total, int act,
                                int group) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float g = to_f32(gate[(i / cols) * gate_stride + (i % cols) / group]);
    const float sg = 1.f / (1.f + expf(-g));
    x[i] = from_f32<T>(to_f32(x[i]) * (act == 1 ? sg : g * sg));
}

LQ_EXPORT int lq_gate_mul(void* x, const void* gate, int gate_stride, int dtype, int gate_dtype, int rows, int cols, int act,
                          int group, cudaStream_t stream) {
    const size_t total = (size_t)rows * cols;
    if (total == 0) return LQ_OK;
    if ((act != 1 && act != 2) || group < 1 || cols % group) return LQ_BAD_SIZE;
    unsigned blocks = (unsigned)((total + 255) / 256);
    typedef __nv_bfloat16 bf;
    if (dtype == LQ_F32 && gate_dtype == LQ_F32)
        return launch_pdl(gate_mul_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (float*)x, (const float*)gate, gate_stride, cols, total, act, group);
    if (dtype == LQ_BF16 && gate_dtype == LQ_BF16)
        return launch_pdl(gate_mul_kernel<bf, bf>, dim3(blocks), dim3(256), 0, stream, (bf*)x, (const bf*)gate, gate_stride, cols, total, act, group);
    if (dtype == LQ_BF16 && gate_dtype == LQ_F32)
        return launch_pdl(gate_mul_kernel<bf, float>, dim3(blocks), dim3(256), 0, stream, (bf*)x, (const float*)gate, gate_stride, cols, total, act, group);
    return LQ_BAD_DTYPE;
}

// x <- cap * tanh(x / cap) in place (float32 logits).
__global__ void softcap_kernel(float* __restrict__ x, size_t total, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = cap * tanhf(x[i] / cap);
}

LQ_EXPORT int lq_softcap(float* x, long long total, float cap, cudaStream_t stream) {
    if (total <= 0) return LQ_OK;
    return launch_pdl(softcap_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, (size_t)total, cap);
}

// ------------------------------------------------------------------ attention over the cache
// One block per (token, query head).  Keys start..pos of the token's own sequence are
// read from its pages in chunks of ATT_CHUNK; the running maximum, sum and output
// are carried from chunk to chunk, and inside a chunk every sum runs in key order.
// The same kernel serves a prompt's tokens and a decoded token, so both reduce in the
// same order.  cap > 0: score <- cap * tanh(score / cap) after the scale.  keep_first: with a window, the first
// keep_first positions of the sequence stay visible (at their own positions) when the window has moved past them.
constexpr int ATT_CHUNK = 128;

template <typename T, typename TG>
__global__ void __launch_bounds__(ATT_CHUNK)
attention_plain_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_pages,
                       const T* __restrict__ v_pages, const int* __restrict__ page_table, int pt_stride,
                       const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                       const int* __restrict__ slots, T* __restrict__ out, int H, int Hkv, int hd,
                       int page_size, float scale, int window, int vd, const float* __restrict__ sink,
                       const TG* __restrict__ gate, int gate_stride, float cap, int keep_first, int gate_per_head) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    float* qs = sm;              // [hd]
    float* sc = sm + hd;         // [ATT_CHUNK]
    int* pg = (int*)(sc + ATT_CHUNK);  // [ATT_CHUNK] page of each key of the chunk
    int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    int pos = tok_pos[t];
    int slot = slots[tok_seq[t]];
    int kvh = h / (H / Hkv);
    int start = lq_first_key(pos, window);
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int i = tid; i < hd; i += ATT_CHUNK) qs[i] = to_f32(qrow[i]);
    __syncthreads();
    float m = -CUDART_INF_F, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;  // output dims tid and tid + ATT_CHUNK (hd <= 256)
    const int* pt = page_table + (size_t)slot * pt_stride;
    // The keys a row sees: the first `head` positions that its window has left behind (keep_first), then its window.
    const int head = min(keep_first, start), total = head + pos - start + 1;
    for (int vbase = 0; vbase < total; vbase += ATT_CHUNK) {
        int n = min(ATT_CHUNK, total - vbase);
        float s = -CUDART_INF_F;
        if (tid < n) {
            int key = vbase + tid < head ? vbase + tid : start + (vbase + tid - head);
            int page = pt[key / page_size];
            pg[tid] = page;
            const T* kr = k_pages + (((size_t)page * Hkv + kvh) * page_size + key % page_size) * hd;
            float d = 0.f;
            for (int i = 0; i < hd; ++i) d = fmaf(qs[i], to_f32(kr[i]), d);
            s = d * scale;
            if (cap > 0.f) s = cap * tanhf(s / cap);
        }
        sc[tid] = s;
        __syncthreads();
        float cm = m;
        for (int j = 0; j < n; ++j) cm = fmaxf(cm, sc[j]);
        float corr = expf(m - cm);  // m = -inf at the first chunk gives 0
        __syncthreads();
        if (tid < n) sc[tid] = expf(sc[tid] - cm);
        __syncthreads();
        float ls = 0.f;
        for (int j = 0; j < n; ++j) ls += sc[j];
        l = l * corr + ls;
        for (int rep = 0; rep < 2; ++rep) {
            int d = tid + rep * ATT_CHUNK;
            if (d >= vd) break;
            float a = 0.f;
            for (int j = 0; j < n; ++j) {
                int key = vbase + j < head ? vbase + j : start + (vbase + j - head);
                const T* vr = v_pages + (((size_t)pg[j] * Hkv + kvh) * page_size + key % page_size) * vd;
                a = fmaf(sc[j], to_f32(vr[d]), a);
            }
            if (rep == 0) acc0 = acc0 * corr + a; else acc1 = acc1 * corr + a;
        }
        m = cm;
        __syncthreads();
    }
    if (sink) {
        // One more term in the denominator: exp(sink) of the head, with no key and no value.
        float s = sink[h], cm = fmaxf(m, s), corr = expf(m - cm);
        l = l * corr + expf(s - cm);
        acc0 *= corr;
        acc1 *= corr;
    }
    float o0 = acc0 / l, o1 = acc1 / l;
    if (gate) {
        // The output gate: each value times sigmoid of the gate's value at the same place, or (gate_per_head) every
        // value of the head times sigmoid of the head's one number, gate [T, H].
        if (gate_per_head) {
            const float sg = 1.f / (1.f + expf(-to_f32(gate[(size_t)t * gate_stride + h])));
            o0 *= sg;
            o1 *= sg;
        } else {
            const TG* g = gate + (size_t)t * gate_stride + (size_t)h * vd;
            if (tid < vd) o0 *= 1.f / (1.f + expf(-to_f32(g[tid])));
            if (tid + ATT_CHUNK < vd) o1 *= 1.f / (1.f + expf(-to_f32(g[tid + ATT_CHUNK])));
        }
    }
    T* orow = out + ((size_t)t * H + h) * vd;
    if (tid < vd) orow[tid] = from_f32<T>(o0);
    if (tid + ATT_CHUNK < vd) orow[tid + ATT_CHUNK] = from_f32<T>(o1);
}

LQ_EXPORT int lq_attention_plain(const void* q, int q_stride, int dtype, const void* k_pages, const void* v_pages,
                                 const int* page_table, int pt_stride, const int* tok_pos, const int* tok_seq,
                                 const int* slots, void* out, int T, int H, int Hkv, int hd, int page_size,
                                 float scale, int window, int vd, const float* sink, const void* gate, int gate_stride,
                                 int gate_dtype, float cap, int keep_first, int gate_per_head, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (vd <= 0) vd = hd;
    if (vd > 2 * ATT_CHUNK || H % Hkv) return LQ_BAD_SIZE;
    dim3 grid(T, H);
    size_t smem = (hd + 2 * ATT_CHUNK) * sizeof(float);
    if (dtype == LQ_F32)
        return launch_pdl(attention_plain_kernel<float, float>, grid, dim3(ATT_CHUNK), smem, stream, (const float*)q, q_stride, (const float*)k_pages,
            (const float*)v_pages, page_table, pt_stride, tok_pos, tok_seq, slots, (float*)out, H, Hkv, hd, page_size, scale, window,
            vd, sink, (const float*)gate, gate_stride, cap, keep_first, gate_per_head);
    else if (dtype == LQ_BF16 && gate && gate_dtype == LQ_F32)
        return launch_pdl(attention_plain_kernel<__nv_bfloat16, float>, grid, dim3(ATT_CHUNK), smem, stream, (const __nv_bfloat16*)q, q_stride,
            (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, page_table, pt_stride, tok_pos, tok_seq, slots,
            (__nv_bfloat16*)out, H, Hkv, hd, page_size, scale, window, vd, sink, (const float*)gate, gate_stride, cap, keep_first, gate_per_head);
    else if (dtype == LQ_BF16)
        return launch_pdl(attention_plain_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(ATT_CHUNK), smem, stream, (const __nv_bfloat16*)q, q_stride,
            (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, page_table, pt_stride, tok_pos, tok_seq, slots,
            (__nv_bfloat16*)out, H, Hkv, hd, page_size, scale, window, vd, sink, (const __nv_bfloat16*)gate, gate_stride, cap, keep_first, gate_per_head);
    else
        return LQ_BAD_DTYPE;
    return lq_launch_status();
}

// ------------------------------------------------------------------ swiglu
// out = up * gate / (1 + e^-gate) from gu [T, 2F].  block == 0: gate in columns
// [0, F), up in [F, 2F).  block == b > 0: columns alternate b gate, b up, b gate, ...
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t total, int block) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t t = i / F;
    int f = (int)(i % F);
    int gi = block ? (f / block) * 2 * block + f % block : f;
    int ui = block ? gi + block : F + f;
    float g = to_f32(gu[t * 2 * F + gi]);
    float u = to_f32(gu[t * 2 * F + ui]);
    out[i] = from_f32<T>(u * (g / (1.0f + expf(-g))));
}

LQ_EXPORT int lq_swiglu(const void* gu, void* out, int dtype, int T, int F, int block, cudaStream_t stream) {
    size_t total = (size_t)T * F;
    if (total == 0) return LQ_OK;
    if (block < 0 || (block && F % block)) return LQ_BAD_SIZE;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == LQ_F32)
        return launch_pdl(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, F, total, block);
    else if (dtype == LQ_BF16)
        return launch_pdl(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, F, total, block);
    else
        return LQ_BAD_DTYPE;
    return lq_launch_status();
}

// ------------------------------------------------------------------ clearing the unwritten end of a page
// A page that a sequence is given may hold what another sequence left there.  Kernels that load whole
// pages multiply the rows beyond the sequence's length by probability zero, which gives zero only for
// finite values; so the rows of a new page that the step will not write are cleared before the step.
// pages [entry][page][kv head][token][head_dim]; work item = (page, first row to clear).
#define LQ_CLEAR_MAX 120
struct ClearList { int page[LQ_CLEAR_MAX]; int first_row[LQ_CLEAR_MAX]; };

__global__ void clear_page_tails_kernel(uint32_t* __restrict__ k_pages, uint32_t* __restrict__ v_pages, ClearList list,
                                        size_t entry_words, size_t page_words, int Hkv, int page_size, int row_words) {
    const int item = blockIdx.x, entry = blockIdx.y, head = blockIdx.z;
    const int first = list.first_row[item];
    const size_t base = (size_t)entry * entry_words + (size_t)list.page[item] * page_words
                      + ((size_t)head * page_size + first) * row_words;
    const int n = (page_size - first) * row_words;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        k_pages[base + i] = 0u;
        v_pages[base + i] = 0u;
    }
}

LQ_EXPORT int lq_clear_page_tails(void* k_pages, void* v_pages, int dtype, const int* pages, const int* first_rows,
                                  int n_items, int n_entries, int n_pages, int Hkv, int page_size, int hd,
                                  cudaStream_t stream) {
    if (n_items <= 0 || n_entries <= 0) return LQ_OK;
    if (dtype != LQ_F32 && dtype != LQ_BF16) return LQ_BAD_DTYPE;
    const int elt = dtype == LQ_F32 ? 4 : 2;
    if ((hd * elt) % 4) return LQ_BAD_SIZE;
    const int row_words = hd * elt / 4;
    const size_t page_words = (size_t)Hkv * page_size * row_words;
    for (int at = 0; at < n_items; at += LQ_CLEAR_MAX) {
        ClearList list;
        const int n = n_items - at < LQ_CLEAR_MAX ? n_items - at : LQ_CLEAR_MAX;
        for (int i = 0; i < n; ++i) {
            if (pages[at + i] < 0 || pages[at + i] >= n_pages || first_rows[at + i] < 0 || first_rows[at + i] > page_size)
                return LQ_BAD_SIZE;
            list.page[i] = pages[at + i];
            list.first_row[i] = first_rows[at + i];
        }
        int rc = launch_after(clear_page_tails_kernel, dim3(n, n_entries, Hkv), dim3(256), 0, stream, (uint32_t*)k_pages,
                              (uint32_t*)v_pages, list, page_words * (size_t)n_pages, page_words, Hkv, page_size, row_words);
        if (rc != LQ_OK) return rc;
    }
    return LQ_OK;
}
