// A feed-forward that sends each token to a few of many small experts.
//
//   lq_moe_route   router logits -> the chosen experts of every token and their weights
//   lq_moe_up      u[t, j, :] = act(W_up[e(t, j)] h[t])             for the j-th chosen expert of token t
//                  (gated: act(W_gate h) * (W_up h), the expert's gate rows stacked ahead of its up rows)
//   lq_moe_down    y[t, :] = sum_j w(t, j) W_down[e(t, j)] u[t, j, :], in the order of j; optionally
//                  + sigmoid(z_s[t]) * shared[t, :], and the whole added into the float32 stream
//
// Experts numbered n_real and above are identity experts: no matrices, their output is the weight times h[t] itself.
//
// Routing (the form the kernel started with; lq_moe_route's comment lists the others): scores s = sigmoid(z).  The experts form `groups` equal groups of neighbours; a group's score is the
// sum of its two largest scores; only experts of the `keep` best groups can be chosen; of those the `top` with
// the largest scores are (ties go to the lower index).  Weights: the chosen scores over their sum (+ 1e-20),
// times `route_scale`.  Everything here is float32.
//
// Every token streams the matrices of its own experts (a warp per output row, lanes along the contraction), so a
// step of few tokens reads each chosen expert about once; tokens that share an expert meet in L2.
#include "common.cuh"
#include <math_constants.h>

constexpr int MR_WARPS = 4;

// Index of the largest value among vals[0..n) (ties: the lowest index), found by a whole warp.
__device__ __forceinline__ int warp_argmax(const float* vals, int n, int lane) {
    float best = -CUDART_INF_F;
    int at = 0x7fffffff;
    for (int i = lane; i < n; i += 32)
        if (vals[i] > best) { best = vals[i]; at = i; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    return at == 0x7fffffff ? 0 : at;
}

// score_fn 0: s = sigmoid(z); 1: s = softmax(z) over all E.  correction (optional, [E]): the choice is made by s + correction,
// the weights by s alone.  group_rule 0: a group's score is the sum of its two largest choice scores; 1: its largest.
// normalize: the chosen s over their sum (+ 1e-20); either way times route_scale.  Choice scores may be negative: what
// cannot be chosen counts as minus infinity.
__global__ void __launch_bounds__(MR_WARPS * 32) moe_route_kernel(const float* __restrict__ z, int z_stride, int* __restrict__ ids,
                                                                  float* __restrict__ weights, int T, int E, int groups, int keep,
                                                                  int top, float route_scale, int score_fn,
                                                                  const float* __restrict__ correction, int group_rule,
                                                                  int normalize) {
    pdl_launch_dependents();
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = blockIdx.x * MR_WARPS + warp;
    float* score = sm + (size_t)warp * (3 * E + groups);      // [E] the scores
    float* choice = score + E;                                // [E] the scores that the choice is made by
    float* cand = choice + E;                                 // [E] the choice scores still to be chosen from (-inf: not)
    float* gs = cand + E;                                     // [groups]
    pdl_wait();
    if (t >= T) return;
    const int per = E / groups;
    const float* zr = z + (size_t)t * z_stride;
    if (score_fn == 1) {
        float mx = -CUDART_INF_F;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float v = expf(zr[e] - mx); score[e] = v; sum += v; }
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) score[e] = score[e] / sum;
    } else {
        for (int e = lane; e < E; e += 32) score[e] = 1.f / (1.f + expf(-zr[e]));
    }
    for (int e = lane; e < E; e += 32) choice[e] = score[e] + (correction ? correction[e] : 0.f);
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {
        float a = -CUDART_INF_F, b = -CUDART_INF_F;           // the two largest of the group
        for (int i = 0; i < per; ++i) {
            const float v = choice[g * per + i];
            if (v > a) { b = a; a = v; } else if (v > b) b = v;
        }
        gs[g] = a + ((group_rule == 0 && per > 1) ? b : 0.f);
    }
    for (int e = lane; e < E; e += 32) cand[e] = -CUDART_INF_F;
    __syncwarp();
    for (int n = 0; n < keep; ++n) {
        const int g = warp_argmax(gs, groups, lane);
        __syncwarp();
        for (int i = lane; i < per; i += 32) cand[g * per + i] = choice[g * per + i];
        if (lane == 0) gs[g] = -CUDART_INF_F;
        __syncwarp();
    }
    float sum = 0.f;
    for (int n = 0; n < top; ++n) {
        const int e = warp_argmax(cand, E, lane);
        __syncwarp();
        sum += score[e];
        if (lane == 0) { ids[(size_t)t * top + n] = e; cand[e] = -CUDART_INF_F; }
        __syncwarp();
    }
    const float mult = normalize ? route_scale / (sum + 1e-20f) : route_scale;
    for (int n = lane; n < top; n += 32) weights[(size_t)t * top + n] = score[ids[(size_t)t * top + n]] * mult;
}

LQ_EXPORT int lq_moe_route(const float* z, int z_stride, int* ids, float* weights, int T, int E, int groups, int keep, int top,
                           float route_scale, int score_fn, const float* correction, int group_rule, int normalize,
                           cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (E < 1 || groups < 1 || E % groups || keep < 1 || keep > groups || top < 1 || top > keep * (E / groups)) return LQ_BAD_SIZE;
    const size_t smem = (size_t)MR_WARPS * (3 * E + groups) * sizeof(float);
    if (smem > 200 * 1024) return LQ_BAD_SIZE;
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_pdl(moe_route_kernel, dim3((T + MR_WARPS - 1) / MR_WARPS), dim3(MR_WARPS * 32), smem, stream, z, z_stride, ids,
                      weights, T, E, groups, keep, top, route_scale, score_fn, correction, group_rule, normalize);
}

// act: 0 none, 1 gelu (erf), 2 gelu (tanh form), 3 silu, 4 relu
__device__ __forceinline__ float moe_act(float v, int act) {
    switch (act) {
        case 1: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
        case 2: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case 3: return v / (1.f + expf(-v));
        case 4: return fmaxf(v, 0.f);
        default: return v;
    }
}

// sum_k x[k] * w[k] over a row of n numbers, by one warp (x float32 in shared memory).  bfloat16 rows whose length is a
// multiple of 8 are read 16 bytes a lane at a time (rows then start on 16-byte boundaries), two loads in flight.
// (The lane's share of the sum: the caller adds the lanes with warp_sum, once for all that it has to add.)
__device__ __forceinline__ float row_part(const float* __restrict__ x, const float* __restrict__ w, int n, int lane) {
    float s = 0.f;
    for (int k = lane; k < n; k += 32) s = fmaf(x[k], w[k], s);
    return s;
}
__device__ __forceinline__ float dot8(const float* x, uint4 v, float s) {
    const float4 a = *reinterpret_cast<const float4*>(x), b = *reinterpret_cast<const float4*>(x + 4);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
    const float2 w0 = __bfloat1622float2(p[0]), w1 = __bfloat1622float2(p[1]), w2 = __bfloat1622float2(p[2]), w3 = __bfloat1622float2(p[3]);
    s = fmaf(a.x, w0.x, s); s = fmaf(a.y, w0.y, s); s = fmaf(a.z, w1.x, s); s = fmaf(a.w, w1.y, s);
    s = fmaf(b.x, w2.x, s); s = fmaf(b.y, w2.y, s); s = fmaf(b.z, w3.x, s); s = fmaf(b.w, w3.y, s);
    return s;
}
__device__ __forceinline__ float row_part(const float* __restrict__ x, const __nv_bfloat16* __restrict__ w, int n, int lane) {
    float s0 = 0.f, s1 = 0.f;
    if ((n & 7) == 0) {
        const uint4* w4 = reinterpret_cast<const uint4*>(w);
        const int n8 = n >> 3;
        int k = lane;
        for (; k + 32 < n8; k += 64) {
            const uint4 v0 = __ldg(w4 + k), v1 = __ldg(w4 + k + 32);
            s0 = dot8(x + 8 * k, v0, s0);
            s1 = dot8(x + 8 * (k + 32), v1, s1);
        }
        if (k < n8) s0 = dot8(x + 8 * k, __ldg(w4 + k), s0);
    } else {
        for (int k = lane; k < n; k += 32) s0 = fmaf(x[k], __bfloat162float(w[k]), s0);
    }
    return s0 + s1;
}

constexpr int MX_WARPS = 8;
constexpr int MX_PER_WARP = 4;        // output rows a warp makes one after the other

// grid (T * top, ceil(F / (MX_WARPS * MX_PER_WARP))): h[t] in shared memory as float32; a warp per output row.
template <typename T>
__global__ void __launch_bounds__(MX_WARPS * 32) moe_up_kernel(const T* __restrict__ h, const T* __restrict__ w_up,
                                                               const int* __restrict__ ids, T* __restrict__ u, int top, int D,
                                                               int F, int act, int gated, int n_real, int block) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float xs[];   // [D]
    const int pair = blockIdx.x, t = pair / top, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    for (int d = tid; d < D; d += MX_WARPS * 32) xs[d] = to_f32(h[(size_t)t * D + d]);
    const int e = ids[pair];
    if (e >= n_real) return;                       // an identity expert has no matrices: its output is the input itself
    __syncthreads();
    const T* w = w_up + (size_t)e * (gated ? 2 : 1) * F * D;     // gated: F gate rows, then F up rows (block 0) ...
    // ... or `block` gate rows and the `block` up rows that go with them by turns (the layout whose product the
    // tensor-core kernels' gated epilogue reads)
    auto gate_row = [&](int f) { return block ? (size_t)(f / block) * 2 * block + f % block : (size_t)f; };
    const size_t up_after = block ? (size_t)block : (size_t)F;
    // The lanes' shares of all the warp's outputs first (their loads are in flight together), then the sums.
    float part[MX_PER_WARP];
#pragma unroll
    for (int i = 0; i < MX_PER_WARP; ++i) {
        const int f = (blockIdx.y * MX_PER_WARP + i) * MX_WARPS + warp;
        part[i] = f < F ? row_part(xs, w + (gated ? gate_row(f) : (size_t)f) * D, D, lane) : 0.f;
    }
    float part_up[MX_PER_WARP];
#pragma unroll
    for (int i = 0; i < MX_PER_WARP; ++i) {
        const int f = (blockIdx.y * MX_PER_WARP + i) * MX_WARPS + warp;
        part_up[i] = (gated && f < F) ? row_part(xs, w + (gate_row(f) + up_after) * D, D, lane) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < MX_PER_WARP; ++i) {
        const int f = (blockIdx.y * MX_PER_WARP + i) * MX_WARPS + warp;
        const float s = warp_sum(part[i]);
        const float up = gated ? warp_sum(part_up[i]) : 1.f;
        // gated: the activated gate is rounded as a product's output would be before it meets the up value
        if (lane == 0 && f < F) u[(size_t)pair * F + f] = from_f32<T>(gated ? moe_act(s, act) * up : moe_act(s, act));
    }
}

// grid (T, ceil(D / (MX_WARPS * MX_PER_WARP))): the token's `top` rows of u in shared memory; a warp per output.
template <typename T>
__global__ void __launch_bounds__(MX_WARPS * 32) moe_down_kernel(const T* __restrict__ u, const T* __restrict__ w_down,
                                                                 const int* __restrict__ ids, const float* __restrict__ weights,
                                                                 const float* __restrict__ shared, const float* __restrict__ zs,
                                                                 int zs_stride, float* __restrict__ x, int accumulate, int top,
                                                                 int D, int F, const T* __restrict__ h, int n_real,
                                                                 float shared_scale) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float us[];   // [top][F]
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    for (int i = tid; i < top * F; i += MX_WARPS * 32) us[i] = to_f32(u[(size_t)t * top * F + i]);
    __syncthreads();
    const float sg = ((shared && zs) ? 1.f / (1.f + expf(-zs[(size_t)t * zs_stride])) : 1.f) * shared_scale;
    float part[MX_PER_WARP];
#pragma unroll
    for (int i = 0; i < MX_PER_WARP; ++i) {
        const int d = (blockIdx.y * MX_PER_WARP + i) * MX_WARPS + warp;
        part[i] = 0.f;
        if (d < D)
            for (int j = 0; j < top; ++j) {          // the choices in their order, weighted inside each lane's share
                if (ids[(size_t)t * top + j] >= n_real) continue;
                const T* wr = w_down + ((size_t)ids[(size_t)t * top + j] * D + d) * F;
                part[i] = fmaf(weights[(size_t)t * top + j], row_part(us + j * F, wr, F, lane), part[i]);
            }
    }
#pragma unroll
    for (int i = 0; i < MX_PER_WARP; ++i) {
        const int d = (blockIdx.y * MX_PER_WARP + i) * MX_WARPS + warp;
        float y = warp_sum(part[i]);
        if (d >= D) continue;
        if (lane == 0) {
            for (int j = 0; j < top; ++j)            // identity experts: the weight times the input itself
                if (ids[(size_t)t * top + j] >= n_real) y = fmaf(weights[(size_t)t * top + j], to_f32(h[(size_t)t * D + d]), y);
            if (shared) y = fmaf(sg, shared[(size_t)t * D + d], y);
            float* o = x + (size_t)t * D + d;
            *o = accumulate ? *o + y : y;
        }
    }
}

// block (gated only): 0 = an expert's F gate rows, then its F up rows; b > 0 (F a multiple of b) = b gate rows and b up rows by turns.
LQ_EXPORT int lq_moe_up_rows(const void* h, const void* w_up, const int* ids, void* u, int dtype, int T, int top, int D, int F, int act,
                             int gated, int n_real, int block, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (act < 0 || act > 4 || (size_t)D * 4 > 200 * 1024) return LQ_BAD_SIZE;
    if (block < 0 || (block && (!gated || F % block))) return LQ_BAD_SIZE;
    dim3 grid(T * top, (F + MX_WARPS * MX_PER_WARP - 1) / (MX_WARPS * MX_PER_WARP));
    const size_t smem = (size_t)D * sizeof(float);
    typedef __nv_bfloat16 bf;
#define LQ_GO(TT) do { if (smem > 48 * 1024) cudaFuncSetAttribute(moe_up_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return launch_pdl(moe_up_kernel<TT>, grid, dim3(MX_WARPS * 32), smem, stream, (const TT*)h, (const TT*)w_up, ids, (TT*)u, top, D, F, act, gated, n_real, block); } while (0)
    if (dtype == LQ_F32) LQ_GO(float);
    if (dtype == LQ_BF16) LQ_GO(bf);
#undef LQ_GO
    return LQ_BAD_DTYPE;
}

LQ_EXPORT int lq_moe_up(const void* h, const void* w_up, const int* ids, void* u, int dtype, int T, int top, int D, int F, int act,
                        int gated, int n_real, cudaStream_t stream) {
    return lq_moe_up_rows(h, w_up, ids, u, dtype, T, top, D, F, act, gated, n_real, 0, stream);
}

LQ_EXPORT int lq_moe_down(const void* u, const void* w_down, const int* ids, const float* weights, const float* shared,
                          const float* zs, int zs_stride, float* x, int accumulate, int dtype, int T, int top, int D, int F,
                          const void* h, int n_real, float shared_scale, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    const size_t smem = (size_t)top * F * sizeof(float);
    if (smem > 200 * 1024) return LQ_BAD_SIZE;
    dim3 grid(T, (D + MX_WARPS * MX_PER_WARP - 1) / (MX_WARPS * MX_PER_WARP));
    typedef __nv_bfloat16 bf;
#define LQ_GO(TT) do { if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return launch_pdl(moe_down_kernel<TT>, grid, dim3(MX_WARPS * 32), smem, stream, (const TT*)u, (const TT*)w_down, ids, weights, \
                          shared, zs, zs_stride, x, accumulate, top, D, F, (const TT*)h, n_real, shared_scale); } while (0)
    if (dtype == LQ_F32) LQ_GO(float);
    if (dtype == LQ_BF16) LQ_GO(bf);
#undef LQ_GO
    return LQ_BAD_DTYPE;
}
