// Many small matrix products in one launch, on the tensor cores (mma.sync m16n8k16, bfloat16 in, float32 sums):
//
//     out[row(r), g-th column block] = epilogue( A[a_row(r), g-th column block] . W[g]^T )      W[g] [N, K], K contiguous
//
// for groups g = 0 .. G-1.  Two ways of saying which rows belong to a group:
//   uniform   every group has the same M rows 0 .. M-1 (one small matrix per head: a_group_stride / o_group_stride
//             move A and out from head to head inside a row)
//   listed    `rows` lists row numbers group by group, group g owning rows[group_off[g] .. group_off[g+1]) (routed
//             experts: the (token, choice) pairs sorted by expert; A's row is rows[r] / a_div, so that the `top`
//             choices of a token read the token's one input row; out's row is rows[r]).  lq_group_rows makes the list
//             on the device from the chosen experts, so that nothing of a step waits for the host.
// A block makes a 64 x BN tile of one group (BN 256 for wide outputs, else 128): 2 x BN/64 warps of 32 x 64, operands
// through shared memory in steps of 32 along K (cp.async, two stages, rows padded against bank conflicts).  Measured
// on B200 with 64 x 128 tiles: deeper pipelines and longer steps ran slower (fewer blocks fit a multiprocessor); the
// bound is the traffic from L2 into shared memory, which a wider tile lowers per product.
#include "common.cuh"
#include <math_constants.h>

namespace {

#ifndef GG_BK
#define GG_BK 32
#endif
#ifndef GG_STAGES
#define GG_STAGES 2
#endif
constexpr int BM = 64, BK = GG_BK, PAD = 8, LDS = BK + PAD, STAGES = GG_STAGES;
constexpr size_t gg_smem_bytes(int BN) { return (size_t)STAGES * (BM + BN) * LDS * 2; }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// act: 0 none, 1 gelu (erf), 2 gelu (tanh form), 3 silu, 4 relu
__device__ __forceinline__ float gg_act(float v, int act) {
    switch (act) {
        case 1: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
        case 2: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case 3: return v / (1.f + expf(-v));
        case 4: return fmaxf(v, 0.f);
        default: return v;
    }
}

struct GroupedArgs {
    const __nv_bfloat16* A;
    long long lda, a_group_stride;
    int a_div;
    const __nv_bfloat16* W;
    long long w_group_stride;
    void* out;
    long long ldo, o_group_stride;
    const int* rows;                 // listed: row numbers, group by group (null: uniform)
    const int* group_off;            // listed: [G + 1]
    const int* tile_off;             // listed: [G + 1] prefix of each group's row tiles
    int G, M, N, K, act;
};

template <typename TO, int BN>
__global__ void __launch_bounds__(BN) grouped_gemm_kernel(GroupedArgs a) {
    constexpr int WN = BN / 64, NT = 2 * WN * 32;
    extern __shared__ __align__(16) uint8_t gg_smem[];
    typedef __nv_bfloat16 (*TileA)[BM][LDS];
    typedef __nv_bfloat16 (*TileB)[BN][LDS];
    TileA sa = reinterpret_cast<TileA>(gg_smem);
    TileB sb = reinterpret_cast<TileB>(gg_smem + (size_t)STAGES * BM * LDS * 2);
    __shared__ int s_rows[BM];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t = lane & 3;
    const int wm = warp / WN, wn = warp % WN;
    pdl_launch_dependents();
    pdl_wait();
    // Which group, and which of its row tiles.
    int g, r_first, r_end;
    if (a.rows) {
        const int tile = blockIdx.x;
        if (tile >= a.tile_off[a.G]) return;
        int lo = 0, hi = a.G - 1;
        while (lo < hi) {                        // the last group whose first tile is not beyond this one
            const int mid = (lo + hi + 1) >> 1;
            if (a.tile_off[mid] <= tile) lo = mid; else hi = mid - 1;
        }
        g = lo;
        r_first = a.group_off[g] + (tile - a.tile_off[g]) * BM;
        r_end = a.group_off[g + 1];
    } else {
        const int tiles = (a.M + BM - 1) / BM;
        g = blockIdx.x / tiles;
        r_first = (blockIdx.x % tiles) * BM;
        r_end = a.M;
    }
    const int n_rows = min(BM, r_end - r_first), n0 = blockIdx.y * BN;
    if (tid < BM) s_rows[tid] = tid < n_rows ? (a.rows ? a.rows[r_first + tid] : r_first + tid) : -1;
    __syncthreads();
    const __nv_bfloat16* A = a.A + (long long)g * a.a_group_stride;
    const __nv_bfloat16* W = a.W + (long long)g * a.w_group_stride;
    const int K = a.K, N = a.N;
    auto load = [&](int k0, int stage) {
        for (int i = tid; i < BM * (BK / 8); i += NT) {
            const int r = i / (BK / 8), c = k0 + (i % (BK / 8)) * 8, row = s_rows[r];
            const bool ok = row >= 0 && c < K;
            cp_async16((uint32_t)__cvta_generic_to_shared(&sa[stage][r][c - k0]), ok ? A + (long long)(row / a.a_div) * a.lda + c : A, ok);
        }
        for (int i = tid; i < BN * (BK / 8); i += NT) {
            const int r = i / (BK / 8), c = k0 + (i % (BK / 8)) * 8;
            const bool ok = n0 + r < N && c < K;
            cp_async16((uint32_t)__cvta_generic_to_shared(&sb[stage][r][c - k0]), ok ? W + (long long)(n0 + r) * K + c : W, ok);
        }
    };
    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
    const int steps = (K + BK - 1) / BK;
    for (int p = 0; p < STAGES - 1; ++p) {
        if (p < steps) load(p * BK, p);
        cp_async_commit();
    }
    for (int s = 0; s < steps; ++s) {
        const int stage = s % STAGES;
        cp_async_wait<STAGES - 2>();
        __syncthreads();                          // step s has landed, and everyone is done with the stage that is loaded next
        if (s + STAGES - 1 < steps) load((s + STAGES - 1) * BK, (s + STAGES - 1) % STAGES);
        cp_async_commit();
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            uint32_t af[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = wm * 32 + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = kk * 16 + (lane >> 4) * 8;
                ldsm_x4((uint32_t)__cvta_generic_to_shared(&sa[stage][r][c]), af[i][0], af[i][1], af[i][2], af[i][3]);
            }
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                const int r = wn * 64 + jp * 16 + (lane & 7) + (lane >> 4) * 8, c = kk * 16 + ((lane >> 3) & 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4((uint32_t)__cvta_generic_to_shared(&sb[stage][r][c]), b0, b1, b2, b3);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma_bf16(acc[i][2 * jp], af[i][0], af[i][1], af[i][2], af[i][3], b0, b1);
                    mma_bf16(acc[i][2 * jp + 1], af[i][0], af[i][1], af[i][2], af[i][3], b2, b3);
                }
            }
        }
    }
    TO* out = (TO*)a.out + (long long)g * a.o_group_stride;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = s_rows[wm * 32 + i * 16 + gq + half * 8];
            if (row < 0) continue;
            TO* o = out + (long long)row * a.ldo;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int n = n0 + wn * 64 + j * 8 + 2 * t;
                if (n < N) o[n] = from_f32<TO>(gg_act(acc[i][j][2 * half], a.act));
                if (n + 1 < N) o[n + 1] = from_f32<TO>(gg_act(acc[i][j][2 * half + 1], a.act));
            }
        }
}

// ids [n] (each in [0, G)) -> rows [n]: the indices 0 .. n-1 group by group; group_off [G + 1]; tile_off [G + 1]: the
// prefix of ceil(count / 64).  One block; the order inside a group is whatever the atomics give (no result depends on it).
__global__ void __launch_bounds__(1024) group_rows_kernel(const int* __restrict__ ids, int n, int G, int* __restrict__ rows,
                                                          int* __restrict__ group_off, int* __restrict__ tile_off) {
    pdl_launch_dependents();
    extern __shared__ int sm[];                  // [G] counts, then [G] cursors
    int* count = sm;
    int* cursor = sm + G;
    pdl_wait();
    for (int g = threadIdx.x; g < G; g += blockDim.x) count[g] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&count[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int g = 0; g < G; ++g) {
            group_off[g] = at;
            tile_off[g] = tiles;
            cursor[g] = at;
            at += count[g];
            tiles += (count[g] + BM - 1) / BM;
        }
        group_off[G] = at;
        tile_off[G] = tiles;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) rows[atomicAdd(&cursor[ids[i]], 1)] = i;
}

// The same list with every group's rows padded to whole tiles of `tile` rows, for a product whose row tiles each
// belong to one group: src [cap] = the index that stands at each padded place (-1: padding), dst [n] = the place of
// each index, tile_group [cap / tile] = each tile's group (-1 behind the last).  cap = (ceil(n / tile) + G) * tile holds every case.
// Indices whose group is G or above (groups without rows of their own) take no place: their dst is -1.
__global__ void __launch_bounds__(1024) group_rows_padded_kernel(const int* __restrict__ ids, int n, int G, int tile, int cap,
                                                                 int* __restrict__ src, int* __restrict__ dst,
                                                                 int* __restrict__ tile_group) {
    pdl_launch_dependents();
    extern __shared__ int sm[];
    int* count = sm;
    int* cursor = sm + G;
    pdl_wait();
    for (int g = threadIdx.x; g < G; g += blockDim.x) count[g] = 0;
    for (int i = threadIdx.x; i < cap; i += blockDim.x) src[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        if (ids[i] < G) atomicAdd(&count[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int g = 0; g < G; ++g) {
            cursor[g] = at;
            const int tiles = (count[g] + tile - 1) / tile;
            for (int k = 0; k < tiles; ++k) tile_group[at / tile + k] = g;
            at += tiles * tile;
        }
        for (int k = at / tile; k < cap / tile; ++k) tile_group[k] = -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (ids[i] >= G) {
            dst[i] = -1;
            continue;
        }
        const int p = atomicAdd(&cursor[ids[i]], 1);
        src[p] = i;
        dst[i] = p;
    }
}

// out[p, :] = a[src[p] / div, :] (zeros where src[p] < 0): the rows of a product's input in the padded order.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ a, const int* __restrict__ src, int div,
                                                          uint4* __restrict__ out, int cap, int row16) {
    pdl_launch_dependents();
    pdl_wait();
    const int p = blockIdx.x, s = src[p];
    for (int i = threadIdx.x; i < row16; i += 256)
        out[(size_t)p * row16 + i] = s >= 0 ? a[(size_t)(s / div) * row16 + i] : make_uint4(0, 0, 0, 0);
}

// x[t, :] (+)= sum_j weights[t, j] y[row(t, j), :] (+ shared_scale * sigmoid(zs[t]) * shared[t, :]), the choices added in
// their order.  row(t, j) = place[t * top + j] with `place` (the dst of the padded order), else the pair t * top + j itself.
// With `ids` and `h`, a pair whose id is E or above has no row in y: it adds weights[t, j] * h[t, :] (an expert that passes
// its input on).
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place,
                                                          const float* __restrict__ weights, const float* __restrict__ shared,
                                                          const float* __restrict__ zs, int zs_stride, float* __restrict__ x,
                                                          int accumulate, int top, int D, const int* __restrict__ ids, int E,
                                                          const __nv_bfloat16* __restrict__ h, float shared_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float sg = shared_scale * ((shared && zs) ? 1.f / (1.f + expf(-zs[(size_t)t * zs_stride])) : 1.f);
    for (int d = threadIdx.x; d < D; d += 256) {
        float s = 0.f;
        for (int j = 0; j < top; ++j) {
            const size_t pair = (size_t)t * top + j;
            const float v = (ids && ids[pair] >= E) ? __bfloat162float(h[(size_t)t * D + d])
                                                    : y[(place ? (size_t)place[pair] : pair) * D + d];
            s = fmaf(weights[pair], v, s);
        }
        if (shared) s = fmaf(sg, shared[(size_t)t * D + d], s);
        float* o = x + (size_t)t * D + d;
        *o = accumulate ? *o + s : s;
    }
}

}  // namespace

LQ_EXPORT int lq_group_rows(const int* ids, int n, int G, int* rows, int* group_off, int* tile_off, cudaStream_t stream) {
    if (n <= 0 || G <= 0) return LQ_BAD_SIZE;
    const size_t smem = 2 * (size_t)G * sizeof(int);
    if (smem > 48 * 1024) return LQ_BAD_SIZE;
    return launch_pdl(group_rows_kernel, dim3(1), dim3(1024), smem, stream, ids, n, G, rows, group_off, tile_off);
}

// Row tiles that a listed launch of n rows in G groups can need at most.
LQ_EXPORT int lq_grouped_gemm_tiles(int n, int G) { return (n + BM - 1) / BM + G; }

LQ_EXPORT int lq_grouped_gemm(const void* A, long long lda, long long a_group_stride, int a_div, const void* W,
                              long long w_group_stride, void* out, int out_dtype, long long ldo, long long o_group_stride,
                              const int* rows, const int* group_off, const int* tile_off, int n_listed, int G, int M, int N,
                              int K, int act, cudaStream_t stream) {
    if (G <= 0 || N <= 0) return LQ_OK;
    if (K % 8 || lda % 8 || a_group_stride % 8 || w_group_stride % 8 || a_div < 1 || act < 0 || act > 4) return LQ_BAD_SIZE;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return LQ_BAD_SIZE;
    if (rows ? (!group_off || !tile_off || n_listed <= 0) : M <= 0) return LQ_BAD_SIZE;
    GroupedArgs a{(const __nv_bfloat16*)A, lda, a_group_stride, a_div, (const __nv_bfloat16*)W, w_group_stride, out, ldo,
                  o_group_stride, rows, group_off, tile_off, G, M, N, K, act};
    const int row_tiles = rows ? lq_grouped_gemm_tiles(n_listed, G) : G * ((M + BM - 1) / BM);
#define LQ_GO(TO, BN) do { \
        cudaFuncSetAttribute(grouped_gemm_kernel<TO, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gg_smem_bytes(BN)); \
        return launch_pdl(grouped_gemm_kernel<TO, BN>, dim3(row_tiles, (N + BN - 1) / BN), dim3(BN), gg_smem_bytes(BN), stream, a); } while (0)
    if (out_dtype == LQ_F32) { if (N >= 256) LQ_GO(float, 256); LQ_GO(float, 128); }
    if (out_dtype == LQ_BF16) { if (N >= 256) LQ_GO(__nv_bfloat16, 256); LQ_GO(__nv_bfloat16, 128); }
#undef LQ_GO
    return LQ_BAD_DTYPE;
}

LQ_EXPORT int lq_group_rows_padded(const int* ids, int n, int G, int tile, int cap, int* src, int* dst, int* tile_group,
                                   cudaStream_t stream) {
    if (n <= 0 || G <= 0 || tile <= 0 || cap % tile || cap < ((n + tile - 1) / tile + G) * tile) return LQ_BAD_SIZE;
    const size_t smem = 2 * (size_t)G * sizeof(int);
    if (smem > 48 * 1024) return LQ_BAD_SIZE;
    return launch_pdl(group_rows_padded_kernel, dim3(1), dim3(1024), smem, stream, ids, n, G, tile, cap, src, dst, tile_group);
}

// a [*, row_bytes] -> out [cap, row_bytes]; row_bytes a multiple of 16, both 16-byte aligned.
LQ_EXPORT int lq_gather_rows(const void* a, const int* src, int div, void* out, int cap, int row_bytes, cudaStream_t stream) {
    if (cap <= 0) return LQ_OK;
    if (row_bytes % 16 || div < 1 || (((uintptr_t)a | (uintptr_t)out) & 15)) return LQ_BAD_SIZE;
    return launch_pdl(gather_rows_kernel, dim3(cap), dim3(256), 0, stream, (const uint4*)a, src, div, (uint4*)out, cap, row_bytes / 16);
}

// ids (with E and h, bfloat16 [T, D]) or null; place or null: see moe_combine_kernel.
LQ_EXPORT int lq_moe_combine_more(const float* y, const int* place, const float* weights, const float* shared, const float* zs,
                                  int zs_stride, float* x, int accumulate, int T, int top, int D, const int* ids, int E,
                                  const void* h, float shared_scale, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (ids && !h) return LQ_BAD_SIZE;
    return launch_pdl(moe_combine_kernel, dim3(T), dim3(256), 0, stream, y, place, weights, shared, zs, zs_stride, x, accumulate,
                      top, D, ids, E, (const __nv_bfloat16*)h, shared_scale);
}

LQ_EXPORT int lq_moe_combine_at(const float* y, const int* place, const float* weights, const float* shared, const float* zs,
                                int zs_stride, float* x, int accumulate, int T, int top, int D, cudaStream_t stream) {
    return lq_moe_combine_more(y, place, weights, shared, zs, zs_stride, x, accumulate, T, top, D, nullptr, 0, nullptr, 1.f, stream);
}

LQ_EXPORT int lq_moe_combine(const float* y, const float* weights, const float* shared, const float* zs, int zs_stride, float* x,
                             int accumulate, int T, int top, int D, cudaStream_t stream) {
    return lq_moe_combine_more(y, nullptr, weights, shared, zs, zs_stride, x, accumulate, T, top, D, nullptr, 0, nullptr, 1.f, stream);
}
