// Mixers that carry a matrix of fixed size per head from token to token instead of keys and values:
//
//   S_t = a_t S_(t-1) + b_t k_t v_t^T          o_t = S_t^T q_t
//
// with a_t, b_t scalars per head and token (or a_t a vector over the key channels: S_t = diag(a_t) S_(t-1) + ...).  Instances:
//   retention   a_t = the head's fixed decay, b_t = 1
//   channel decays   a_t[r] = sigmoid(z_t[r] + bias[r])^(1/tau) for key channel r, z from a 32-bit product of its own, b_t = 1
//   mlstm       a_t = exp(f_t + m_(t-1) - m_t), b_t = exp(i_t - m_t), m_t = max(f_t + m_(t-1), i_t), m_0 = 0,
//               i_t = cap tanh(x_i / cap), f_t = logsigmoid(cap tanh(x_f / cap)); the normaliser n_t (the same
//               recurrence with v = 1) rides along as one more value column, so n_t . q_t is that column's output
//
// State, products and gates are float32 whatever the activations' storage is; q and k are rotated (optionally)
// and scaled in float32 as they are staged, so nothing that enters the recurrence is rounded on the way.
// A sequence's tokens are walked in order from the state that the step before left in the sequence's slot, so a
// prompt gives the same bits however it is cut into portions; steps of one token per sequence have a form of
// their own (the same recurrence, sums in another order).
#include "common.cuh"
#include <math_constants.h>

constexpr int SC_R = 32;         // threads that share one value column: a warp, lane r holding key rows r, r + 32, ...
constexpr int SC_COLS = 16;      // value columns of a block (one warp each)
constexpr int SC_THREADS = SC_R * SC_COLS;
constexpr int SC_CHUNK = 16;     // tokens staged in shared memory at a time

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

struct ScanArgs {
    const void* qkv;             // [rows, stride]: q at q_off, k at k_off (H heads of dk each), v at v_off (H heads of dv)
    int stride, q_off, k_off, v_off;
    const float* cos_t;          // [positions, rot/2] or null
    const float* sin_t;
    int rot;                     // rotated dimensions of a head (pairs i, i + rot/2)
    const int* tok_pos;          // position of every row
    const float* gate_pre;       // mlstm: [rows, 2H] pre-activations of the input gates (H) and forget gates (H), no bias
    const float* gate_bias;      // mlstm: [2H]
    float gate_cap;
    const float* decay;          // retention: [H]
    float q_scale, k_scale;
    float* state;                // [slots][H][dk (+1)][dvx]; mlstm's extra row holds m (in every column)
    long long slot_stride;
    const int* cu_rows;          // [B + 1]
    const int* slots;            // [B]
    float* out;                  // [rows, H, dvx] raw S^T q (mlstm: column dv holds n . q)
    float* exp_neg_m;            // mlstm: [rows, H] exp(-m_t)
    int H, dk, dv;
    int in_act;                  // 0: q, k and v enter as stored; 1: each goes through silu first (in float32)
    const float* decay_pre;      // channel decays: [rows, decay_stride], head h's dk pre-activations at column h * dk
    int decay_stride;
    const float* decay_bias;     // channel decays: [H * dk] or null
    float inv_tau;               // channel decays: a = exp(logsigmoid(pre + bias) * inv_tau)
};

__device__ __forceinline__ float scan_in(float x, int act) { return act ? x / (1.f + expf(-x)) : x; }

// One block walks the tokens of one (sequence, head, 16 value columns) in chunks of SC_CHUNK; a warp owns a column,
// lane r the key rows r, r + 32, ... of it (KR of them).  While a chunk is multiplied, the next chunk's q, k and v
// are already on their way from memory into registers; they go to the other of two shared-memory buffers when
// the chunk is done (then rotated there pair by pair, then scaled).  Within a chunk a lane's share of S advances
// token by token (its only dependence); the outputs' partial sums stay in registers and are added across the
// warp once per chunk, in a fixed order.  The block's tile of the state comes and goes through shared memory in
// whole rows.
template <typename T, int KR, bool MLSTM, bool VEC>
__global__ void __launch_bounds__(SC_THREADS) linear_scan_kernel(ScanArgs a) {
    pdl_launch_dependents();
    extern __shared__ float sm[];
    const int dk = a.dk, dv = a.dv, dvx = dv + (MLSTM ? 1 : 0), dkx = dk + (MLSTM ? 1 : 0), H = a.H;
    const int qk_floats = SC_CHUNK * dk;
    // Two buffers each of q [CHUNK][dk], k [CHUNK][dk] and v [CHUNK][COLS].
    auto qs = [&](int buf) { return sm + buf * 2 * qk_floats; };
    auto ks = [&](int buf) { return sm + buf * 2 * qk_floats + qk_floats; };
    auto vs = [&](int buf) { return sm + 4 * qk_floats + buf * SC_CHUNK * SC_COLS; };
    float* as2 = sm + 4 * qk_floats + 2 * SC_CHUNK * SC_COLS;     // [2][CHUNK] a_t of the chunk in each buffer
    float* gi = as2 + 2 * SC_CHUNK;              // [CHUNK] b_t of the chunk being staged
    float* ms = gi + SC_CHUNK;                   // [CHUNK + 1] the running maximum after the chunk being staged
    float* tile = ms + SC_CHUNK + 1;             // [dkx][COLS + 1]: the block's columns of the state
    float* dsm = tile + (dk + 1) * (SC_COLS + 1);                 // channel decays: two buffers of [CHUNK][dk]
    auto ds = [&](int buf) { return dsm + buf * qk_floats; };
    const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * SC_COLS;
    const int tid = threadIdx.x, c = tid / SC_R, rr = tid % SC_R, col = col0 + c;
    const int n_cols = min(SC_COLS, dvx - col0);
    const bool live = c < n_cols;
    const T* base = (const T*)a.qkv;
    const int half = a.rot >> 1;
    constexpr int RF = (KR + 1) / 2;             // a thread's share of a chunk's rotated pairs
    pdl_wait();
    const int row0 = a.cu_rows[b], row1 = a.cu_rows[b + 1];
    float m = 0.f;
    float q_pf[KR], k_pf[KR], d_pf[VEC ? KR : 1], cs_pf[RF], sn_pf[RF], v_pf = 0.f, gi_pf = 0.f, gf_pf = 0.f;
    // Element e of a chunk's q (k) is token e / dk, dimension e % dk; thread tid holds e = tid + i * THREADS.
    // Which token and which place that is does not change from chunk to chunk: worked out once.
    int e_tok[KR], e_off[KR], e_dec[VEC ? KR : 1], r_tok[RF], r_dim[RF];
#pragma unroll
    for (int i = 0; i < KR; ++i) {
        const int e = tid + i * SC_THREADS;
        e_tok[i] = e / dk;                                            // >= CHUNK beyond the chunk
        e_off[i] = e_tok[i] * a.stride + h * dk + e % dk;
        if (VEC) e_dec[i] = e_tok[i] * a.decay_stride + h * dk + e % dk;
    }
#pragma unroll
    for (int i = 0; i < RF; ++i) {
        const int e = tid + i * SC_THREADS;
        r_tok[i] = half ? e / half : SC_CHUNK;
        r_dim[i] = half ? e % half : 0;
    }
    const int v_tok = tid / SC_COLS, v_col = col0 + tid % SC_COLS;
    const int v_at = v_tok * a.stride + a.v_off + h * dv + v_col;
    auto fetch = [&](int t0) {
        const int n = min(SC_CHUNK, row1 - t0);
        const T* rows = base + (size_t)t0 * a.stride;
#pragma unroll
        for (int i = 0; i < KR; ++i) {
            q_pf[i] = k_pf[i] = 0.f;
            if (e_tok[i] < n) {
                q_pf[i] = scan_in(to_f32(rows[e_off[i] + a.q_off]), a.in_act);
                k_pf[i] = scan_in(to_f32(rows[e_off[i] + a.k_off]), a.in_act);
                if (VEC) d_pf[i] = a.decay_pre[(size_t)t0 * a.decay_stride + e_dec[i]];
            }
        }
        if (half) {
#pragma unroll
            for (int i = 0; i < RF; ++i) {
                cs_pf[i] = 1.f;
                sn_pf[i] = 0.f;
                if (r_tok[i] < n) {
                    const size_t at = (size_t)a.tok_pos[t0 + r_tok[i]] * half + r_dim[i];
                    cs_pf[i] = a.cos_t[at];
                    sn_pf[i] = a.sin_t[at];
                }
            }
        }
        if (v_tok < SC_CHUNK) {
            v_pf = 0.f;
            if (v_tok < n) {
                if (v_col < dv) v_pf = scan_in(to_f32(rows[v_at]), a.in_act);
                else if (MLSTM && v_col == dv) v_pf = 1.f;
            }
        }
        if (MLSTM && tid < n) {
            const float* g = a.gate_pre + (size_t)(t0 + tid) * 2 * H;
            gi_pf = g[h] + a.gate_bias[h];
            gf_pf = g[H + h] + a.gate_bias[H + h];
        }
    };
    // What was fetched goes to buffer `buf`, ready for the recurrence: rotated, scaled, the gates worked out.
    auto stage = [&](int t0, int buf) {
        const int n = min(SC_CHUNK, row1 - t0);
#pragma unroll
        for (int i = 0; i < KR; ++i) {
            if (e_tok[i] < n) {
                qs(buf)[tid + i * SC_THREADS] = q_pf[i];
                ks(buf)[tid + i * SC_THREADS] = k_pf[i];
                if (VEC) {
                    // The decay of this token's key channel: sigmoid(z + bias)^(1/tau), through the logarithm, in 32-bit.
                    const int ch = h * dk + (tid + i * SC_THREADS) % dk;
                    const float z = d_pf[i] + (a.decay_bias ? a.decay_bias[ch] : 0.f);
                    ds(buf)[tid + i * SC_THREADS] = expf(log_sigmoid(z) * a.inv_tau);
                }
            }
        }
        if (MLSTM && tid < 32) {
            // The gates of the chunk's tokens, one lane each, and the running maximum
            //   m_t = max(f_t + m_(t-1), i_t) = F_t + max(m_0, max_(s<=t)(i_s - F_s)),  F_t = f_1 + ... + f_t,
            // as a prefix sum and a prefix maximum over the lanes.  Whatever rounding m_t has, a_t, b_t and
            // exp(-m_t) are made from the same m_t, so state and normaliser stay scaled alike.
            const float cap = a.gate_cap;
            const bool in = tid < n;
            const float li = in ? cap * tanhf(gi_pf / cap) : -CUDART_INF_F;
            const float lf = in ? log_sigmoid(cap * tanhf(gf_pf / cap)) : 0.f;
            float F = lf;
#pragma unroll
            for (int o = 1; o < SC_CHUNK; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, F, o);
                if (tid >= o) F += up;
            }
            float g = li - F;
#pragma unroll
            for (int o = 1; o < SC_CHUNK; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, g, o);
                if (tid >= o) g = fmaxf(g, up);
            }
            const float m_new = F + fmaxf(m, g);
            float m_old = __shfl_up_sync(0xffffffffu, m_new, 1);
            if (tid == 0) m_old = m;
            if (in) {
                as2[buf * SC_CHUNK + tid] = expf(lf + m_old - m_new);
                gi[tid] = expf(li - m_new);
                if (blockIdx.z == 0) a.exp_neg_m[(size_t)(t0 + tid) * H + h] = expf(-m_new);
            }
            if (tid == n - 1) ms[0] = m_new;
        }
        __syncthreads();
        if (MLSTM) m = ms[0];
        if (half) {
#pragma unroll
            for (int i = 0; i < RF; ++i) {
                if (r_tok[i] < n) {
                    const int t = r_tok[i], f = r_dim[i];
                    const float cs = cs_pf[i], sn = sn_pf[i];
                    float* qp = qs(buf) + t * dk + f;
                    float* kp = ks(buf) + t * dk + f;
                    const float qu = qp[0], qw = qp[half], ku = kp[0], kw = kp[half];
                    qp[0] = qu * cs - qw * sn;
                    qp[half] = qw * cs + qu * sn;
                    kp[0] = ku * cs - kw * sn;
                    kp[half] = kw * cs + ku * sn;
                }
            }
        }
        __syncthreads();
        if (v_tok < n) vs(buf)[tid] = MLSTM ? v_pf * gi[v_tok] : v_pf;
#pragma unroll
        for (int i = 0; i < KR; ++i) {                              // the scales come after the rotation
            if (e_tok[i] < n) {
                qs(buf)[tid + i * SC_THREADS] *= a.q_scale;
                ks(buf)[tid + i * SC_THREADS] *= a.k_scale;
            }
        }
        __syncthreads();
    };

    if (row0 < row1) fetch(row0);                // on its way while the state's tile arrives
    float* st = a.state + (long long)a.slots[b] * a.slot_stride + (size_t)h * dkx * dvx + col0;
    for (int e = tid; e < dkx * SC_COLS; e += SC_THREADS) {
        const int r = e / SC_COLS, cc = e % SC_COLS;
        tile[r * (SC_COLS + 1) + cc] = cc < n_cols ? st[(size_t)r * dvx + cc] : 0.f;
    }
    __syncthreads();
    float S[KR];
#pragma unroll
    for (int i = 0; i < KR; ++i) {
        const int r = i * SC_R + rr;
        S[i] = r < dk ? tile[r * (SC_COLS + 1) + c] : 0.f;
    }
    if (MLSTM) m = tile[dk * (SC_COLS + 1)];
    const float decay = (MLSTM || VEC) ? 0.f : a.decay[h];

    if (row0 < row1) stage(row0, 0);
    int buf = 0;
    for (int t0 = row0; t0 < row1; t0 += SC_CHUNK, buf ^= 1) {
        const int n = min(SC_CHUNK, row1 - t0);
        const bool more = t0 + SC_CHUNK < row1;
        if (more) fetch(t0 + SC_CHUNK);          // in flight while this chunk is multiplied
        float acc[SC_CHUNK];
#pragma unroll
        for (int t = 0; t < SC_CHUNK; ++t) {
            acc[t] = 0.f;
            if (t < n) {
                const float at = MLSTM ? as2[buf * SC_CHUNK + t] : decay;
                const float bv = vs(buf)[t * SC_COLS + c];
                const float* kt = ks(buf) + t * dk;
                const float* qt = qs(buf) + t * dk;
                const float* dt = VEC ? ds(buf) + t * dk : nullptr;
#pragma unroll
                for (int i = 0; i < KR; ++i) {
                    const int r = i * SC_R + rr;
                    if (r < dk) {
                        S[i] = fmaf(VEC ? dt[r] : at, S[i], bv * kt[r]);
                        acc[t] = fmaf(S[i], qt[r], acc[t]);
                    }
                }
            }
        }
        // Sixteen sums over the warp's lanes at once: in each of four steps a lane hands half of its values to
        // the lane across and adds the half it keeps, so that lane l is left with token (l & 15)'s sum over the
        // lanes that agree with it in bit 4; one more exchange adds the two halves of the warp.
#pragma unroll
        for (int w = 8; w >= 1; w >>= 1) {
            const bool upper = rr & w;
#pragma unroll
            for (int t = 0; t < w; ++t) {
                const float give = upper ? acc[t] : acc[t + w];
                const float keep = upper ? acc[t + w] : acc[t];
                acc[t] = keep + __shfl_xor_sync(0xffffffffu, give, w);
            }
        }
        const float mine = acc[0] + __shfl_xor_sync(0xffffffffu, acc[0], 16);
        const int my_tok = rr & 15;              // bits 3..0 of the lane chose the upper or lower half at w = 8, 4, 2, 1
        if (live && rr < 16 && my_tok < n) a.out[((size_t)(t0 + my_tok) * H + h) * dvx + col] = mine;
        if (more) stage(t0 + SC_CHUNK, buf ^ 1);
        else __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < KR; ++i) {
        const int r = i * SC_R + rr;
        if (r < dk) tile[r * (SC_COLS + 1) + c] = S[i];
    }
    if (MLSTM && rr == 0) tile[dk * (SC_COLS + 1) + c] = m;
    __syncthreads();
    for (int e = tid; e < dkx * SC_COLS; e += SC_THREADS) {
        const int r = e / SC_COLS, cc = e % SC_COLS;
        if (cc < n_cols) st[(size_t)r * dvx + cc] = tile[r * (SC_COLS + 1) + cc];
    }
}

// The same recurrence for a step in which every sequence brings one token: nothing to pipeline, so the state
// streams through once.  A block per (sequence, head, 32 value columns); a lane per column, so that a row of the
// state is one contiguous read; the eight warps share the key rows (warp w: rows w, w + 8, ...) and their partial
// outputs meet in shared memory, added in the order of the warps.
constexpr int SS_WARPS = 8;

template <typename T, bool MLSTM, bool VEC>
__global__ void __launch_bounds__(SS_WARPS * 32) linear_scan_single_kernel(ScanArgs a) {
    pdl_launch_dependents();
    extern __shared__ float sm[];
    const int dk = a.dk, dv = a.dv, dvx = dv + (MLSTM ? 1 : 0), dkx = dk + (MLSTM ? 1 : 0), H = a.H;
    float* qs = sm;                              // [dk] rotated, scaled
    float* ks = qs + dk;                         // [dk]
    float* red = ks + dk;                        // [WARPS][32]
    float* as = red + SS_WARPS * 32;             // channel decays: [dk]
    const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col = blockIdx.z * 32 + lane;
    const bool live = col < dvx;
    const int half = a.rot >> 1;
    pdl_wait();
    const int row = a.cu_rows[b];
    const T* x = (const T*)a.qkv + (size_t)row * a.stride;
    float* st = a.state + (long long)a.slots[b] * a.slot_stride + (size_t)h * dkx * dvx;
    for (int j = tid; j < dk; j += SS_WARPS * 32) {
        float qv = scan_in(to_f32(x[a.q_off + h * dk + j]), a.in_act), kv = scan_in(to_f32(x[a.k_off + h * dk + j]), a.in_act);
        if (j < a.rot) {
            const int f = j < half ? j : j - half, jp = j < half ? j + half : j - half;
            const size_t at = (size_t)a.tok_pos[row] * half + f;
            const float cs = a.cos_t[at], sn = j < half ? -a.sin_t[at] : a.sin_t[at];
            qv = qv * cs + scan_in(to_f32(x[a.q_off + h * dk + jp]), a.in_act) * sn;
            kv = kv * cs + scan_in(to_f32(x[a.k_off + h * dk + jp]), a.in_act) * sn;
        }
        qs[j] = qv * a.q_scale;
        ks[j] = kv * a.k_scale;
        if (VEC) {
            const float z = a.decay_pre[(size_t)row * a.decay_stride + h * dk + j] + (a.decay_bias ? a.decay_bias[h * dk + j] : 0.f);
            as[j] = expf(log_sigmoid(z) * a.inv_tau);
        }
    }
    float v = 0.f;
    if (col < dv) v = scan_in(to_f32(x[a.v_off + h * dv + col]), a.in_act);
    else if (MLSTM && col == dv) v = 1.f;
    float keep = (MLSTM || VEC) ? 0.f : a.decay[h], m_new = 0.f;
    if (MLSTM) {
        const float cap = a.gate_cap;
        const float* g = a.gate_pre + (size_t)row * 2 * H;
        const float li = cap * tanhf((g[h] + a.gate_bias[h]) / cap);
        const float lf = log_sigmoid(cap * tanhf((g[H + h] + a.gate_bias[H + h]) / cap));
        const float m_old = st[(size_t)dk * dvx + (live ? col : blockIdx.z * 32)];
        m_new = fmaxf(lf + m_old, li);
        keep = expf(lf + m_old - m_new);
        v *= expf(li - m_new);
        if (blockIdx.z == 0 && tid == 0) a.exp_neg_m[(size_t)row * H + h] = expf(-m_new);
    }
    __syncthreads();
    float acc = 0.f;
    if (live) {
#pragma unroll 4
        for (int r = warp; r < dk; r += SS_WARPS) {
            float* sp = st + (size_t)r * dvx + col;
            const float s_new = fmaf(VEC ? as[r] : keep, *sp, v * ks[r]);
            *sp = s_new;
            acc = fmaf(s_new, qs[r], acc);
        }
        if (MLSTM && warp == 0) st[(size_t)dk * dvx + col] = m_new;
    }
    red[warp * 32 + lane] = acc;
    __syncthreads();
    if (warp == 0 && live) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < SS_WARPS; ++w) total += red[w * 32 + lane];
        a.out[((size_t)row * H + h) * dvx + col] = total;
    }
}

template <typename T, bool MLSTM, bool VEC>
static int scan_single_launch(const ScanArgs& a, int B, cudaStream_t stream) {
    const int dvx = a.dv + (MLSTM ? 1 : 0);
    const size_t smem = (size_t)(2 * a.dk + SS_WARPS * 32 + (VEC ? a.dk : 0)) * sizeof(float);
    return launch_pdl(linear_scan_single_kernel<T, MLSTM, VEC>, dim3(B, a.H, (dvx + 31) / 32), dim3(SS_WARPS * 32), smem, stream, a);
}

template <typename T, bool MLSTM, bool VEC>
static int scan_launch(const ScanArgs& a, int B, cudaStream_t stream) {
    const int dvx = a.dv + (MLSTM ? 1 : 0);
    dim3 grid(B, a.H, (dvx + SC_COLS - 1) / SC_COLS);
    const size_t smem = (size_t)(4 * SC_CHUNK * a.dk + 2 * SC_CHUNK * SC_COLS + 4 * SC_CHUNK + 1 +
                                 (a.dk + 1) * (SC_COLS + 1) + (VEC ? 2 * SC_CHUNK * a.dk : 0)) * sizeof(float);      // a little more than the kernel lays out
    auto go = [&](auto kernel) {
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return lq_launch_status();
        return launch_pdl(kernel, grid, dim3(SC_THREADS), smem, stream, a);
    };
    if (a.dk <= 1 * SC_R) return go(linear_scan_kernel<T, 1, MLSTM, VEC>);
    if (a.dk <= 2 * SC_R) return go(linear_scan_kernel<T, 2, MLSTM, VEC>);
    if (a.dk <= 4 * SC_R) return go(linear_scan_kernel<T, 4, MLSTM, VEC>);
    if (a.dk <= 8 * SC_R) return go(linear_scan_kernel<T, 8, MLSTM, VEC>);
    return LQ_BAD_SIZE;
}

LQ_EXPORT int lq_linear_scan(const void* qkv, int dtype, int stride, int q_off, int k_off, int v_off, const float* cos_t,
                             const float* sin_t, int rot, const int* tok_pos, const float* gate_pre,
                             const float* gate_bias, float gate_cap, const float* decay, float q_scale, float k_scale,
                             float* state, long long slot_stride, const int* cu_rows, const int* slots, float* out,
                             float* exp_neg_m, int B, int H, int dk, int dv, int mlstm, int single, int in_act,
                             const float* decay_pre, int decay_stride, const float* decay_bias, float inv_tau,
                             cudaStream_t stream) {
    if (B <= 0) return LQ_OK;
    if (in_act < 0 || in_act > 1) return LQ_BAD_SIZE;
    if (rot % 2 || rot > dk || (rot && (!cos_t || !sin_t))) return LQ_BAD_SIZE;
    const bool vec = decay_pre != nullptr;          // a decay per key channel and token instead of one per head
    if (mlstm ? (!gate_pre || !gate_bias || !exp_neg_m || vec) : (!decay && !vec)) return LQ_BAD_SIZE;
    ScanArgs a{qkv, stride, q_off, k_off, v_off, cos_t, sin_t, rot, tok_pos, gate_pre, gate_bias, gate_cap, decay,
               q_scale, k_scale, state, slot_stride, cu_rows, slots, out, exp_neg_m, H, dk, dv, in_act,
               decay_pre, decay_stride, decay_bias, inv_tau};
    typedef __nv_bfloat16 bf;
    if (dtype != LQ_F32 && dtype != LQ_BF16) return LQ_BAD_DTYPE;
    const bool f32 = dtype == LQ_F32;
    if (single) {
        // Every sequence brings exactly one token (row cu_rows[b]).
        if (dk > 256) return LQ_BAD_SIZE;
        if (mlstm) return f32 ? scan_single_launch<float, true, false>(a, B, stream) : scan_single_launch<bf, true, false>(a, B, stream);
        if (vec) return f32 ? scan_single_launch<float, false, true>(a, B, stream) : scan_single_launch<bf, false, true>(a, B, stream);
        return f32 ? scan_single_launch<float, false, false>(a, B, stream) : scan_single_launch<bf, false, false>(a, B, stream);
    }
    if (mlstm) return f32 ? scan_launch<float, true, false>(a, B, stream) : scan_launch<bf, true, false>(a, B, stream);
    if (vec) return f32 ? scan_launch<float, false, true>(a, B, stream) : scan_launch<bf, false, true>(a, B, stream);
    return f32 ? scan_launch<float, false, false>(a, B, stream) : scan_launch<bf, false, false>(a, B, stream);
}

// ------------------------------------------------------------------ per-head unit norm, weight and gate
// raw [rows, H, dvx] float32 -> out [rows, H * dv]: each head's dv values (divided by the head's denominator
// first, where there is one) over their root mean square, times weight [H * dv] (optional), times
// act(gate[row, h * dv + d]) (0: no gate, 1: sigmoid, 2: silu).  One warp per (row, head); the sum of squares
// runs in an order that depends on dv alone.
// Denominator (mlstm): max(|raw[row, h, dv]|, exp_neg_m[row, h]) + 1e-6.
template <typename T>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const float* __restrict__ raw, int dvx,
                                                             const float* __restrict__ exp_neg_m,
                                                             const float* __restrict__ weight, const T* __restrict__ gate,
                                                             int gate_stride, int act, T* __restrict__ out, int n_pairs,
                                                             int H, int dv, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    const int row = pair / H, h = pair % H;
    const float* r = raw + (size_t)pair * dvx;
    float inv = 1.f;
    if (exp_neg_m) inv = 1.f / (fmaxf(fabsf(r[dv]), exp_neg_m[pair]) + 1e-6f);
    float s = 0.f;
    for (int d = lane; d < dv; d += 32) {
        const float v = r[d] * inv;
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    const float scale = inv / sqrtf(s / (float)dv + eps);
    for (int d = lane; d < dv; d += 32) {
        float v = r[d] * scale;
        if (weight) v *= weight[h * dv + d];
        if (act) {
            const float g = to_f32(gate[(size_t)row * gate_stride + h * dv + d]);
            const float sg = 1.f / (1.f + expf(-g));
            v *= act == 1 ? sg : g * sg;
        }
        out[(size_t)row * H * dv + h * dv + d] = from_f32<T>(v);
    }
}

// The same for heads of many values (all heads normed together count as one head): a block per (row, head).
template <typename T>
__global__ void __launch_bounds__(256) head_norm_gate_wide_kernel(const float* __restrict__ raw, int dvx,
                                                                  const float* __restrict__ exp_neg_m,
                                                                  const float* __restrict__ weight, const T* __restrict__ gate,
                                                                  int gate_stride, int act, T* __restrict__ out, int H, int dv,
                                                                  float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[8];
    const int pair = blockIdx.x, tid = threadIdx.x;
    const int row = pair / H, h = pair % H;
    const float* r = raw + (size_t)pair * dvx;
    float inv = 1.f;
    if (exp_neg_m) inv = 1.f / (fmaxf(fabsf(r[dv]), exp_neg_m[pair]) + 1e-6f);
    float s = 0.f;
    for (int d = tid; d < dv; d += 256) {
        const float v = r[d] * inv;
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    if ((tid & 31) == 0) red[tid >> 5] = s;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += red[w];
    const float scale = inv / sqrtf(total / (float)dv + eps);
    for (int d = tid; d < dv; d += 256) {
        float v = r[d] * scale;
        if (weight) v *= weight[h * dv + d];
        if (act) {
            const float g = to_f32(gate[(size_t)row * gate_stride + h * dv + d]);
            const float sg = 1.f / (1.f + expf(-g));
            v *= act == 1 ? sg : g * sg;
        }
        out[(size_t)row * H * dv + h * dv + d] = from_f32<T>(v);
    }
}

LQ_EXPORT int lq_head_norm_gate(const float* raw, int dvx, const float* exp_neg_m, const float* weight, const void* gate,
                                int gate_stride, int act, void* out, int dtype, int rows, int H, int dv, float eps,
                                cudaStream_t stream) {
    const int n = rows * H;
    if (n <= 0) return LQ_OK;
    if (act < 0 || act > 2 || (act && !gate)) return LQ_BAD_SIZE;
    if (dv >= 512) {
        if (dtype == LQ_F32)
            return launch_pdl(head_norm_gate_wide_kernel<float>, dim3(n), dim3(256), 0, stream, raw, dvx, exp_neg_m, weight,
                              (const float*)gate, gate_stride, act, (float*)out, H, dv, eps);
        if (dtype == LQ_BF16)
            return launch_pdl(head_norm_gate_wide_kernel<__nv_bfloat16>, dim3(n), dim3(256), 0, stream, raw, dvx, exp_neg_m, weight,
                              (const __nv_bfloat16*)gate, gate_stride, act, (__nv_bfloat16*)out, H, dv, eps);
        return LQ_BAD_DTYPE;
    }
    dim3 grid((n + 3) / 4);
    if (dtype == LQ_F32)
        return launch_pdl(head_norm_gate_kernel<float>, grid, dim3(128), 0, stream, raw, dvx, exp_neg_m, weight,
                          (const float*)gate, gate_stride, act, (float*)out, n, H, dv, eps);
    if (dtype == LQ_BF16)
        return launch_pdl(head_norm_gate_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, raw, dvx, exp_neg_m, weight,
                          (const __nv_bfloat16*)gate, gate_stride, act, (__nv_bfloat16*)out, n, H, dv, eps);
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ a projection onto few outputs, in 32-bit
// out[t, j] = sum_k x[t, k] W[j, k] in float32 for a weight of few rows (the gates of a recurrent mixer: two per
// head).  One block per four rows of x (kept in shared memory as float32) and eight outputs, a warp per output, its lanes
// striding over k, partial sums added across the lanes in a fixed order: the order of sums depends on K alone.
constexpr int SP_ROWS = 4;       // rows of x per block: a row of W is read once for all of them
template <typename TX, typename TW>
__global__ void __launch_bounds__(256) small_proj_kernel(const TX* __restrict__ x, const TW* __restrict__ w,
                                                         float* __restrict__ out, int rows, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float xs[];                 // [SP_ROWS][K]
    const int t0 = blockIdx.x * SP_ROWS, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = min(SP_ROWS, rows - t0);
    for (int e = threadIdx.x; e < SP_ROWS * K; e += 256) xs[e] = e < n * K ? to_f32(x[(size_t)t0 * K + e]) : 0.f;
    __syncthreads();
    {
        const int j = blockIdx.y * 8 + warp;       // a warp per output
        if (j >= N) return;
        const TW* wr = w + (size_t)j * K;
        float s[SP_ROWS][4] = {};
        int k = lane;
        for (; k + 96 < K; k += 128) {
            const float w0 = to_f32(wr[k]), w1 = to_f32(wr[k + 32]), w2 = to_f32(wr[k + 64]), w3 = to_f32(wr[k + 96]);
#pragma unroll
            for (int r = 0; r < SP_ROWS; ++r) {
                const float* xr = xs + r * K + k;
                s[r][0] = fmaf(xr[0], w0, s[r][0]);
                s[r][1] = fmaf(xr[32], w1, s[r][1]);
                s[r][2] = fmaf(xr[64], w2, s[r][2]);
                s[r][3] = fmaf(xr[96], w3, s[r][3]);
            }
        }
        for (; k < K; k += 32) {
            const float w0 = to_f32(wr[k]);
#pragma unroll
            for (int r = 0; r < SP_ROWS; ++r) s[r][0] = fmaf(xs[r * K + k], w0, s[r][0]);
        }
#pragma unroll
        for (int r = 0; r < SP_ROWS; ++r) {
            const float v = warp_sum((s[r][0] + s[r][1]) + (s[r][2] + s[r][3]));
            if (lane == 0 && r < n) out[(size_t)(t0 + r) * N + j] = v;
        }
    }
}

LQ_EXPORT int lq_small_proj(const void* x, int x_dtype, const void* w, int w_dtype, float* out, int rows, int N, int K,
                            cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return LQ_OK;
    const size_t smem = (size_t)SP_ROWS * K * sizeof(float);
    if (smem > 200 * 1024) return LQ_BAD_SIZE;
    auto go = [&](auto kernel, auto xp, auto wp) {
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return lq_launch_status();
        return launch_pdl(kernel, dim3((rows + SP_ROWS - 1) / SP_ROWS, (N + 7) / 8), dim3(256), smem, stream, xp, wp, out, rows, N, K);
    };
    typedef __nv_bfloat16 bf;
    if (x_dtype == LQ_F32 && w_dtype == LQ_F32) return go(small_proj_kernel<float, float>, (const float*)x, (const float*)w);
    if (x_dtype == LQ_F32 && w_dtype == LQ_BF16) return go(small_proj_kernel<float, bf>, (const float*)x, (const bf*)w);
    if (x_dtype == LQ_BF16 && w_dtype == LQ_F32) return go(small_proj_kernel<bf, float>, (const bf*)x, (const float*)w);
    if (x_dtype == LQ_BF16 && w_dtype == LQ_BF16) return go(small_proj_kernel<bf, bf>, (const bf*)x, (const bf*)w);
    return LQ_BAD_DTYPE;
}
