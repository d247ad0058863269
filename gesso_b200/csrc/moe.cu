// Routed feed-forward (mixture of experts): the router, and the expert products for steps of few rows.
//
// Router (one warp per token, all float32).  The logits z = W_router x come from a matrix product with float32
// accumulation (bfloat16 operands are exact in it, so a bfloat16 run's logits are the float32 sums of the same
// numbers); this kernel does the rest:
//   z_e += logit_bias[e] (optional),
//   s_e = score(z_e)  (sigmoid, softmax over the experts, or z_e itself for weights that are the softmax over
//   the CHOSEN experts' logits only),
//   c_e = s_e + correction[e]                  (the score an expert is CHOSEN by; the weight uses s_e),
//   experts form `n_groups` equal groups of neighbours; a group's score is the sum of its `group_top`
//   largest c_e; only experts of the `keep_groups` best groups can be chosen (the others' c_e count as
//   -inf); the `top` largest c_e among those are chosen (ties: the lower index);
//   weight_k = s_e of the chosen expert, divided by the sum of the chosen weights with `renorm`,
//   times `weight_scale`.
// A token's choice and weights depend on its own logits only, not on what else is in the step.
//
// Expert products by (token, chosen expert) pair, for steps of few tokens, for the float32 path and for
// sizes the tensor-core path does not take: `moe_pair_up` computes act[pair] = act_fn(W_up[e] x) (a block
// per pair and 32 outputs, a warp per output, 16-byte weight reads), `moe_pair_down` computes
// y[token] = sum_k weight_k * (W_down[e_k] act[token, k]) in the order of the choice (a block per token and
// 32 outputs).  Weights of all experts are stacked: W_up [E, F, K], W_down [E, N, F].
//
// A gated activation (`MOE_ACT_GLU_CLAMPED`: g = min(gate, limit), u = clamp(up, -limit, limit),
// act = g * sigmoid(1.702 g) * (u + 1)) takes W_up [E, 2F, K] with an expert's gate and up rows together: groups
// of 8 gate rows followed by their 8 up rows (`glu_packed`, F % 8 == 0), or all F gate rows and then all F up rows;
// a warp then computes the eight gate rows and the eight up rows of its outputs.  `moe_pair_down` with
// `accumulate` adds its sums to what y holds (a shared expert's output, say).
#include <math.h>

#include "common.cuh"

enum { MOE_SCORE_SIGMOID = 0, MOE_SCORE_SOFTMAX = 1, MOE_SCORE_SOFTMAX_CHOSEN = 2 };
enum { MOE_ACT_RELU2 = 0, MOE_ACT_SILU = 1, MOE_ACT_GELU_TANH = 2, MOE_ACT_GLU_CLAMPED = 3 };
#define MOE_GLU_ALPHA 1.702f

__device__ __forceinline__ float moe_act(float v, int act) {
    if (act == MOE_ACT_RELU2) { const float r = fmaxf(v, 0.f); return r * r; }
    if (act == MOE_ACT_SILU) return v / (1.f + expf(-v));
    return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ logit_bias,
                 const float* __restrict__ correction, int* __restrict__ top_idx, float* __restrict__ top_w, int n_tokens, int E, int top,
                 int n_groups, int keep_groups, int group_top, int score_fn, int renorm, float weight_scale) {
    extern __shared__ float moe_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int t = blockIdx.x * 4 + wid;
    if (t >= n_tokens) return;                       // whole warps leave; no block barrier below
    float* s = moe_smem + (size_t)wid * (2 * E + n_groups);   // scores
    float* c = s + E;                                           // choice scores (-inf once taken or shut out)
    float* gs = c + E;                                          // group scores
    for (int e = lane; e < E; e += 32) s[e] = logits[(size_t)t * E + e] + (logit_bias ? logit_bias[e] : 0.f);
    __syncwarp();
    if (score_fn == MOE_SCORE_SOFTMAX) {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, s[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += expf(s[e] - m);
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) s[e] = expf(s[e] - m) / sum;
    } else if (score_fn == MOE_SCORE_SIGMOID) {
        for (int e = lane; e < E; e += 32) s[e] = 1.f / (1.f + expf(-s[e]));
    }                                                // MOE_SCORE_SOFTMAX_CHOSEN: the logits themselves
    __syncwarp();
    for (int e = lane; e < E; e += 32) c[e] = s[e] + (correction ? correction[e] : 0.f);
    __syncwarp();
    const int gsz = E / n_groups;
    if (keep_groups < n_groups) {
        // a group's score: the sum of its group_top largest choice scores
        for (int g = lane; g < n_groups; g += 32) {
            float sum = 0.f;
            int taken_a = -1, taken_b = -1;          // group_top <= 2 keeps the taken ones in two registers
            for (int k = 0; k < group_top && k < gsz; ++k) {
                float best = -INFINITY;
                int bi = -1;
                for (int i = 0; i < gsz; ++i) {
                    if (i == taken_a || i == taken_b) continue;
                    const float v = c[g * gsz + i];
                    if (bi < 0 || v > best) { best = v; bi = i; }
                }
                sum += best;
                if (k == 0) taken_a = bi; else taken_b = bi;
            }
            gs[g] = sum;
        }
        __syncwarp();
        // shut out the groups that are not among the keep_groups best (ties: the lower index wins)
        for (int g = lane; g < n_groups; g += 32) {
            int ahead = 0;
            const float mine = gs[g];
            for (int o = 0; o < n_groups; ++o) ahead += (gs[o] > mine) || (gs[o] == mine && o < g);
            if (ahead >= keep_groups)
                for (int i = 0; i < gsz; ++i) c[g * gsz + i] = -INFINITY;
        }
        __syncwarp();
    }
    float wsum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = c[e];
            if (v > best || (v == best && e < bi && v != -INFINITY)) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;                // fewer open experts than `top`: cannot happen for valid sizes
        const float w = s[bi];
        wsum += w;
        if (lane == 0) {
            top_idx[(size_t)t * top + k] = bi;
            top_w[(size_t)t * top + k] = w;
            c[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (score_fn == MOE_SCORE_SOFTMAX_CHOSEN) {      // softmax over the chosen experts' logits, nothing else
        const float z = lane < top ? top_w[(size_t)t * top + lane] : -INFINITY;
        const float m = warp_max(z);
        const float ex = lane < top ? expf(z - m) : 0.f;
        const float sum = warp_sum(ex);
        if (lane < top) top_w[(size_t)t * top + lane] = ex / sum * weight_scale;
        return;
    }
    if (lane < top) {
        float w = top_w[(size_t)t * top + lane];
        if (renorm) w /= wsum;
        top_w[(size_t)t * top + lane] = w * weight_scale;
    }
}

// logits [tokens, E], logit_bias [E] (or null) and correction [E] (or null) float32; top_idx / top_w [tokens, top].
GESSO_API int gesso_moe_route(const float* logits, const float* logit_bias, const float* correction, int* top_idx,
                              float* top_w, int n_tokens, int E, int top, int n_groups, int keep_groups,
                              int group_top, int score_fn, int renorm, float weight_scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (E <= 0 || top < 1 || top > E || top > 32 || n_groups < 1 || E % n_groups != 0 || keep_groups < 1 ||
        keep_groups > n_groups || group_top < 1 || group_top > 2 || (E / n_groups) * keep_groups < top)
        return GESSO_ERR_BAD_SIZE;
    const size_t smem = (size_t)4 * (2 * E + n_groups) * sizeof(float);
    if (smem > 48 * 1024) return GESSO_ERR_BAD_SIZE;
    const dim3 grid((n_tokens + 3) / 4);
    launch_pdl(moe_route_kernel, grid, dim3(128), smem, stream, logits, logit_bias, correction, top_idx, top_w, n_tokens, E, top,
               n_groups, keep_groups, group_top, score_fn, renorm, weight_scale);
    return launch_status();
}

// ---- expert products by (token, expert) pair -------------------------------------------------------------
// Dots of R weight rows (`stride` elements apart) with one float32 vector in shared memory.  All R rows' loads of
// a step are issued before any is used, so a lane keeps R 16-byte reads in flight: these kernels are bound by
// the latency of the weight stream, not by arithmetic.  Lanes stride over 8-element pieces (16-byte reads of
// bfloat16, two of float32) when the length and the alignment allow it.
template <typename TW> struct Piece;
template <> struct Piece<bf16> {
    uint4 u;
    __device__ __forceinline__ void load(const bf16* p) { u = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ float dot(const float* v) const {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc += __low2float(p[i]) * v[2 * i] + __high2float(p[i]) * v[2 * i + 1];
        return acc;
    }
};
template <> struct Piece<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = *reinterpret_cast<const float4*>(p);
        b = *reinterpret_cast<const float4*>(p + 4);
    }
    __device__ __forceinline__ float dot(const float* v) const {
        return a.x * v[0] + a.y * v[1] + a.z * v[2] + a.w * v[3] + b.x * v[4] + b.y * v[5] + b.z * v[6] + b.w * v[7];
    }
};

template <typename TW, int R>
__device__ __forceinline__ void rows_dot(const TW* __restrict__ w, size_t stride, int n_rows, const float* __restrict__ v,
                                         int K, int lane, float (&out)[R]) {
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    if (K % 8 == 0 && ((size_t)w & 15) == 0 && (stride * sizeof(TW)) % 16 == 0) {
        for (int j = lane * 8; j < K; j += 256) {
            Piece<TW> pc[R];
#pragma unroll
            for (int r = 0; r < R; ++r) pc[r].load(w + (size_t)(r < n_rows ? r : 0) * stride + j);
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] += pc[r].dot(v + j);
        }
    } else {
        for (int j = lane; j < K; j += 32) {
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] += to_f32(w[(size_t)(r < n_rows ? r : 0) * stride + j]) * v[j];
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) out[r] = warp_sum(acc[r]);
}

#define MOE_PAIR_OUTS 32      // outputs per block (8 per warp, taken together)
#define MOE_PAIR_MAX_SMEM (200 * 1024)     // the input row (up) or a token's activations of all its experts (down), float32

template <typename TX, typename TW>
__global__ void __launch_bounds__(128)
moe_pair_up_kernel(const TX* __restrict__ x, const TW* __restrict__ w_up, const int* __restrict__ top_idx,
                   TX* __restrict__ act_out, int top, int K, int F, int act, float limit, int glu_packed) {
    extern __shared__ float moe_smem[];
    const int pair = blockIdx.x, f0 = blockIdx.y * MOE_PAIR_OUTS;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    const int tok = pair / top;
    const int e = top_idx[pair];
    for (int j = threadIdx.x; j < K; j += 128) moe_smem[j] = to_f32(x[(size_t)tok * K + j]);
    __syncthreads();
    const int f = f0 + 8 * wid;                       // this warp's eight outputs
    if (f >= F) return;
    const int n_rows = min(8, F - f);
    float v[8];
    if (act == MOE_ACT_GLU_CLAMPED) {
        // the expert's 2F rows: gate rows of outputs f .. f+7, and their up rows 8 (packed) or F rows further on
        const TW* wg = w_up + ((size_t)e * 2 * F + (glu_packed ? 2 * f : f)) * K;
        float u[8];
        rows_dot<TW, 8>(wg, (size_t)K, n_rows, moe_smem, K, lane, v);
        rows_dot<TW, 8>(wg + (size_t)(glu_packed ? 8 : F) * K, (size_t)K, n_rows, moe_smem, K, lane, u);
        if (lane < n_rows) {
            float g = v[0], up = u[0];
#pragma unroll
            for (int r = 1; r < 8; ++r) { g = lane == r ? v[r] : g; up = lane == r ? u[r] : up; }
            g = fminf(g, limit);
            up = fminf(fmaxf(up, -limit), limit);
            act_out[(size_t)pair * F + f + lane] = from_f32<TX>((g / (1.f + expf(-MOE_GLU_ALPHA * g))) * (up + 1.f));
        }
        return;
    }
    rows_dot<TW, 8>(w_up + ((size_t)e * F + f) * K, (size_t)K, n_rows, moe_smem, K, lane, v);
    if (lane < n_rows) {
        float mine = v[0];
#pragma unroll
        for (int r = 1; r < 8; ++r) mine = lane == r ? v[r] : mine;
        act_out[(size_t)pair * F + f + lane] = from_f32<TX>(moe_act(mine, act));
    }
}

template <typename TX, typename TW>
__global__ void __launch_bounds__(128)
moe_pair_down_kernel(const TX* __restrict__ act_in, const TW* __restrict__ w_down, const int* __restrict__ top_idx,
                     const float* __restrict__ top_w, float* __restrict__ y, int top, int F, int N, int accumulate) {
    extern __shared__ float moe_smem[];
    const int tok = blockIdx.x, n0 = blockIdx.y * MOE_PAIR_OUTS;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    for (int j = threadIdx.x; j < top * F; j += 128) moe_smem[j] = to_f32(act_in[(size_t)tok * top * F + j]);
    __syncthreads();
    const int n = n0 + 8 * wid;                       // this warp's eight outputs
    if (n >= N) return;
    const int n_rows = min(8, N - n);
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top; ++k) {                   // in the order of the choice
        const int e = top_idx[(size_t)tok * top + k];
        const float wk = top_w[(size_t)tok * top + k];
        float v[8];
        rows_dot<TW, 8>(w_down + ((size_t)e * N + n) * F, (size_t)F, n_rows, moe_smem + (size_t)k * F, F, lane, v);
#pragma unroll
        for (int r = 0; r < 8; ++r) sum[r] += wk * v[r];
    }
    if (lane < n_rows) {
        float mine = sum[0];
#pragma unroll
        for (int r = 1; r < 8; ++r) mine = lane == r ? sum[r] : mine;
        float* dst = y + (size_t)tok * N + n + lane;
        *dst = accumulate ? *dst + mine : mine;
    }
}

// x [tokens, K] and act [tokens * top, F] of x_dtype; w_up [E, F, K] of w_dtype.
GESSO_API int gesso_moe_pair_up(const void* x, int x_dtype, const void* w_up, int w_dtype, const int* top_idx, void* act_out,
                                int n_tokens, int top, int K, int F, int act, float limit, int glu_packed,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (K <= 0 || F <= 0 || top < 1 || (size_t)K * sizeof(float) > MOE_PAIR_MAX_SMEM) return GESSO_ERR_BAD_SIZE;
    if (act == MOE_ACT_GLU_CLAMPED && glu_packed && F % 8 != 0) return GESSO_ERR_BAD_SIZE;
    const long long pairs = (long long)n_tokens * top;
    const int fb = (F + MOE_PAIR_OUTS - 1) / MOE_PAIR_OUTS;
    if (pairs > 2147483647LL || fb > 65535) return GESSO_ERR_BAD_SIZE;
    const dim3 grid((unsigned)pairs, fb);
    const size_t smem = (size_t)K * sizeof(float);
#define GO(TX, TW)                                                                                                   \
    do {                                                                                                             \
        static size_t configured = 48 * 1024;                                                                        \
        if (smem > configured) {                                                                                     \
            cudaFuncSetAttribute(moe_pair_up_kernel<TX, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                                 MOE_PAIR_MAX_SMEM);                                                                 \
            configured = MOE_PAIR_MAX_SMEM;                                                                          \
        }                                                                                                            \
        launch_pdl(moe_pair_up_kernel<TX, TW>, grid, dim3(128), smem, stream, (const TX*)x, (const TW*)w_up, top_idx, \
                   (TX*)act_out, top, K, F, act, limit, glu_packed);                                                                  \
    } while (0)
    if (x_dtype == GESSO_F32 && w_dtype == GESSO_F32) GO(float, float);
    else if (x_dtype == GESSO_F32 && w_dtype == GESSO_BF16) GO(float, bf16);
    else if (x_dtype == GESSO_BF16 && w_dtype == GESSO_BF16) GO(bf16, bf16);
    else if (x_dtype == GESSO_BF16 && w_dtype == GESSO_F32) GO(bf16, float);
    else return GESSO_ERR_BAD_DTYPE;
#undef GO
    return launch_status();
}

// act [tokens * top, F] of x_dtype; w_down [E, N, F] of w_dtype; y [tokens, N] float32.
GESSO_API int gesso_moe_pair_down(const void* act_in, int x_dtype, const void* w_down, int w_dtype, const int* top_idx,
                                  const float* top_w, float* y, int n_tokens, int top, int F, int N, int accumulate,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (N <= 0 || F <= 0 || top < 1 || (size_t)top * F * sizeof(float) > MOE_PAIR_MAX_SMEM) return GESSO_ERR_BAD_SIZE;
    const int nb = (N + MOE_PAIR_OUTS - 1) / MOE_PAIR_OUTS;
    if (nb > 65535) return GESSO_ERR_BAD_SIZE;
    const dim3 grid((unsigned)n_tokens, nb);
    const size_t smem = (size_t)top * F * sizeof(float);
#define GO(TX, TW)                                                                                                     \
    do {                                                                                                               \
        static size_t configured = 48 * 1024;                                                                          \
        if (smem > configured) {                                                                                       \
            cudaFuncSetAttribute(moe_pair_down_kernel<TX, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                                 MOE_PAIR_MAX_SMEM);                                                                   \
            configured = MOE_PAIR_MAX_SMEM;                                                                            \
        }                                                                                                              \
        launch_pdl(moe_pair_down_kernel<TX, TW>, grid, dim3(128), smem, stream, (const TX*)act_in, (const TW*)w_down,  \
                   top_idx, top_w, y, top, F, N, accumulate);                                                                    \
    } while (0)
    if (x_dtype == GESSO_F32 && w_dtype == GESSO_F32) GO(float, float);
    else if (x_dtype == GESSO_F32 && w_dtype == GESSO_BF16) GO(float, bf16);
    else if (x_dtype == GESSO_BF16 && w_dtype == GESSO_BF16) GO(bf16, bf16);
    else if (x_dtype == GESSO_BF16 && w_dtype == GESSO_F32) GO(bf16, float);
    else return GESSO_ERR_BAD_DTYPE;
#undef GO
    return launch_status();
}
