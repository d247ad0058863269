// Gated linear attention: linear attention whose decay is computed from the input, one number per key channel
// and token, as a recurrence over a per-request state.
//
// Per head, with q_t, k_t, a_t (D features) and v_t (Dv features):
//     a_t = exp(log_sigmoid(z_t) / tau)              (z_t: the decay's logits, float32; 0 < a_t < 1)
//     S_t = diag(a_t) S_{t-1} + k_t v_t^T            (S: [D, Dv] float32, zero at the start of a request)
//     o_t = S_t^T (q_scale * q_t)
// The recurrence runs in float32 whatever the run type: the logits, the decay, the state, the outer product and
// the read-out.  q, k and v arrive as rows of a fused matrix product (q columns, then k, then v; further columns
// may follow) in the run type; the logits as a float32 matrix [tokens, H * D] with an optional bias [H * D].
//
// One kernel serves prompt portions and single tokens.  The columns of S are independent, so a block owns
// (segment, head, a group of value columns) and walks the segment's tokens in order; a column's D state values
// are spread over L lanes (L a power of two, 16 values in registers per lane, zeros behind D), the read-out is
// summed over those lanes by shuffles.  A tile of tokens' q, k, a and v is staged through shared memory at a time.
// The state is stored [slot][head][value column][feature], as the fixed-decay recurrence stores it.
//
// head_gated_rmsnorm: y = (o / sqrt(mean_head(o^2) + eps)) * w * act(g) per head of a token (w has one head's
// width and is shared by the heads; act = sigmoid or silu), the norm in float32; g are columns of the fused
// projection.
#include <math.h>

#include "common.cuh"

#define GLA_THREADS 128
#define GLA_PER_LANE 16

// log(sigmoid(z)) = -softplus(-z), without overflow on either side
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T, int L>
__global__ void __launch_bounds__(GLA_THREADS)
gla_kernel(const T* __restrict__ proj, int row_stride, const float* __restrict__ z, const float* __restrict__ z_bias,
           float inv_tau, float q_scale, float* __restrict__ state, long long slot_stride,
           const int* __restrict__ seg_start, const int* __restrict__ slots, float* __restrict__ out, int H, int D,
           int Dv, int tile) {
    extern __shared__ __align__(16) float gla_smem[];
    constexpr int COLS = GLA_THREADS / L;           // value columns of a block
    constexpr int DP = L * GLA_PER_LANE;            // features of a head, padded to whole lanes (zeros behind D)
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int cw = threadIdx.x / L, part = threadIdx.x % L;
    const int col = c0 + cw;
    const int d0 = part * GLA_PER_LANE;             // this lane's features d0 .. d0 + 15
    const bool live = col < Dv;
    const int t0 = seg_start[s], n = seg_start[s + 1] - t0;
    float* st = state + (size_t)slots[s] * slot_stride + ((size_t)h * Dv + (live ? col : 0)) * D;
    float S[GLA_PER_LANE];
#pragma unroll
    for (int i = 0; i < GLA_PER_LANE; ++i) S[i] = (live && d0 + i < D) ? st[d0 + i] : 0.f;
    float* sq = gla_smem;                           // [tile][DP]
    float* sk = sq + (size_t)tile * DP;             // [tile][DP]
    float* sa = sk + (size_t)tile * DP;             // [tile][DP]
    float* sv = sa + (size_t)tile * DP;             // [tile][COLS]
    const int qo = h * D, ko = H * D + h * D, vo = 2 * H * D + h * Dv;
    for (int base = 0; base < n; base += tile) {
        const int m = min(tile, n - base);
        __syncthreads();
        for (int j = threadIdx.x; j < m * DP; j += GLA_THREADS) {
            const int d = j % DP;
            const size_t tok = (size_t)(t0 + base + j / DP);
            const T* row = proj + tok * row_stride;
            const bool on = d < D;
            sq[j] = on ? q_scale * to_f32(row[qo + d]) : 0.f;
            sk[j] = on ? to_f32(row[ko + d]) : 0.f;
            float zz = on ? z[tok * ((size_t)H * D) + qo + d] : 0.f;
            if (on && z_bias) zz += z_bias[qo + d];
            sa[j] = on ? expf(log_sigmoid_f(zz) * inv_tau) : 0.f;
        }
        for (int j = threadIdx.x; j < m * COLS; j += GLA_THREADS) {
            const int c = c0 + j % COLS;
            sv[j] = c < Dv ? to_f32(proj[(size_t)(t0 + base + j / COLS) * row_stride + vo + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll 2
        for (int i = 0; i < m; ++i) {
            const float v = sv[i * COLS + cw];
            const float4* q4 = reinterpret_cast<const float4*>(sq + (size_t)i * DP + d0);
            const float4* k4 = reinterpret_cast<const float4*>(sk + (size_t)i * DP + d0);
            const float4* a4 = reinterpret_cast<const float4*>(sa + (size_t)i * DP + d0);
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int r = 0; r < GLA_PER_LANE / 4; ++r) {
                const float4 kk = k4[r], qq = q4[r], aa = a4[r];
                S[4 * r] = fmaf(aa.x, S[4 * r], kk.x * v);
                S[4 * r + 1] = fmaf(aa.y, S[4 * r + 1], kk.y * v);
                S[4 * r + 2] = fmaf(aa.z, S[4 * r + 2], kk.z * v);
                S[4 * r + 3] = fmaf(aa.w, S[4 * r + 3], kk.w * v);
                o0 = fmaf(S[4 * r], qq.x, o0);
                o1 = fmaf(S[4 * r + 1], qq.y, o1);
                o0 = fmaf(S[4 * r + 2], qq.z, o0);
                o1 = fmaf(S[4 * r + 3], qq.w, o1);
            }
            float o = o0 + o1;
#pragma unroll
            for (int x = L / 2; x > 0; x >>= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
            if (part == 0 && live) out[(size_t)(t0 + base + i) * H * Dv + (size_t)h * Dv + col] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < GLA_PER_LANE; ++i)
            if (d0 + i < D) st[d0 + i] = S[i];
    }
}

// proj [n_tokens, row_stride] of `dtype`: q at column 0 (H * D), k at H * D, v at 2 * H * D (H * Dv).  z [n_tokens, H * D]
// float32 (+ z_bias [H * D] or null).  state: this layer's view, slot s at state + s * slot_stride floats, [H][Dv][D].
// out [n_tokens, H * Dv] float32.
GESSO_API int gesso_gla(const void* proj, int dtype, int row_stride, const float* z, const float* z_bias, float tau,
                        float q_scale, float* state, long long slot_stride, const int* seg_start, const int* slots,
                        float* out, int n_tokens, int n_segs, int H, int D, int Dv, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segs <= 0) return 0;
    if (H <= 0 || D <= 0 || Dv <= 0 || D > 32 * GLA_PER_LANE || H > 65535 || row_stride < 2 * H * D + H * Dv || !(tau > 0.f))
        return GESSO_ERR_BAD_SIZE;
    int L = 1;
    while (L * GLA_PER_LANE < D) L <<= 1;
    const int cols = GLA_THREADS / L;
    if ((Dv + cols - 1) / cols > 65535) return GESSO_ERR_BAD_SIZE;
    const int dp = L * GLA_PER_LANE;
    int tile = 32;
    while (tile > 1 && (size_t)tile * (3 * dp + cols) * sizeof(float) > 44 * 1024) tile >>= 1;
    const size_t smem = (size_t)tile * (3 * dp + cols) * sizeof(float);
    const dim3 grid(n_segs, H, (Dv + cols - 1) / cols);
#define GO(T, LL)                                                                                                   \
    launch_pdl(gla_kernel<T, LL>, grid, dim3(GLA_THREADS), smem, stream, (const T*)proj, row_stride, z, z_bias,     \
               1.f / tau, q_scale, state, slot_stride, seg_start, slots, out, H, D, Dv, tile)
#define BY_L(T)                                                                                                     \
    switch (L) {                                                                                                    \
        case 1: GO(T, 1); break;                                                                                    \
        case 2: GO(T, 2); break;                                                                                    \
        case 4: GO(T, 4); break;                                                                                    \
        case 8: GO(T, 8); break;                                                                                    \
        case 16: GO(T, 16); break;                                                                                  \
        default: GO(T, 32); break;                                                                                  \
    }
    if (dtype == GESSO_F32) { BY_L(float) }
    else if (dtype == GESSO_BF16) { BY_L(bf16) }
    else return GESSO_ERR_BAD_DTYPE;
#undef BY_L
#undef GO
    return launch_status();
}

// ---- norm per head, times act(gate) ---------------------------------------------------------------------------------
enum { GATE_SIGMOID = 0, GATE_SILU = 1 };

template <typename T>
__global__ void __launch_bounds__(128)
head_gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, const T* __restrict__ gate,
                          int gate_stride, T* __restrict__ out, long long n_rows, int n_heads, int Dv, int gate_act) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long wi = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (wi >= n_rows * n_heads) return;
    const long long r = wi / n_heads;
    const int hh = (int)(wi % n_heads);
    const float* row = o + (r * n_heads + hh) * Dv;
    float ss = 0.f;
    for (int j = lane; j < Dv; j += 32) ss = fmaf(row[j], row[j], ss);
    const float denom = sqrtf(warp_sum(ss) / (float)Dv + eps);
    const T* g = gate + r * gate_stride + (size_t)hh * Dv;
    T* orow = out + (r * n_heads + hh) * Dv;
    for (int j = lane; j < Dv; j += 32) {
        const float gv = to_f32(g[j]);
        const float sg = 1.f / (1.f + expf(-gv));
        orow[j] = from_f32<T>((row[j] / denom) * w[j] * (gate_act == GATE_SILU ? gv * sg : sg));
    }
}

// o [n_rows, n_heads * Dv] float32; w [Dv] float32; gate: [n_rows, gate_stride] of `dtype` (the n_heads * Dv gate
// columns at gate); out [n_rows, n_heads * Dv] of `dtype`.
GESSO_API int gesso_head_gated_rmsnorm(const float* o, const float* w, float eps, const void* gate, int gate_stride,
                                       void* out, int dtype, int n_rows, int n_heads, int Dv, int gate_act,
                                       cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_heads <= 0 || Dv <= 0 || gate_stride < n_heads * Dv) return GESSO_ERR_BAD_SIZE;
    const long long blocks = ((long long)n_rows * n_heads + 3) / 4;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    if (dtype == GESSO_F32)
        launch_pdl(head_gated_rmsnorm_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, stream, o, w, eps,
                   (const float*)gate, gate_stride, (float*)out, (long long)n_rows, n_heads, Dv, gate_act);
    else if (dtype == GESSO_BF16)
        launch_pdl(head_gated_rmsnorm_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, stream, o, w, eps,
                   (const bf16*)gate, gate_stride, (bf16*)out, (long long)n_rows, n_heads, Dv, gate_act);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}
