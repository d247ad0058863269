// Gated linear attention: linear attention whose decay is computed from the input, one number per key channel
// and token, as a recurrence over a per-request state.
//
// Per head, with q_t, k_t, a_t (D features) and v_t (Dv features):
//     a_t = exp(log_sigmoid(z_t) / tau)              (z_t: the decay's logits, float32; 0 < a_t < 1)
//     S_t = diag(a_t) S_{t-1} + k_t v_t^T            (S: [D, Dv] float32, zero at the start of a request)
//     o_t = q_scale * S_t^T q_t
// The recurrence runs in float32 whatever the run type: the logits, the decay, the state, the outer product and
// the read-out.  q, k and v arrive as rows of a fused matrix product (q columns, then k, then v; further columns
// may follow) in the run type; the logits as a float32 matrix [tokens, H * D] with an optional bias [H * D].
//
// A first kernel turns the logits into decays.  The walk kernel then serves three uses:
//   * WALK: a block owns (segment, head, a group of value columns) and walks the segment's tokens in order from
//     the request's state, which it leaves as the last token makes it (steps of single tokens, short portions);
//   * long portions run by the step's 64-token tiles side by side, in three launches: SUMS walks every tile from
//     a zero state without reading out and keeps what the tile adds (its own sum of decayed k v^T, and the
//     product of its decays per key channel); a scan walks each request's tiles in order, S <- prod(a) S + sum,
//     and hands every tile the state it starts from; OUTS walks every tile again from that state and reads out.
//     A tile's tokens are walked twice (1.5 times the arithmetic of one walk), but all tiles at once.
// The columns of S are independent: a thread owns two value columns and 16 key features of them (32 state
// values in registers; L lanes side by side cover a column's D features, four features a lane in turn, zeros
// behind D), the read-out is summed over those lanes by shuffles.  A tile of tokens' q, k (run type), a and v (float32) is staged through shared
// memory at a time, by 16-byte loads where the sizes allow.
// The state is stored [slot][head][value column][feature], as the fixed-decay recurrence stores it.
// These kernels do not let their successor in before they end: each reads what kernels further back than its
// predecessor wrote (the decays, the tiles' sums), and with successors let in early the tiled form was seen to read
// such data before it was complete.
//
// head_gated_rmsnorm: y = (o / sqrt(mean_head(o^2) + eps)) * w * act(g) per head of a token (w has one head's
// width and is shared by the heads; act = sigmoid or silu), the norm in float32; g are columns of the fused
// projection.
#include <math.h>

#include "common.cuh"

#define GLA_THREADS 128
#define GLA_PER_LANE 16
#define GLA_CPT 2                // value columns of a thread
#define GLA_CHUNK 64             // tokens of a tile (the step's query tiles)

// log(sigmoid(z)) = -softplus(-z), without overflow on either side
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

__global__ void __launch_bounds__(256)
gla_decay_kernel(const float* __restrict__ z, const float* __restrict__ z_bias, float inv_tau, float* __restrict__ decay,
                 int HD) {
    pdl_wait();
    const int j = blockIdx.y * 256 + threadIdx.x;          // grid: (tokens, blocks of 256 key channels)
    if (j >= HD) return;
    const size_t i = (size_t)blockIdx.x * HD + j;
    float zz = z[i];
    if (z_bias) zz += z_bias[j];
    decay[i] = expf(log_sigmoid_f(zz) * inv_tau);
}

__device__ __forceinline__ void load4(const float* p, float (&x)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&x)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
    x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
}

enum { GLA_WALK = 0, GLA_SUMS = 1, GLA_OUTS = 2 };

template <typename T, int L, int MODE>
__global__ void __launch_bounds__(GLA_THREADS)
gla_kernel(const T* __restrict__ proj, int row_stride, const float* __restrict__ decay, float q_scale,
           float* __restrict__ state, long long slot_stride, const int* __restrict__ seg_start,
           const int* __restrict__ slots, const int* __restrict__ tile_seg, const int* __restrict__ tile_q0,
           float* __restrict__ ws, float* __restrict__ ws_decay, float* __restrict__ out, int H, int D, int Dv,
           int tile, int vec) {
    extern __shared__ __align__(16) unsigned char gla_smem[];
    constexpr int COLS = GLA_CPT * GLA_THREADS / L;   // value columns of a block
    constexpr int DP = L * GLA_PER_LANE;              // features of a head, padded to whole lanes (zeros behind D)
    pdl_wait();
    const int h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int cw = threadIdx.x / L, part = threadIdx.x % L;
    const int col = c0 + GLA_CPT * cw;                // this thread's columns col, col + 1
    // this lane's 16 features, four at a time: piece r = 0 .. 3 is features 4 (r L + part) .. + 3, so that the L
    // lanes of a column read consecutive 16 bytes of a staged row (no two of them on one bank)
    auto feat = [&](int i) { return 4 * ((i >> 2) * L + part) + (i & 3); };
    int t0, n;
    float* st;                                        // where the walk starts from (WALK, OUTS) and what it leaves (WALK, SUMS)
    if (MODE == GLA_WALK) {
        const int s = blockIdx.x;
        t0 = seg_start[s];
        n = seg_start[s + 1] - t0;
        st = state + (size_t)slots[s] * slot_stride + (size_t)h * Dv * D;
    } else {
        const int s = tile_seg[blockIdx.x], q0 = tile_q0[blockIdx.x];
        t0 = seg_start[s] + q0;
        n = min(GLA_CHUNK, seg_start[s + 1] - t0);
        st = ws + ((size_t)blockIdx.x * H + h) * Dv * D;
    }
    float S[GLA_CPT][GLA_PER_LANE];
#pragma unroll
    for (int c = 0; c < GLA_CPT; ++c)
#pragma unroll
        for (int i = 0; i < GLA_PER_LANE; ++i)
            S[c][i] = (MODE != GLA_SUMS && col + c < Dv && feat(i) < D) ? st[(size_t)(col + c) * D + feat(i)] : 0.f;
    // SUMS: the lanes of the block's first column, in the first group of columns, also keep the product of the decays
    const bool track = MODE == GLA_SUMS && blockIdx.z == 0 && cw == 0;
    float P[GLA_PER_LANE];
#pragma unroll
    for (int i = 0; i < GLA_PER_LANE; ++i) P[i] = 1.f;
    T* sq = reinterpret_cast<T*>(gla_smem);                       // [tile][DP]
    T* sk = sq + (size_t)tile * DP;                               // [tile][DP]
    float* sa = reinterpret_cast<float*>(sk + (size_t)tile * DP); // [tile][DP]
    float* sv = sa + (size_t)tile * DP;                           // [tile][COLS]
    const int qo = h * D, ko = H * D + h * D, vo = 2 * H * D + h * Dv;
    const size_t HD = (size_t)H * D;
    for (int base = 0; base < n; base += tile) {
        const int m = min(tile, n - base);
        __syncthreads();
        if (vec) {     // D is a multiple of 16 (no padding) and every row starts on a 16-byte boundary
            constexpr int PER = 16 / (int)sizeof(T);
            const int nq = D / PER, na = D / 4;
            for (int j = threadIdx.x; j < m * nq; j += GLA_THREADS) {
                const int i = j / nq, x = (j % nq) * PER;
                const T* row = proj + (size_t)(t0 + base + i) * row_stride;
                if (MODE != GLA_SUMS)
                    *reinterpret_cast<uint4*>(sq + (size_t)i * DP + x) = *reinterpret_cast<const uint4*>(row + qo + x);
                *reinterpret_cast<uint4*>(sk + (size_t)i * DP + x) = *reinterpret_cast<const uint4*>(row + ko + x);
            }
            for (int j = threadIdx.x; j < m * na; j += GLA_THREADS) {
                const int i = j / na, x = (j % na) * 4;
                *reinterpret_cast<float4*>(sa + (size_t)i * DP + x) =
                    *reinterpret_cast<const float4*>(decay + (size_t)(t0 + base + i) * HD + qo + x);
            }
        } else {
            for (int j = threadIdx.x; j < m * DP; j += GLA_THREADS) {
                const int d = j % DP;
                const size_t tok = (size_t)(t0 + base + j / DP);
                const T* row = proj + tok * row_stride;
                const bool on = d < D;
                sq[j] = on ? row[qo + d] : from_f32<T>(0.f);
                sk[j] = on ? row[ko + d] : from_f32<T>(0.f);
                sa[j] = on ? decay[tok * HD + qo + d] : 0.f;
            }
        }
        for (int j = threadIdx.x; j < m * COLS; j += GLA_THREADS) {
            const int c = c0 + j % COLS;
            sv[j] = c < Dv ? to_f32(proj[(size_t)(t0 + base + j / COLS) * row_stride + vo + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll 2
        for (int i = 0; i < m; ++i) {
            const float2 v = *reinterpret_cast<const float2*>(sv + i * COLS + GLA_CPT * cw);
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int r = 0; r < GLA_PER_LANE / 4; ++r) {
                float kk[4], qq[4], aa[4];
                load4(sa + (size_t)i * DP + 4 * (r * L + part), aa);
                load4(sk + (size_t)i * DP + 4 * (r * L + part), kk);
                if (MODE != GLA_SUMS) load4(sq + (size_t)i * DP + 4 * (r * L + part), qq);
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    S[0][4 * r + x] = fmaf(aa[x], S[0][4 * r + x], kk[x] * v.x);
                    S[1][4 * r + x] = fmaf(aa[x], S[1][4 * r + x], kk[x] * v.y);
                    if (MODE != GLA_SUMS) {
                        o0 = fmaf(S[0][4 * r + x], qq[x], o0);
                        o1 = fmaf(S[1][4 * r + x], qq[x], o1);
                    }
                    if (MODE == GLA_SUMS && track) P[4 * r + x] *= aa[x];
                }
            }
            if (MODE != GLA_SUMS) {
#pragma unroll
                for (int x = L / 2; x > 0; x >>= 1) {
                    o0 += __shfl_xor_sync(0xffffffffu, o0, x);
                    o1 += __shfl_xor_sync(0xffffffffu, o1, x);
                }
                if (part == 0) {
                    float* orow = out + (size_t)(t0 + base + i) * H * Dv + (size_t)h * Dv + col;
                    if (col < Dv) orow[0] = q_scale * o0;
                    if (col + 1 < Dv) orow[1] = q_scale * o1;
                }
            }
        }
    }
    if (MODE != GLA_OUTS) {
#pragma unroll
        for (int c = 0; c < GLA_CPT; ++c)
#pragma unroll
            for (int i = 0; i < GLA_PER_LANE; ++i)
                if (col + c < Dv && feat(i) < D) st[(size_t)(col + c) * D + feat(i)] = S[c][i];
    }
    if (MODE == GLA_SUMS && track) {
#pragma unroll
        for (int i = 0; i < GLA_PER_LANE; ++i)
            if (feat(i) < D) ws_decay[((size_t)blockIdx.x * H + h) * D + feat(i)] = P[i];
    }
}

// Walks each request's tiles in order: a tile's slot of `ws` holds what the tile adds and gets the state the tile
// starts from; the request's state ends as its last tile leaves it.
__global__ void __launch_bounds__(256)
gla_chunk_scan_kernel(float* __restrict__ state, long long slot_stride, const int* __restrict__ seg_start,
                      const int* __restrict__ slots, const int* __restrict__ tile_seg,
                      const int* __restrict__ tile_q0, int n_tiles, float* __restrict__ ws,
                      const float* __restrict__ ws_decay, int H, int D, int Dv) {
    __shared__ int s_first;
    pdl_wait();
    const int seg = blockIdx.x, h = blockIdx.y;
    if (threadIdx.x == 0) {
        int f = -1;
        for (int t = 0; t < n_tiles; ++t)
            if (tile_seg[t] == seg && tile_q0[t] == 0) { f = t; break; }
        s_first = f;
    }
    __syncthreads();
    const int first = s_first;
    const int e = blockIdx.z * 256 + threadIdx.x;
    if (first < 0 || e >= D * Dv) return;
    const int n = seg_start[seg + 1] - seg_start[seg];
    const int d = e % D;
    float* st = state + (size_t)slots[seg] * slot_stride + (size_t)h * Dv * D + e;
    float S = *st;
    const int nt = (n + GLA_CHUNK - 1) / GLA_CHUNK;
    const size_t tile_stride = (size_t)H * Dv * D, decay_stride = (size_t)H * D;
    float* u = ws + ((size_t)first * H + h) * Dv * D + e;
    const float* a = ws_decay + ((size_t)first * H + h) * D + d;
    // four tiles' sums and decays are read ahead of the chain of dependent products
    for (int c = 0; c < nt; c += 4) {
        float U[4], A[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (c + k < nt) {
                U[k] = u[(size_t)(c + k) * tile_stride];
                A[k] = a[(size_t)(c + k) * decay_stride];
            }
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (c + k < nt) {
                u[(size_t)(c + k) * tile_stride] = S;
                S = fmaf(A[k], S, U[k]);
            }
    }
    *st = S;
}

// proj [n_tokens, row_stride] of `dtype`: q at column 0 (H * D), k at H * D, v at 2 * H * D (H * Dv).  z [n_tokens, H * D]
// float32 (+ z_bias [H * D] or null): the decay's logits; decay: as large as z, receives the decays.  state: this
// layer's view, slot s at state + s * slot_stride floats, [H][Dv][D].  out [n_tokens, H * Dv] float32.
// With n_tiles > 0 the step runs by its 64-token tiles (tile_seg / tile_q0: a tile's segment and first token in
// it; ws: n_tiles * H * Dv * D floats, ws_decay: n_tiles * H * D floats); otherwise token after token.
GESSO_API int gesso_gla(const void* proj, int dtype, int row_stride, const float* z, const float* z_bias, float* decay, float tau,
                        float q_scale, float* state, long long slot_stride, const int* seg_start, const int* slots,
                        const int* tile_seg, const int* tile_q0, int n_tiles, float* ws, float* ws_decay, float* out,
                        int n_tokens, int n_segs, int H, int D, int Dv, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segs <= 0) return 0;
    if (H <= 0 || D <= 0 || Dv <= 0 || D > 32 * GLA_PER_LANE || H > 65535 || row_stride < 2 * H * D + H * Dv || !(tau > 0.f))
        return GESSO_ERR_BAD_SIZE;
    if (!decay) return GESSO_ERR_BAD_SIZE;
    if (n_tiles > 0 && (!tile_seg || !tile_q0 || !ws || !ws_decay)) return GESSO_ERR_BAD_SIZE;
    int L = 1;
    while (L * GLA_PER_LANE < D) L <<= 1;
    const int cols = GLA_CPT * GLA_THREADS / L;
    const int col_blocks = (Dv + cols - 1) / cols;
    if (col_blocks > 65535) return GESSO_ERR_BAD_SIZE;
    const int dp = L * GLA_PER_LANE;
    const size_t esz = dtype == GESSO_F32 ? 4 : 2;
    const size_t per_token = (size_t)dp * (2 * esz + 4) + (size_t)cols * 4;
    int tile = 32;
    while (tile > 4 && tile * per_token > 24 * 1024) tile >>= 1;
    const size_t smem = tile * per_token;
    // 16-byte loads: no padding behind D, and every row of q, k and the decays starts on a 16-byte boundary
    const int vec = (D % 16 == 0 && row_stride % 8 == 0 && ((uintptr_t)proj % 16) == 0 && ((uintptr_t)decay % 16) == 0) ? 1 : 0;
    if ((H * D + 255) / 256 > 65535) return GESSO_ERR_BAD_SIZE;
    launch_pdl(gla_decay_kernel, dim3((unsigned)n_tokens, (unsigned)((H * D + 255) / 256)), dim3(256), 0, stream, z, z_bias,
               1.f / tau, decay, H * D);
#define GO(T, LL, MODE, GRID)                                                                                       \
    launch_pdl(gla_kernel<T, LL, MODE>, GRID, dim3(GLA_THREADS), smem, stream, (const T*)proj, row_stride,          \
               (const float*)decay, q_scale, state, slot_stride, seg_start, slots, tile_seg, tile_q0, ws, ws_decay, out, \
               H, D, Dv, tile, vec)
#define BY_L(T, MODE, GRID)                                                                                         \
    switch (L) {                                                                                                    \
        case 1: GO(T, 1, MODE, GRID); break;                                                                        \
        case 2: GO(T, 2, MODE, GRID); break;                                                                        \
        case 4: GO(T, 4, MODE, GRID); break;                                                                        \
        case 8: GO(T, 8, MODE, GRID); break;                                                                        \
        case 16: GO(T, 16, MODE, GRID); break;                                                                      \
        default: GO(T, 32, MODE, GRID); break;                                                                      \
    }
#define RUN(T)                                                                                                      \
    if (n_tiles > 0) {                                                                                              \
        const dim3 tiles(n_tiles, H, col_blocks), scan(n_segs, H, (D * Dv + 255) / 256);                            \
        BY_L(T, GLA_SUMS, tiles)                                                                                    \
        launch_pdl(gla_chunk_scan_kernel, scan, dim3(256), 0, stream, state, slot_stride, seg_start, slots,         \
                   tile_seg, tile_q0, n_tiles, ws, (const float*)ws_decay, H, D, Dv);                               \
        BY_L(T, GLA_OUTS, tiles)                                                                                    \
    } else {                                                                                                        \
        const dim3 walk(n_segs, H, col_blocks);                                                                     \
        BY_L(T, GLA_WALK, walk)                                                                                     \
    }
    if (dtype == GESSO_F32) { RUN(float) }
    else if (dtype == GESSO_BF16) { RUN(bf16) }
    else return GESSO_ERR_BAD_DTYPE;
#undef RUN
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
