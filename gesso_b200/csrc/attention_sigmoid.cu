// Paged causal attention whose weights are sigmoids of the scores (no softmax, nothing normalized over the keys),
// with a learned bias by distance and a temperature on the queries that grows with the position.
//
// For the query of head h at position p and the key at position u <= p of its kv head (h / (nh / nkv)):
//     w(p, u) = sigmoid( (q . k) * scale * temp(p) + bias[h][min(p - u, n_dist - 1)] )
//     out     = ( sum_u w(p, u) v_u ) * sigmoid(gate[token, h])          (the gate: one number per head, optional)
//     temp(p) = 1 + coef * ln( floor((p + 1) / every) + 1 )              (every <= 0: 1)
// `bias` is a float32 table [nh][n_dist] by distance; every distance from n_dist - 1 on shares the last column.
// Whatever a design adds to the score per head and distance (a bucketed table, a constant per head) is put into
// that table by the caller.  With a window, a query reads only the last `window` positions.
//
// This file holds the FP32-arithmetic kernel (CUDA cores): the kernel of the true 32-bit path, and of sizes the
// tensor-core kernels do not take.  One warp per (token, query head); the lanes stride over the keys, each with a
// private sum over its keys, and the 32 sums are added by one butterfly at the end: what a position's result is
// does not depend on which pages hold the keys or on what else is in the step.  Scores, weights and sums are
// float32; queries and results may be float32 over bfloat16 pages.
#include <math.h>

#include "common.cuh"

__device__ __forceinline__ float query_temperature(int pos, float coef, int every) {
    return every > 0 ? 1.f + coef * logf((float)((pos + 1) / every + 1)) : 1.f;
}

template <typename TQ, typename T, int HD_PAD>
__global__ void __launch_bounds__(128)
sigmoid_attention_generic_kernel(const TQ* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                 const int* __restrict__ block_table, int max_pages, int page_size,
                                 const int* __restrict__ positions, const int* __restrict__ seg_of_token,
                                 TQ* __restrict__ out, int n_tokens, int nh, int nkv, int hd, int vd, float scale,
                                 const float* __restrict__ dist_bias, int n_dist, float temp_coef, int temp_every,
                                 const T* __restrict__ gate, int gate_stride, int window) {
    __shared__ float q_s[4][HD_PAD];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long wi = (long long)blockIdx.x * 4 + wid;
    if (wi >= (long long)n_tokens * nh) return;   // whole warps leave together; no block barrier below
    const int t = (int)(wi / nh), h = (int)(wi % nh);
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int* bt = block_table + (size_t)seg_of_token[t] * max_pages;
    const TQ* qrow = q + ((size_t)t * nh + h) * hd;
    const float qscale = scale * query_temperature(pos, temp_coef, temp_every);
    const float* bias = dist_bias ? dist_bias + (size_t)h * n_dist : nullptr;
    for (int j = lane; j < HD_PAD; j += 32) q_s[wid][j] = j < hd ? to_f32(qrow[j]) : 0.f;
    __syncwarp();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float acc[HD_PAD];
#pragma unroll
    for (int j = 0; j < HD_PAD; ++j) acc[j] = 0.f;
    for (int u = lo + lane; u <= pos; u += 32) {
        const int page = bt[u / page_size];
        if (page < 0) continue;
        const T* kr = k_pages + (((size_t)page * nkv + kvh) * page_size + (u % page_size)) * hd;
        // V is stored [feature][slot] inside a page
        const T* vr = v_pages + ((size_t)page * nkv + kvh) * vd * page_size + (u % page_size);
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < HD_PAD; ++j)
            if (j < hd) dot += q_s[wid][j] * to_f32(kr[j]);
        float sc = dot * qscale;
        if (bias) sc += bias[min(pos - u, n_dist - 1)];
        const float p = 1.f / (1.f + expf(-sc));
#pragma unroll
        for (int j = 0; j < HD_PAD; ++j)
            if (j < vd) acc[j] += p * to_f32(vr[(size_t)j * page_size]);
    }
    TQ* orow = out + ((size_t)t * nh + h) * vd;
    const float g = gate ? 1.f / (1.f + expf(-to_f32(gate[(size_t)t * gate_stride + h]))) : 1.f;
#pragma unroll
    for (int j = 0; j < HD_PAD; ++j) {
        const float a = warp_sum(acc[j]);
        if (j < vd && (j & 31) == lane) orow[j] = from_f32<TQ>(a * g);
    }
}

template <typename TQ, typename T>
static int launch_sigmoid_generic(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                  int max_pages, int page_size, const int* positions, const int* seg_of_token,
                                  void* out, int n_tokens, int nh, int nkv, int hd, int vd, float scale,
                                  const float* dist_bias, int n_dist, float temp_coef, int temp_every,
                                  const void* gate, int gate_stride, int window, cudaStream_t stream) {
    const long long total = (long long)n_tokens * nh;
    const long long blocks = (total + 3) / 4;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
#define GO(PAD)                                                                                               \
    sigmoid_attention_generic_kernel<TQ, T, PAD><<<(unsigned)blocks, 128, 0, stream>>>(                        \
        (const TQ*)q, (const T*)k_pages, (const T*)v_pages, block_table, max_pages, page_size, positions,     \
        seg_of_token, (TQ*)out, n_tokens, nh, nkv, hd, vd, scale, dist_bias, n_dist, temp_coef, temp_every,   \
        (const T*)gate, gate_stride, window)
    const int wide = hd > vd ? hd : vd;
    if (wide <= 32) GO(32);
    else if (wide <= 64) GO(64);
    else if (wide <= 128) GO(128);
    else if (wide <= 256) GO(256);
    else return GESSO_ERR_BAD_SIZE;
#undef GO
    return launch_status();
}

// `q_dtype`: the type of q and of the result; `dtype`: the type of the pages and of the gate.  A float32 q may read
// bfloat16 pages; otherwise the two are equal.  gate: element [t * gate_stride + h] is head h's gate of token t
// (columns of a fused projection, say), or null.  dist_bias: [nh][n_dist] float32 or null.
GESSO_API int gesso_sigmoid_attention_generic(const void* q, const void* k_pages, const void* v_pages, int dtype,
                                              const int* block_table, int max_pages, int page_size,
                                              const int* positions, const int* seg_of_token, void* out, int n_tokens,
                                              int nh, int nkv, int hd, int vd, float scale, const float* dist_bias,
                                              int n_dist, float temp_coef, int temp_every, const void* gate,
                                              int gate_stride, int q_dtype, int window, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || vd <= 0 || page_size <= 0) return GESSO_ERR_BAD_SIZE;
    if ((dist_bias && n_dist < 1) || (gate && gate_stride < nh)) return GESSO_ERR_BAD_SIZE;
#define ARGS q, k_pages, v_pages, block_table, max_pages, page_size, positions, seg_of_token, out, n_tokens, nh, nkv, hd, \
             vd, scale, dist_bias, n_dist, temp_coef, temp_every, gate, gate_stride, window, stream
    if (dtype == GESSO_F32 && q_dtype == GESSO_F32) return launch_sigmoid_generic<float, float>(ARGS);
    if (dtype == GESSO_BF16 && q_dtype == GESSO_BF16) return launch_sigmoid_generic<bf16, bf16>(ARGS);
    if (dtype == GESSO_BF16 && q_dtype == GESSO_F32) return launch_sigmoid_generic<float, bf16>(ARGS);
#undef ARGS
    return GESSO_ERR_BAD_DTYPE;
}
