// RMS norm in groups, with the residual add folded in.
//
// A row of H features is cut into G equal consecutive groups; a group is divided by its own
// sqrt(mean(group^2) + eps), and the whole row is then multiplied by a weight vector:
//     N(x; w)[j] = x[j] / sqrt(mean_{k in group(j)} x[k]^2 + eps) * w[j]
// A layer that norms a sublayer's output before adding it ("post" norm) and norms the sum again for the
// next sublayer ("pre" norm) does both in this one pass over the float32 residual stream:
//     v   = h + N(delta + bias; w_post)      (or delta + bias itself without a post norm)
//     h   = v                                (not with a row list: only the listed rows are computed, h stays)
//     out = N(v; w_pre)                      (rounded to the run type; no output without a pre norm)
// Everything is float32 inside.  One warp per (row, group): the sums of squares are added in lane order and
// by one butterfly, so a row's result does not depend on what else is in the step.  Groups of 128, 256, 512 or
// 1,024 features are held in registers (16-byte loads, every operand read once); other widths walk the group
// three times.
#include <math.h>

#include "common.cuh"

template <typename TD, typename TO>
__global__ void __launch_bounds__(128)
add_group_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ delta_bias,
                         const float* __restrict__ post_w, const float* __restrict__ pre_w, float eps,
                         TO* __restrict__ out, const int* __restrict__ rows, long long n_out, int H, int G) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long wi = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (wi >= n_out * G) return;                      // whole warps leave; no block barrier below
    const long long i = wi / G;
    const int g = (int)(wi % G), gw = H / G, j0 = g * gw;
    const long long r = rows ? rows[i] : i;
    float* hr = h + r * H + j0;
    const TD* dr = delta ? delta + r * H + j0 : nullptr;
    const float* br = delta_bias ? delta_bias + j0 : nullptr;
    float post_den = 1.f;
    if (dr && post_w) {
        float ss = 0.f;
        for (int j = lane; j < gw; j += 32) {
            const float d = to_f32(dr[j]) + (br ? br[j] : 0.f);
            ss = fmaf(d, d, ss);
        }
        post_den = sqrtf(warp_sum(ss) / (float)gw + eps);
    }
    auto value = [&](int j) -> float {
        float v = hr[j];
        if (dr) {
            const float d = to_f32(dr[j]) + (br ? br[j] : 0.f);
            v += post_w ? (d / post_den) * post_w[j0 + j] : d;
        }
        return v;
    };
    float ss = 0.f;
    if (dr && !rows) {
        for (int j = lane; j < gw; j += 32) {
            const float v = value(j);
            hr[j] = v;
            ss = fmaf(v, v, ss);
        }
        dr = nullptr;                                 // h holds the sum now
    } else if (pre_w) {
        for (int j = lane; j < gw; j += 32) {
            const float v = value(j);
            ss = fmaf(v, v, ss);
        }
    }
    if (!pre_w) return;
    const float den = sqrtf(warp_sum(ss) / (float)gw + eps);
    TO* orow = out + i * H + j0;
    for (int j = lane; j < gw; j += 32) orow[j] = from_f32<TO>((value(j) / den) * pre_w[j0 + j]);
}

__device__ __forceinline__ void load_vec4(const float* p, float (&x)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
__device__ __forceinline__ void load_vec4(const bf16* p, float (&x)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
    x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
}
__device__ __forceinline__ void store_vec4(float* p, const float (&x)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
}
__device__ __forceinline__ void store_vec4(bf16* p, const float (&x)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
    uint2 v;
    v.x = *reinterpret_cast<unsigned*>(&a);
    v.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = v;
}

// The same for groups of NV * 128 features: lane l holds features 4 (32 c + l) .. + 3 of chunk c = 0 .. NV - 1.
template <typename TD, typename TO, int NV>
__global__ void __launch_bounds__(128)
add_group_rmsnorm_reg_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ delta_bias,
                             const float* __restrict__ post_w, const float* __restrict__ pre_w, float eps,
                             TO* __restrict__ out, const int* __restrict__ rows, long long n_out, int H, int G) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long wi = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (wi >= n_out * G) return;
    const long long i = wi / G;
    constexpr int gw = NV * 128;
    const int j0 = (int)(wi % G) * gw;
    const long long r = rows ? rows[i] : i;
    float* hr = h + r * H + j0;
    float x[NV][4];
    if (delta) {
        const TD* dr = delta + r * H + j0;
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < NV; ++c) {
            const int j = 4 * (32 * c + lane);
            load_vec4(dr + j, x[c]);
            if (delta_bias) {
                float b[4];
                load_vec4(delta_bias + j0 + j, b);
#pragma unroll
                for (int k = 0; k < 4; ++k) x[c][k] += b[k];
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) ss = fmaf(x[c][k], x[c][k], ss);
        }
        if (post_w) {
            const float post_den = sqrtf(warp_sum(ss) / (float)gw + eps);
#pragma unroll
            for (int c = 0; c < NV; ++c) {
                float w[4];
                load_vec4(post_w + j0 + 4 * (32 * c + lane), w);
#pragma unroll
                for (int k = 0; k < 4; ++k) x[c][k] = (x[c][k] / post_den) * w[k];
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
        const int j = 4 * (32 * c + lane);
        float v[4];
        load_vec4(hr + j, v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            x[c][k] = delta ? v[k] + x[c][k] : v[k];
            ss = fmaf(x[c][k], x[c][k], ss);
        }
        if (delta && !rows) store_vec4(hr + j, x[c]);
    }
    if (!pre_w) return;
    const float den = sqrtf(warp_sum(ss) / (float)gw + eps);
    TO* orow = out + i * H + j0;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
        const int j = 4 * (32 * c + lane);
        float w[4], y[4];
        load_vec4(pre_w + j0 + j, w);
#pragma unroll
        for (int k = 0; k < 4; ++k) y[k] = (x[c][k] / den) * w[k];
        store_vec4(orow + j, y);
    }
}

// h: float32 [N, H], updated in place unless `rows` is given.  delta: [N, H] of delta_dtype, or null; delta_bias
// [H] float32 or null (added to delta before its norm).  post_w / pre_w [H] float32, null: that norm is absent.
// out: [n_out, H] of out_dtype (unused without a pre norm).  H must be a multiple of `groups`.
GESSO_API int gesso_add_group_rmsnorm(float* h, const void* delta, int delta_dtype, const float* delta_bias,
                                      const float* post_w, const float* pre_w, float eps, int groups, void* out,
                                      int out_dtype, const int* rows, int n_out, int H, cudaStream_t stream) {
    if (n_out <= 0 || H <= 0) return 0;
    if (groups <= 0 || H % groups != 0) return GESSO_ERR_BAD_SIZE;
    if (!delta && !pre_w) return 0;
    const long long warps = (long long)n_out * groups;
    const long long blocks = (warps + 3) / 4;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    // groups held in registers: whole 16-byte pieces per lane, and every pointer on a 16-byte boundary
    const int gw = H / groups;
    const bool aligned = ((uintptr_t)h % 16) == 0 && ((uintptr_t)delta % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
                         ((uintptr_t)delta_bias % 16) == 0 && ((uintptr_t)post_w % 16) == 0 && ((uintptr_t)pre_w % 16) == 0;
    const int nv = (aligned && gw % 128 == 0) ? gw / 128 : 0;
#define ARGS dim3((unsigned)blocks), dim3(128), 0, stream, h, (const TD*)delta, delta_bias, post_w, pre_w, eps, (TO*)out, \
             rows, (long long)n_out, H, groups
#define GO(TD_, TO_)                                                                                            \
    do {                                                                                                        \
        typedef TD_ TD;                                                                                         \
        typedef TO_ TO;                                                                                         \
        if (nv == 1) launch_pdl(add_group_rmsnorm_reg_kernel<TD, TO, 1>, ARGS);                                 \
        else if (nv == 2) launch_pdl(add_group_rmsnorm_reg_kernel<TD, TO, 2>, ARGS);                            \
        else if (nv == 4) launch_pdl(add_group_rmsnorm_reg_kernel<TD, TO, 4>, ARGS);                            \
        else if (nv == 8) launch_pdl(add_group_rmsnorm_reg_kernel<TD, TO, 8>, ARGS);                            \
        else launch_pdl(add_group_rmsnorm_kernel<TD, TO>, ARGS);                                                \
    } while (0)
    const bool d16 = delta && delta_dtype == GESSO_BF16;
    if (delta && delta_dtype != GESSO_BF16 && delta_dtype != GESSO_F32) return GESSO_ERR_BAD_DTYPE;
    if (out_dtype == GESSO_BF16) {
        if (d16) GO(bf16, bf16); else GO(float, bf16);
    } else if (out_dtype == GESSO_F32) {
        if (d16) GO(bf16, float); else GO(float, float);
    } else {
        return GESSO_ERR_BAD_DTYPE;
    }
#undef GO
#undef ARGS
    return launch_status();
}
