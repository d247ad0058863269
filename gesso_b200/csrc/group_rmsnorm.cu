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
// by one butterfly, so a row's result does not depend on what else is in the step.
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
#define GO(TD, TO)                                                                                              \
    launch_pdl(add_group_rmsnorm_kernel<TD, TO>, dim3((unsigned)blocks), dim3(128), 0, stream, h,               \
               (const TD*)delta, delta_bias, post_w, pre_w, eps, (TO*)out, rows, (long long)n_out, H, groups)
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
    return launch_status();
}
