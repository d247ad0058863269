// Activations between the two matrix products of a feed-forward, evaluated in float32.
//
// gelu_erf:     out = 0.5 x (1 + erf(x / sqrt 2)), elementwise on [N, F].
// glu_clamped:  a gated unit with clamped inputs on the fused gate/up projection [N, 2F]:
//                   g = min(gate, limit),  u = clamp(up, -limit, limit),
//                   out = g * sigmoid(alpha * g) * (u + 1)                  [N, F]
//               Plain layout: columns [0, F) are the gate projection, [F, 2F) the up projection.  Packed layout:
//               every group of 16 columns holds 8 gate columns and then the matching 8 up columns.
// xielu:        see below.
#include <math.h>

#include "common.cuh"

template <typename T>
__global__ void gelu_erf_kernel(const T* __restrict__ x, T* __restrict__ out, long long n) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = to_f32(x[i]);
    out[i] = from_f32<T>(0.5f * v * (1.f + erff(v * 0.70710678118654752f)));
}

GESSO_API int gesso_gelu_erf(const void* x, void* out, int dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    if (dtype == GESSO_F32)
        launch_pdl(gelu_erf_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)x, (float*)out, n);
    else if (dtype == GESSO_BF16)
        launch_pdl(gelu_erf_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)x, (bf16*)out, n);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}

template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ out, long long n_rows, int F, int packed,
                                   float limit, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * F) return;
    const long long r = i / F;
    const int f = (int)(i % F);
    const T* row = gu + r * 2 * F;
    const int gi = packed ? 16 * (f >> 3) + (f & 7) : f;
    const int ui = packed ? gi + 8 : F + f;
    const float g = fminf(to_f32(row[gi]), limit);
    const float u = fminf(fmaxf(to_f32(row[ui]), -limit), limit);
    out[i] = from_f32<T>((g / (1.f + expf(-alpha * g))) * (u + 1.f));
}

GESSO_API int gesso_glu_clamped(const void* gu, void* out, int dtype, int n_rows, int F, int packed, float limit,
                                float alpha, cudaStream_t stream) {
    if (n_rows <= 0 || F <= 0) return 0;
    if (packed && F % 8 != 0) return GESSO_ERR_BAD_SIZE;
    const long long total = (long long)n_rows * F, blocks = (total + 255) / 256;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    if (dtype == GESSO_F32)
        launch_pdl(glu_clamped_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)gu, (float*)out,
                   (long long)n_rows, F, packed, limit, alpha);
    else if (dtype == GESSO_BF16)
        launch_pdl(glu_clamped_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out,
                   (long long)n_rows, F, packed, limit, alpha);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}

// xielu: a piecewise activation with two learned numbers p and q (read from device memory, so that a step never
// waits for the host):
//     z > 0:   softplus(p) z^2 + z / 2
//     z <= 0:  (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
__device__ __forceinline__ float softplus_f(float a) { return fmaxf(a, 0.f) + log1pf(expf(-fabsf(a))); }

template <typename T>
__global__ void xielu_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, const float* __restrict__ pq) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float sp = softplus_f(pq[0]), sq = 0.5f + softplus_f(pq[1]);
    const float z = to_f32(x[i]);
    const float y = z > 0.f ? fmaf(sp * z, z, 0.5f * z) : fmaf(sq, expm1f(z) - z, 0.5f * z);
    out[i] = from_f32<T>(y);
}

GESSO_API int gesso_xielu(const void* x, void* out, int dtype, long long n, const float* pq, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    if (dtype == GESSO_F32)
        launch_pdl(xielu_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)x, (float*)out, n, pq);
    else if (dtype == GESSO_BF16)
        launch_pdl(xielu_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)x, (bf16*)out, n, pq);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}
