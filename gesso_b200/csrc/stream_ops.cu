// Small operations on the residual stream between layers.
//
// concat_cast:     out[r] = [a[r]; b[r]] rounded to the run type (two float32 streams of H features side by side,
//                  the operand of a matrix product that mixes them).
// rows_add_vector: h[r, j] += v[j] for every row (float32).
#include "common.cuh"

template <typename TO>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, TO* __restrict__ out,
                                   long long n_rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * 2 * H) return;
    const long long r = idx / (2 * H);
    const int j = (int)(idx % (2 * H));
    out[idx] = from_f32<TO>(j < H ? a[r * H + j] : b[r * H + (j - H)]);
}

GESSO_API int gesso_concat_cast(const float* a, const float* b, void* out, int out_dtype, int n_rows, int H,
                                cudaStream_t stream) {
    if (n_rows <= 0 || H <= 0) return 0;
    const long long total = (long long)n_rows * 2 * H;
    const long long blocks = (total + 255) / 256;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    if (out_dtype == GESSO_F32)
        launch_pdl(concat_cast_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, a, b, (float*)out,
                   (long long)n_rows, H);
    else if (out_dtype == GESSO_BF16)
        launch_pdl(concat_cast_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, stream, a, b, (bf16*)out,
                   (long long)n_rows, H);
    else
        return GESSO_ERR_BAD_DTYPE;
    return launch_status();
}

__global__ void rows_add_vector_kernel(float* __restrict__ h, const float* __restrict__ v, long long n_rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * H) return;
    h[idx] += v[idx % H];
}

GESSO_API int gesso_rows_add_vector(float* h, const float* v, int n_rows, int H, cudaStream_t stream) {
    if (n_rows <= 0 || H <= 0) return 0;
    const long long total = (long long)n_rows * H;
    const long long blocks = (total + 255) / 256;
    if (blocks > 2147483647LL) return GESSO_ERR_BAD_SIZE;
    launch_pdl(rows_add_vector_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, h, v, (long long)n_rows, H);
    return launch_status();
}
