// Two elementwise kernels of the layer shapes that are not pre-norm (a norm behind a part, a norm on a part's output,
// no norm at all): adding a part's output into the float32 residual stream, and converting rows between float32 and
// the compute dtype.  The pre-norm shape needs neither: its additions ride in the norm kernels.
#include "common.cuh"

namespace {
template <typename TD>
__global__ void add_into_f32_kernel(float* __restrict__ residual, const TD* __restrict__ delta, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) residual[i] += to_f32<TD>(delta[i]);
}
template <typename TS, typename TD>
__global__ void convert_rows_kernel(const TS* __restrict__ src, TD* __restrict__ dst, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = from_f32<TD>(to_f32<TS>(src[i]));
}
}  // namespace

// residual[i] += delta[i], i < n; delta_dtype: EG_F32 or EG_BF16
EG_API int eg_add_into_f32(cudaStream_t stream, float* residual, const void* delta, int delta_dtype, long long n) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (delta_dtype == EG_BF16) add_into_f32_kernel<bf16><<<blocks, 256, 0, stream>>>(residual, (const bf16*)delta, n);
    else add_into_f32_kernel<float><<<blocks, 256, 0, stream>>>(residual, (const float*)delta, n);
    return eg_launch_status();
}

// dst[i] = src[i] converted, i < n; dtypes: EG_F32 or EG_BF16
EG_API int eg_convert_rows(cudaStream_t stream, const void* src, int src_dtype, void* dst, int dst_dtype, long long n) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (src_dtype == EG_F32 && dst_dtype == EG_BF16) convert_rows_kernel<float, bf16><<<blocks, 256, 0, stream>>>((const float*)src, (bf16*)dst, n);
    else if (src_dtype == EG_BF16 && dst_dtype == EG_F32) convert_rows_kernel<bf16, float><<<blocks, 256, 0, stream>>>((const bf16*)src, (float*)dst, n);
    else if (src_dtype == EG_F32) convert_rows_kernel<float, float><<<blocks, 256, 0, stream>>>((const float*)src, (float*)dst, n);
    else convert_rows_kernel<bf16, bf16><<<blocks, 256, 0, stream>>>((const bf16*)src, (bf16*)dst, n);
    return eg_launch_status();
}

namespace {
// residual[t, j] = (residual[t, j] + first[t, j]) + offset[j]
__global__ void stream_add_kernel(float* __restrict__ residual, const float* __restrict__ first, const float* __restrict__ offset, long long n, int hidden) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = residual[i];
    if (first) v += first[i];
    residual[i] = v + offset[i % hidden];
}
__global__ void softcap_kernel(float* __restrict__ x, long long n, float cap, float inv_cap) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] * inv_cap);
}
}  // namespace

// What a repeated run of layers adds to the stream before a pass: residual [tokens, hidden] += first (the stream as the
// embedding left it; may be null) and += offset [hidden] (a learned vector of the pass), in that order, in float32.
EG_API int eg_stream_add(cudaStream_t stream, float* residual, const float* first, const float* offset, int tokens, int hidden) {
    const long long n = (long long)tokens * hidden;
    if (n <= 0) return 0;
    stream_add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(residual, first, offset, n, hidden);
    return eg_launch_status();
}

// x[i] = cap * tanh(x[i] / cap), i < n (float32, accurate tanh)
EG_API int eg_softcap(cudaStream_t stream, float* x, long long n, float cap) {
    if (n <= 0) return 0;
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, n, cap, 1.0f / cap);
    return eg_launch_status();
}

namespace {
__global__ void add_bias_rows_kernel(float* __restrict__ x, long long ld, const float* __restrict__ bias, int rows, int cols) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols) return;
    const int c = (int)(i % cols);
    x[(size_t)(i / cols) * ld + c] += bias[c];
}
template <typename TD>
__global__ void convert_columns_kernel(const float* __restrict__ src, long long lds, TD* __restrict__ dst, long long ldd, int rows, int cols, int padded) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * padded) return;
    const int c = (int)(i % padded);
    const size_t r = (size_t)(i / padded);
    dst[r * ldd + c] = from_f32<TD>(c < cols ? src[r * lds + c] : 0.f);
}
}  // namespace

// x [rows, ld] float32: x[r, c] += bias[c], c < cols (the bias of a product whose library form writes float32 without one)
EG_API int eg_add_bias_rows(cudaStream_t stream, float* x, long long ld, const float* bias, int rows, int cols) {
    const long long n = (long long)rows * cols;
    if (n <= 0) return 0;
    add_bias_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, ld, bias, rows, cols);
    return eg_launch_status();
}

// A block of columns of float32 rows as rows of their own: dst[r, c] = src[r, c] for c < cols and 0 for cols <= c < padded
// (dst_dtype EG_F32 or EG_BF16; rows lds and ldd elements apart).  For a product that reads a few columns of another's output.
EG_API int eg_convert_columns(cudaStream_t stream, const float* src, long long lds, void* dst, int dst_dtype, long long ldd, int rows, int cols, int padded) {
    const long long n = (long long)rows * padded;
    if (n <= 0) return 0;
    if (padded < cols) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dst_dtype == EG_BF16) convert_columns_kernel<bf16><<<blocks, 256, 0, stream>>>(src, lds, (bf16*)dst, ldd, rows, cols, padded);
    else convert_columns_kernel<float><<<blocks, 256, 0, stream>>>(src, lds, (float*)dst, ldd, rows, cols, padded);
    return eg_launch_status();
}
