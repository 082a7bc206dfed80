// A per-layer token input: every token brings a small vector e of its own (a row of a table, by token id) that is gated
// by the stream, mapped to the model's width, normed and added:
//
//   g = gelu_tanh(G x) * e;   y = P g;   x <- x + w * y / sqrt(mean(y^2) + eps)        G [side, hidden], P [hidden, side]
//
// The two maps are products over all tokens of a step and run as such; this file has what stands between them:
//   eg_add_scaled_rows   takes in up to two branch outputs that are still to be added, each times a gain per channel
//                        (x <- x + s_a * d_a + s_b * d_b, float32, in place) and writes x in the precision the product reads:
//                        the end of a layer whose branches run side by side costs one pass over the stream
//   eg_token_side_gate   g = gelu_tanh(z) * e from the first product's float32 sums
//   eg_add_scaled        the add alone
#include "common.cuh"

namespace {
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TD> __device__ __forceinline__ float load_as_f32(const void* p, size_t i) { return to_f32<TD>(((const TD*)p)[i]); }
__device__ __forceinline__ float load_dyn(const void* p, int dtype, size_t i) { return dtype == EG_BF16 ? load_as_f32<bf16>(p, i) : load_as_f32<float>(p, i); }

// four values a thread; n and hidden are multiples of 4
template <typename TO>
__global__ void add_scaled_rows_kernel(float* __restrict__ stream, const void* __restrict__ delta_a, int dtype_a, const float* __restrict__ scale_a,
                                       const void* __restrict__ delta_b, int dtype_b, const float* __restrict__ scale_b, TO* __restrict__ rows, long long n,
                                       int hidden, int per) {
    const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * per;
    if (i0 >= n) return;
    const int j0 = (int)(i0 % hidden);
    float v[4];
    for (int e = 0; e < per; ++e) v[e] = stream[i0 + e];
    if (delta_a)
        for (int e = 0; e < per; ++e) v[e] = fmaf(scale_a ? scale_a[j0 + e] : 1.0f, load_dyn(delta_a, dtype_a, (size_t)(i0 + e)), v[e]);
    if (delta_b)
        for (int e = 0; e < per; ++e) v[e] = fmaf(scale_b ? scale_b[j0 + e] : 1.0f, load_dyn(delta_b, dtype_b, (size_t)(i0 + e)), v[e]);
    for (int e = 0; e < per; ++e) {
        if (delta_a || delta_b) stream[i0 + e] = v[e];
        rows[i0 + e] = from_f32<TO>(v[e]);
    }
}

template <typename TW>
__global__ void token_side_gate_kernel(const float* __restrict__ z, long long ldz, const int* __restrict__ token_ids, const TW* __restrict__ table, int vocab,
                                       TW* __restrict__ g, int tokens, int side, int* status) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * side) return;
    const int t = (int)(i / side), o = (int)(i % side);
    int id = token_ids[t];
    if (id < 0 || id >= vocab) {
        atomicOr(status, EG_STATUS_BAD_TOKEN);
        id = 0;
    }
    g[i] = from_f32<TW>(gelu_tanh_f(z[(size_t)t * ldz + o]) * to_f32<TW>(table[(size_t)id * side + o]));
}

template <typename TD>
__global__ void add_scaled_kernel(float* __restrict__ stream, const TD* __restrict__ delta, const float* __restrict__ scale, long long n, int hidden) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) stream[i] += scale[i % hidden] * to_f32<TD>(delta[i]);
}
}  // namespace

// residual float32 [tokens, hidden], in place, += scale_a * delta_a + scale_b * delta_b (deltas [tokens, hidden] in dtype_a / dtype_b or null,
// gains float32 [hidden] or null: 1); rows [tokens, hidden] in rows_dtype = the sum
EG_API int eg_add_scaled_rows(cudaStream_t stream, float* residual, const void* delta_a, int dtype_a, const float* scale_a, const void* delta_b, int dtype_b,
                              const float* scale_b, void* rows, int rows_dtype, int tokens, int hidden) {
    const long long n = (long long)tokens * hidden;
    if (n <= 0) return 0;
    if (!residual || !rows) return (int)cudaErrorInvalidValue;
    const int per = hidden % 4 == 0 ? 4 : 1;
    const unsigned blocks = (unsigned)((n / per + 255) / 256);
    if (rows_dtype == EG_BF16)
        add_scaled_rows_kernel<bf16><<<blocks, 256, 0, stream>>>(residual, delta_a, dtype_a, scale_a, delta_b, dtype_b, scale_b, (bf16*)rows, n, hidden, per);
    else
        add_scaled_rows_kernel<float><<<blocks, 256, 0, stream>>>(residual, delta_a, dtype_a, scale_a, delta_b, dtype_b, scale_b, (float*)rows, n, hidden, per);
    return eg_launch_status();
}

// z float32 [tokens, ldz] -> g [tokens, side] in `dtype` = gelu_tanh(z) * table[token id]; table [vocab, side] in `dtype`
EG_API int eg_token_side_gate(cudaStream_t stream, int dtype, const float* z, long long ldz, const int* token_ids, const void* table, int vocab, void* g,
                              int tokens, int side, int* status) {
    const long long n = (long long)tokens * side;
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == EG_BF16) token_side_gate_kernel<bf16><<<blocks, 256, 0, stream>>>(z, ldz, token_ids, (const bf16*)table, vocab, (bf16*)g, tokens, side, status);
    else token_side_gate_kernel<float><<<blocks, 256, 0, stream>>>(z, ldz, token_ids, (const float*)table, vocab, (float*)g, tokens, side, status);
    return eg_launch_status();
}

// residual [tokens, hidden] += scale [hidden] * delta [tokens, hidden]
EG_API int eg_add_scaled(cudaStream_t stream, float* residual, const void* delta, int delta_dtype, const float* scale, int tokens, int hidden) {
    const long long n = (long long)tokens * hidden;
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (delta_dtype == EG_BF16) add_scaled_kernel<bf16><<<blocks, 256, 0, stream>>>(residual, (const bf16*)delta, scale, n, hidden);
    else add_scaled_kernel<float><<<blocks, 256, 0, stream>>>(residual, (const float*)delta, scale, n, hidden);
    return eg_launch_status();
}
