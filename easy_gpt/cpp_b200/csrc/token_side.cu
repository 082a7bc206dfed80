// A per-layer token input: every token brings a small vector e of its own (a row of a table, by token id) that is gated
// by the stream, mapped to the model's width, normed and added:
//
//   g = gelu_tanh(G x) * e;   y = P g;   x <- x + w * y / sqrt(mean(y^2) + eps)        G [side, hidden], P [hidden, side]
//
// eg_token_side does this in one kernel, a block per token, and first takes in up to two branch outputs that are still to
// be added, each times a gain per channel (x <- x + s_a * d_a + s_b * d_b): the end of a layer whose branches run side by
// side costs one pass over the stream.  eg_token_side_rows is the unfused form (rows in, y out, no norm, no add).
// eg_add_scaled is the add alone.  All sums are float32; the weights are read in the precision they are stored in.
#include "common.cuh"

namespace {
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TD> __device__ __forceinline__ float load_as_f32(const void* p, size_t i) { return to_f32<TD>(((const TD*)p)[i]); }
__device__ __forceinline__ float load_dyn(const void* p, int dtype, size_t i) { return dtype == EG_BF16 ? load_as_f32<bf16>(p, i) : load_as_f32<float>(p, i); }

// TW: the weights' type.  rows_in null: x is the stream (updated in place, with the deltas, the norm and the add);
// else x = rows_in[t] (type TW) and y goes to y_out.
template <typename TW>
__global__ void token_side_kernel(float* __restrict__ stream, const void* __restrict__ delta_a, int dtype_a, const float* __restrict__ scale_a,
                                  const void* __restrict__ delta_b, int dtype_b, const float* __restrict__ scale_b, const TW* __restrict__ rows_in,
                                  long long ld_in, float* __restrict__ y_out, const int* __restrict__ token_ids, const TW* __restrict__ table, int vocab,
                                  const TW* __restrict__ gate_w, const TW* __restrict__ proj_w, const float* __restrict__ norm_gain, float eps, int hidden,
                                  int side, int* status) {
    extern __shared__ float smem[];                  // [hidden] the row, then y; [side] g
    __shared__ float scratch[32];
    float* xs = smem;
    float* gs = smem + hidden;
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    float* x = stream ? stream + (size_t)t * hidden : nullptr;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float v;
        if (rows_in) {
            v = to_f32<TW>(rows_in[(size_t)t * ld_in + j]);
        } else {
            v = x[j];
            if (delta_a) v += (scale_a ? scale_a[j] : 1.0f) * load_dyn(delta_a, dtype_a, (size_t)t * hidden + j);
            if (delta_b) v += (scale_b ? scale_b[j] : 1.0f) * load_dyn(delta_b, dtype_b, (size_t)t * hidden + j);
            if (delta_a || delta_b) x[j] = v;
        }
        xs[j] = v;
    }
    __syncthreads();
    int id = token_ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, EG_STATUS_BAD_TOKEN);
        id = 0;
    }
    for (int o = warp; o < side; o += warps) {
        const TW* w = gate_w + (size_t)o * hidden;
        float acc = 0.f;
        for (int j = lane; j < hidden; j += 32) acc = fmaf(to_f32<TW>(w[j]), xs[j], acc);
        acc = warp_sum(acc);
        if (lane == 0) gs[o] = gelu_tanh_f(acc) * to_f32<TW>(table[(size_t)id * side + o]);
    }
    __syncthreads();
    float ss = 0.f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const TW* w = proj_w + (size_t)j * side;
        float acc = 0.f;
        for (int o = 0; o < side; ++o) acc = fmaf(to_f32<TW>(w[o]), gs[o], acc);
        if (rows_in) y_out[(size_t)t * hidden + j] = acc;
        else xs[j] = acc;
        ss = fmaf(acc, acc, ss);
    }
    if (rows_in) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) x[j] += norm_gain[j] * (xs[j] * inv);
}

template <typename TD>
__global__ void add_scaled_kernel(float* __restrict__ stream, const TD* __restrict__ delta, const float* __restrict__ scale, long long n, int hidden) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) stream[i] += scale[i % hidden] * to_f32<TD>(delta[i]);
}
}  // namespace

// residual float32 [tokens, hidden], in place.  delta_a / delta_b [tokens, hidden] (dtype_a / dtype_b) with gains scale_a / scale_b
// float32 [hidden] (null: 1), or null.  table [vocab, side], gate_w [side, hidden], proj_w [hidden, side] in `dtype`.
EG_API int eg_token_side(cudaStream_t stream, int dtype, float* residual, const void* delta_a, int dtype_a, const float* scale_a, const void* delta_b, int dtype_b,
                         const float* scale_b, const int* token_ids, const void* table, int vocab, const void* gate_w, const void* proj_w,
                         const float* norm_gain, float eps, int tokens, int hidden, int side, int* status) {
    if (tokens <= 0) return 0;
    const size_t smem = (size_t)(hidden + side) * sizeof(float);
    if (smem > 48 * 1024 || side <= 0) return (int)cudaErrorInvalidValue;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == EG_BF16)
        token_side_kernel<bf16><<<tokens, threads, smem, stream>>>(residual, delta_a, dtype_a, scale_a, delta_b, dtype_b, scale_b, nullptr, 0, nullptr, token_ids,
                                                                   (const bf16*)table, vocab, (const bf16*)gate_w, (const bf16*)proj_w, norm_gain, eps, hidden, side, status);
    else
        token_side_kernel<float><<<tokens, threads, smem, stream>>>(residual, delta_a, dtype_a, scale_a, delta_b, dtype_b, scale_b, nullptr, 0, nullptr, token_ids,
                                                                    (const float*)table, vocab, (const float*)gate_w, (const float*)proj_w, norm_gain, eps, hidden, side,
                                                                    status);
    return eg_launch_status();
}

// rows [tokens, ld] in `dtype` -> y float32 [tokens, hidden] = P (gelu_tanh(G rows) * e)
EG_API int eg_token_side_rows(cudaStream_t stream, int dtype, const void* rows, long long ld, float* y, const int* token_ids, const void* table, int vocab,
                              const void* gate_w, const void* proj_w, int tokens, int hidden, int side, int* status) {
    if (tokens <= 0) return 0;
    const size_t smem = (size_t)(hidden + side) * sizeof(float);
    if (smem > 48 * 1024 || side <= 0 || !rows || !y) return (int)cudaErrorInvalidValue;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == EG_BF16)
        token_side_kernel<bf16><<<tokens, threads, smem, stream>>>(nullptr, nullptr, 0, nullptr, nullptr, 0, nullptr, (const bf16*)rows, ld, y, token_ids,
                                                                   (const bf16*)table, vocab, (const bf16*)gate_w, (const bf16*)proj_w, nullptr, 0.f, hidden, side, status);
    else
        token_side_kernel<float><<<tokens, threads, smem, stream>>>(nullptr, nullptr, 0, nullptr, nullptr, 0, nullptr, (const float*)rows, ld, y, token_ids,
                                                                    (const float*)table, vocab, (const float*)gate_w, (const float*)proj_w, nullptr, 0.f, hidden, side,
                                                                    status);
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
