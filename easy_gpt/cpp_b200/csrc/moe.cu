// A routed feed-forward: a router that picks `top` of the experts per token, gated experts, experts that hand their
// input through unchanged, and a gate on a shared expert.
//
//   eg_moe_route     logits = R h (float32); s = softmax(logits) over all router outputs; the `top` largest of
//                    s + correction are chosen (ties: the lower index); their weights are s itself, not renormalised.
//                    Also g[t] = sigmoid(w_g . h), the gate of the shared expert, when w_g is given.
//   eg_moe_hidden    a[t, k, :] = silu(G_e h) * (U_e h) for the k-th chosen expert e of token t (skipped for router
//                    outputs >= experts: those stand for the identity)
//   eg_moe_combine   out[t, :] = sum_k weight[t, k] * (D_e a[t, k, :]  or  h[t, :] for an identity choice)
//                                + g[t] * shared[t, :]                   (float32)
//
// eg_moe_hidden and eg_moe_combine read each chosen expert's weights per token: the form for steps of few tokens.
// For steps of many tokens the rows are sorted by expert instead, so that every expert's weights meet all of its rows in
// one grouped product on the tensor cores (eg_gemm_tcgen05_grouped):
//   eg_moe_dispatch  counts the rows of every expert, gives each expert a run of rows that starts at a multiple of 128,
//                    says which expert every tile of 128 rows belongs to, and copies each token's row to its places
//   eg_moe_gather    out[t, :] = sum_k weight[t, k] * (y[row_of[t, k], :] or h[t, :]) + g[t] * shared[t, :]
// The sizes of the runs stay on the device: nothing here waits for the host.
// Products accumulate in float32; the router is float32 throughout.
//
// Variants, each a parameter: `scoring` 1 takes s = sigmoid(logits) instead of the softmax (the correction may then be null);
// `activation` 1 is the clamped gate g' = min(g, limit), u' = clamp(u, -limit, limit), a = g' sigmoid(1.702 g') (u' + 1);
// `input_weights` (eg_moe_hidden, eg_moe_dispatch) multiply an expert's INPUT row, expert(w h), and eg_moe_combine / eg_moe_gather
// then get null weights (every term counts once); a null gate adds the shared expert's output as it is.
#include "common.cuh"

namespace {

// grid (token, chunk of eight router outputs): a warp per output computes its logit (the output past the last one is the
// shared expert's gate), so that a step of few tokens still fills the SMs
template <typename T>
__global__ void __launch_bounds__(256) moe_logits_kernel(const T* __restrict__ h, long long ld, const float* __restrict__ router,
                                                         const float* __restrict__ gate_w, float* __restrict__ logits, float* __restrict__ gate, int width,
                                                         int outputs) {
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.y * (blockDim.x >> 5) + warp;
    if (e >= outputs + (gate_w ? 1 : 0)) return;
    const float* w = e < outputs ? router + (size_t)e * width : gate_w;
    const T* row = h + (size_t)t * ld;
    float acc = 0.f;
#pragma unroll 8
    for (int j = lane; j < width; j += 32) acc = fmaf(w[j], to_f32<T>(row[j]), acc);
    acc = warp_sum(acc);
    if (lane == 0) {
        if (e < outputs) logits[(size_t)t * outputs + e] = acc;
        else gate[t] = 1.0f / (1.0f + expf(-acc));
    }
}

// a warp per token: softmax over the logits (left in place as scores), then the `top` largest of score + correction
__global__ void __launch_bounds__(128) moe_select_kernel(float* __restrict__ logits, const float* __restrict__ correction, int* __restrict__ ids,
                                                         float* __restrict__ weights, int tokens, int outputs, int top, int scoring) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= tokens) return;
    float* logit = logits + (size_t)t * outputs;
    if (scoring == 1) {
        for (int e = lane; e < outputs; e += 32) logit[e] = 1.0f / (1.0f + expf(-logit[e]));      // now the scores s
    } else {
        float top_logit = -INFINITY;
        for (int e = lane; e < outputs; e += 32) top_logit = fmaxf(top_logit, logit[e]);
        top_logit = warp_max(top_logit);
        float sum = 0.f;
        for (int e = lane; e < outputs; e += 32) sum += expf(logit[e] - top_logit);
        sum = warp_sum(sum);
        for (int e = lane; e < outputs; e += 32) logit[e] = expf(logit[e] - top_logit) / sum;      // now the scores s
    }
    __syncwarp();
    unsigned long long taken = 0ull;             // a lane tracks which of its own outputs are taken: bit k for e = lane + 32 k
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane, i = 0; e < outputs; e += 32, ++i) {
            if ((taken >> i) & 1ull) continue;
            const float v = logit[e] + (correction ? correction[e] : 0.f);
            if (v > best) { best = v; arg = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg != 0x7fffffff && arg % 32 == lane) taken |= 1ull << (arg / 32);
        if (lane == 0) {
            ids[(size_t)t * top + k] = arg == 0x7fffffff ? outputs : arg;
            weights[(size_t)t * top + k] = arg == 0x7fffffff ? 0.f : logit[arg];
        }
    }
}

// grid (token, choice, chunk of ff); a warp per hidden unit; GU [experts, 2 ff, width] with the gate row of unit f at
// 2 f and its up row at 2 f + 1
template <typename T>
__global__ void __launch_bounds__(256) moe_hidden_kernel(const T* __restrict__ h, long long ld, const T* __restrict__ GU, const int* __restrict__ ids,
                                                         const float* __restrict__ input_weights, T* __restrict__ act, int width, int ff, int top,
                                                         int experts, int activation, float limit) {
    extern __shared__ float row[];
    const int t = blockIdx.x, k = blockIdx.y;
    const int e = ids[(size_t)t * top + k];
    if (e >= experts) return;
    for (int j = threadIdx.x; j < width; j += blockDim.x) row[j] = to_f32<T>(h[(size_t)t * ld + j]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int f = blockIdx.z * warps + warp;
    if (f >= ff) return;
    const T* g = GU + ((size_t)e * 2 * ff + 2 * f) * width;
    const T* u = g + width;
    float ag = 0.f, au = 0.f;
    if (sizeof(T) == 2 && width % 8 == 0) {                      // eight weights a load
        const uint4* g8 = reinterpret_cast<const uint4*>(g);
        const uint4* u8 = reinterpret_cast<const uint4*>(u);
#pragma unroll 2
        for (int j = lane; j < width / 8; j += 32) {
            const uint4 gv = g8[j], uv = u8[j];
            const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
            const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 gf = __bfloat1622float2(gp[q]), uf = __bfloat1622float2(up[q]);
                ag = fmaf(gf.x, row[8 * j + 2 * q], ag);
                ag = fmaf(gf.y, row[8 * j + 2 * q + 1], ag);
                au = fmaf(uf.x, row[8 * j + 2 * q], au);
                au = fmaf(uf.y, row[8 * j + 2 * q + 1], au);
            }
        }
    } else {
        for (int j = lane; j < width; j += 32) {
            ag = fmaf(to_f32<T>(g[j]), row[j], ag);
            au = fmaf(to_f32<T>(u[j]), row[j], au);
        }
    }
    ag = warp_sum(ag);
    au = warp_sum(au);
    if (input_weights) {                                         // the expert reads w h: its two products are w times these
        const float wgt = input_weights[(size_t)t * top + k];
        ag *= wgt;
        au *= wgt;
    }
    float a;
    if (activation == 1) {
        ag = fminf(ag, limit);
        au = fminf(fmaxf(au, -limit), limit);
        a = ag / (1.0f + expf(-1.702f * ag)) * (au + 1.0f);
    } else {
        a = ag / (1.0f + expf(-ag)) * au;
    }
    if (lane == 0) act[((size_t)t * top + k) * ff + f] = from_f32<T>(a);
}

// grid (token, chunk of width); a warp per output value; Dn [experts, width, ff]
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const T* __restrict__ h, long long ld, const T* __restrict__ act, const T* __restrict__ Dn,
                                                          const int* __restrict__ ids, const float* __restrict__ weights, const void* __restrict__ shared,
                                                          int shared_dtype, const float* __restrict__ gate, float* __restrict__ out, int width, int ff,
                                                          int top, int experts) {
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int j = blockIdx.y * warps + warp;
    if (j >= width) return;
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        const int e = ids[(size_t)t * top + k];
        const float wgt = weights ? weights[(size_t)t * top + k] : 1.0f;
        if (e >= experts) {
            total += wgt * to_f32<T>(h[(size_t)t * ld + j]);
            continue;
        }
        const T* d = Dn + ((size_t)e * width + j) * ff;
        const T* a = act + ((size_t)t * top + k) * ff;
        float acc = 0.f;
        if (sizeof(T) == 2 && ff % 8 == 0) {                     // eight weights a load
            const uint4* d8 = reinterpret_cast<const uint4*>(d);
            const uint4* a8 = reinterpret_cast<const uint4*>(a);
#pragma unroll 2
            for (int f = lane; f < ff / 8; f += 32) {
                const uint4 dv = d8[f], av = a8[f];
                const __nv_bfloat162* dp = reinterpret_cast<const __nv_bfloat162*>(&dv);
                const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 df = __bfloat1622float2(dp[q]), af = __bfloat1622float2(ap[q]);
                    acc = fmaf(df.x, af.x, acc);
                    acc = fmaf(df.y, af.y, acc);
                }
            }
        } else {
            for (int f = lane; f < ff; f += 32) acc = fmaf(to_f32<T>(d[f]), to_f32<T>(a[f]), acc);
        }
        total += wgt * warp_sum(acc);
    }
    if (shared) {
        const size_t i = (size_t)t * width + j;
        total += (gate ? gate[t] : 1.0f) * (shared_dtype == EG_BF16 ? __bfloat162float(((const bf16*)shared)[i]) : ((const float*)shared)[i]);
    }
    if (lane == 0) out[(size_t)t * width + j] = total;
}

}  // namespace

// ids [T, top] int32 (router outputs; those >= the number of experts stand for the identity), weights [T, top] float32,
// gate [T] float32 (only with gate_w); logits [T, outputs] float32 is scratch (it ends up holding the scores)
EG_API int eg_moe_route(cudaStream_t stream, int dtype, const void* h, long long ld, const float* router, const float* correction, const float* gate_w,
                        float* logits, int* ids, float* weights, float* gate, int tokens, int width, int outputs, int top, int scoring) {
    if (tokens <= 0) return 0;
    if (top < 1 || top > outputs || outputs > 2048 || !logits || scoring < 0 || scoring > 1) return (int)cudaErrorInvalidValue;
    dim3 grid(tokens, (outputs + (gate_w ? 1 : 0) + 7) / 8);
    if (dtype == EG_BF16) moe_logits_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)h, ld, router, gate_w, logits, gate, width, outputs);
    else moe_logits_kernel<float><<<grid, 256, 0, stream>>>((const float*)h, ld, router, gate_w, logits, gate, width, outputs);
    moe_select_kernel<<<(tokens + 3) / 4, 128, 0, stream>>>(logits, correction, ids, weights, tokens, outputs, top, scoring);
    return eg_launch_status();
}

// act [T, top, ff] in the compute dtype; rows of identity choices (ids >= experts) are left untouched
EG_API int eg_moe_hidden(cudaStream_t stream, int dtype, const void* h, long long ld, const void* gate_up, const int* ids, const float* input_weights,
                         void* act, int tokens, int width, int ff, int top, int experts, int activation, float limit) {
    if (tokens <= 0 || experts <= 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    dim3 grid(tokens, top, (ff + 7) / 8);
    if (dtype == EG_BF16) moe_hidden_kernel<bf16><<<grid, 256, smem, stream>>>((const bf16*)h, ld, (const bf16*)gate_up, ids, input_weights, (bf16*)act, width, ff, top, experts, activation, limit);
    else moe_hidden_kernel<float><<<grid, 256, smem, stream>>>((const float*)h, ld, (const float*)gate_up, ids, input_weights, (float*)act, width, ff, top, experts, activation, limit);
    return eg_launch_status();
}

// out [T, width] float32; shared [T, width] (shared_dtype) with gate [T], or null
EG_API int eg_moe_combine(cudaStream_t stream, int dtype, const void* h, long long ld, const void* act, const void* down, const int* ids,
                          const float* weights, const void* shared, int shared_dtype, const float* gate, float* out, int tokens, int width, int ff,
                          int top, int experts) {
    if (tokens <= 0) return 0;
    dim3 grid(tokens, (width + 7) / 8);
    if (dtype == EG_BF16)
        moe_combine_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)h, ld, (const bf16*)act, (const bf16*)down, ids, weights, shared, shared_dtype, gate,
                                                          out, width, ff, top, experts);
    else
        moe_combine_kernel<float><<<grid, 256, 0, stream>>>((const float*)h, ld, (const float*)act, (const float*)down, ids, weights, shared, shared_dtype,
                                                           gate, out, width, ff, top, experts);
    return eg_launch_status();
}

namespace {
__global__ void moe_count_kernel(const int* __restrict__ ids, int* __restrict__ counts, int pairs, int experts) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < pairs && ids[i] < experts) atomicAdd(&counts[ids[i]], 1);
}
// one block: starts[e] = first row of expert e's run (runs padded to 128 rows), cursors to zero, tiles labelled
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ starts, int* __restrict__ cursors, int* __restrict__ tile_group,
                                   int experts, int max_tiles) {
    for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_group[i] = -1;
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            starts[e] = at;
            at += (counts[e] + 127) / 128 * 128;
        }
        starts[experts] = at;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        cursors[e] = 0;
        for (int tile = starts[e] / 128; tile < starts[e + 1] / 128 && tile < max_tiles; ++tile) tile_group[tile] = e;
    }
}
// a warp per (token, choice): takes the next row of the expert's run and copies the token's row there
__global__ void __launch_bounds__(256) moe_scatter_kernel(const bf16* __restrict__ h, long long ld, const int* __restrict__ ids, const int* __restrict__ starts,
                                                          int* __restrict__ cursors, int* __restrict__ row_of, bf16* __restrict__ rows,
                                                          const float* __restrict__ input_weights, int pairs, int width, int top, int experts, int max_rows) {
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= pairs) return;
    const int e = ids[pair];
    if (e >= experts) {
        if (lane == 0) row_of[pair] = -1;
        return;
    }
    int row = 0;
    if (lane == 0) {
        row = starts[e] + atomicAdd(&cursors[e], 1);
        if (row >= max_rows) row = -1;
        row_of[pair] = row;
    }
    row = __shfl_sync(0xffffffffu, row, 0);
    if (row < 0) return;
    const bf16* src = h + (size_t)(pair / top) * ld;
    bf16* dst = rows + (size_t)row * width;
    if (input_weights) {                                        // the expert's input is the row times the pair's weight
        const float wgt = input_weights[pair];
        for (int j = lane; j < width; j += 32) dst[j] = __float2bfloat16_rn(wgt * __bfloat162float(src[j]));
    } else if (width % 8 == 0 && ld % 8 == 0) {
        for (int j = lane; j < width / 8; j += 32) reinterpret_cast<uint4*>(dst)[j] = reinterpret_cast<const uint4*>(src)[j];
    } else {
        for (int j = lane; j < width; j += 32) dst[j] = src[j];
    }
}
__global__ void moe_gather_kernel(const bf16* __restrict__ y, const int* __restrict__ row_of, const int* __restrict__ ids, const float* __restrict__ weights,
                                  const bf16* __restrict__ h, long long ld, const void* __restrict__ shared, int shared_dtype, const float* __restrict__ gate,
                                  float* __restrict__ out, int tokens, int width, int top, int experts) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * width) return;
    const int t = (int)(i / width), j = (int)(i % width);
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        const int e = ids[(size_t)t * top + k];
        const float wgt = weights ? weights[(size_t)t * top + k] : 1.0f;
        if (e >= experts) total += wgt * __bfloat162float(h[(size_t)t * ld + j]);
        else {
            const int row = row_of[(size_t)t * top + k];
            if (row >= 0) total += wgt * __bfloat162float(y[(size_t)row * width + j]);
        }
    }
    if (shared) total += (gate ? gate[t] : 1.0f) * (shared_dtype == EG_BF16 ? __bfloat162float(((const bf16*)shared)[i]) : ((const float*)shared)[i]);
    out[i] = total;
}
}  // namespace

// Sorts the step's (token, choice) pairs by expert (bfloat16 rows).  counts, cursors [experts] and starts [experts + 1] are
// scratch; tile_group [max_rows / 128] and row_of [tokens * top] are results, rows [max_rows, width] receives the copies.
// max_rows: a multiple of 128, at least tokens * top rounded up to 128 plus 128 per expert.
EG_API int eg_moe_dispatch(cudaStream_t stream, const void* h, long long ld, const int* ids, const float* input_weights, int* counts, int* starts, int* cursors,
                           int* tile_group, int* row_of, void* rows, int tokens, int width, int top, int experts, int max_rows) {
    const int pairs = tokens * top;
    if (pairs <= 0 || experts <= 0) return 0;
    if (max_rows % 128 || max_rows < (pairs + 127) / 128 * 128 + 128 * experts || experts > 2048) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaMemsetAsync(counts, 0, (size_t)experts * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
    moe_count_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(ids, counts, pairs, experts);
    moe_offsets_kernel<<<1, 256, 0, stream>>>(counts, starts, cursors, tile_group, experts, max_rows / 128);
    moe_scatter_kernel<<<(pairs + 7) / 8, 256, 0, stream>>>((const bf16*)h, ld, ids, starts, cursors, row_of, (bf16*)rows, input_weights, pairs, width, top, experts, max_rows);
    return eg_launch_status();
}

// out [T, width] float32 from the experts' outputs y [max_rows, width] (bfloat16) in sorted order
EG_API int eg_moe_gather(cudaStream_t stream, const void* y, const int* row_of, const int* ids, const float* weights, const void* h, long long ld,
                         const void* shared, int shared_dtype, const float* gate, float* out, int tokens, int width, int top, int experts) {
    const long long n = (long long)tokens * width;
    if (n <= 0) return 0;
    moe_gather_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const bf16*)y, row_of, ids, weights, (const bf16*)h, ld, shared, shared_dtype, gate, out,
                                                                      tokens, width, top, experts);
    return eg_launch_status();
}
