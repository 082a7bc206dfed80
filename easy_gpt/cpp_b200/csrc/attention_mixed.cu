// Grouped-query attention whose scores are mixed across the heads before the softmax, whose values are the keys as they
// were projected, and whose output is gated.  With H query heads, G key heads of dk values (head h reads key head
// c(h) = h / (H / G)), a matrix M [H, H], q^ and k^ the normed and turned queries and keys and k the raw keys:
//
//   s_h(i, j) = sum_g M[h, g] * scale * (q^_g(i) . k^_c(g)(j))              every head's score is a mix of all heads' scores
//             = sum_c  Q_h,c(i) . k^_c(j),   Q_h,c(i) = scale * sum_{g: c(g) = c} M[h, g] q^_g(i)
//   a_h(i, .) = softmax over j <= i of s_h(i, .);   o_h(i) = sum_j a_h(i, j) k_c(h)(j);   out_h(i) = o_h(i) * sigmoid(gate_h(i))
//
// The mix is folded into the queries: a head's query becomes a row of G * dk values that meets the keys of ALL key heads
// of a token, side by side, so that the attention itself is an ordinary one with one wide key per token (and the value
// of head h is the slice c(h) of the token's raw keys).  The cache keeps two planes per token and key head: k^ and k.
//
//   eg_mixed_attention_prepare   per token: q^ and k^ (unit root mean square per head times a weight [dk], float32; then a half
//                                rotation of the first rot_dims values with the step's cos/sin table times `magnitude`), the folded
//                                queries Q [tokens, H, G * dk], and the token's k^ and k rows in the cache
//   eg_mixed_attention           the attention over the paged cache, a warp per (token, head), float32 sums in chunks of 32
//                                keys from position 0: the order of the sums depends on the token's position alone
#include <algorithm>

#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_PER_LANE = 8;      // dk <= 256

// blocks (t, y): every block norms and turns token t's heads, block y == 0 stores the keys, and the blocks share the
// token's folded queries; proj float32 [tokens, ld]: H query heads, then G key heads
template <typename T>
__global__ void __launch_bounds__(256) mixed_prepare_kernel(const float* __restrict__ proj, long long ld, const float* __restrict__ q_weight,
                                                            const float* __restrict__ k_weight, float eps, const float2* __restrict__ table, int half,
                                                            float magnitude, const float* __restrict__ mix, float scale, const int* __restrict__ slot_map,
                                                            T* __restrict__ k_cache, T* __restrict__ v_cache, long long head_stride, int page_size,
                                                            long long page_stride, long long pool_slots, void* __restrict__ q_out, int q_f32, int heads, int kv_heads,
                                                            int dk, int* status) {
    extern __shared__ float qs[];                     // [heads, dk] normed and turned queries
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int rot = 2 * half;
    for (int h = warp; h < heads + kv_heads; h += warps) {
        const bool is_q = h < heads;
        const float* src = proj + (size_t)t * ld + (size_t)h * dk;
        const float* weight = is_q ? q_weight : k_weight;
        T *k_dst = nullptr, *v_dst = nullptr;
        if (!is_q) {
            if (!k_cache || blockIdx.y != 0) continue;
            const long long slot = slot_map[t];
            if (slot < 0 || slot >= pool_slots) {
                if (lane == 0) atomicOr(status, EG_STATUS_BAD_SLOT);
                continue;
            }
            const long long at = (slot / page_size) * page_stride + (h - heads) * head_stride + (slot % page_size) * (long long)dk;
            k_dst = k_cache + at;
            v_dst = v_cache + at;
        }
        float ss = 0.f;
        for (int d = lane; d < dk; d += 32) ss = fmaf(src[d], src[d], ss);
        ss = warp_sum(ss);
        const float inv = eps >= 0.f ? 1.0f / sqrtf(ss / (float)dk + eps) : 1.0f;
        for (int d = lane; d < dk; d += 32) {
            const float raw = src[d];
            float x = raw * inv * (weight ? weight[d] : 1.0f);
            if (d < rot) {
                const int i = d < half ? d : d - half;
                const int o = d < half ? d + half : d - half;
                const float other = src[o] * inv * (weight ? weight[o] : 1.0f);
                const float2 cs = table[(size_t)t * half + i];
                const float c = cs.x * magnitude, s = cs.y * magnitude;
                x = d < half ? x * c - other * s : x * c + other * s;
            }
            if (is_q) {
                qs[h * dk + d] = x;
            } else {
                k_dst[d] = from_f32<T>(x);
                v_dst[d] = from_f32<T>(raw);
            }
        }
    }
    __syncthreads();
    // the folded queries: a warp per (head h, key head c), over all blocks of the token; a lane takes pairs of values
    const int group = heads / kv_heads, wide = kv_heads * dk;
    for (int hc = blockIdx.y * warps + warp; hc < heads * kv_heads; hc += gridDim.y * warps) {
        const int h = hc / kv_heads, c = hc % kv_heads;
        const float* m = mix + (size_t)h * heads + c * group;
        const float* src = qs + (size_t)c * group * dk;
        const size_t at = (size_t)t * heads * wide + (size_t)h * wide + (size_t)c * dk;
        for (int d = 2 * lane; d < dk; d += 64) {
            float a0 = 0.f, a1 = 0.f;
            for (int g = 0; g < group; ++g) {
                const float w = m[g];
                a0 = fmaf(w, src[g * dk + d], a0);
                if (d + 1 < dk) a1 = fmaf(w, src[g * dk + d + 1], a1);
            }
            a0 *= scale;
            a1 *= scale;
            if (q_f32) {
                ((float*)q_out)[at + d] = a0;
                if (d + 1 < dk) ((float*)q_out)[at + d + 1] = a1;
            } else if (d + 1 < dk && dk % 2 == 0) {
                *(__nv_bfloat162*)((bf16*)q_out + at + d) = __floats2bfloat162_rn(a0, a1);
            } else {
                ((bf16*)q_out)[at + d] = __float2bfloat16_rn(a0);
                if (d + 1 < dk) ((bf16*)q_out)[at + d + 1] = __float2bfloat16_rn(a1);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
mixed_attention_kernel(const void* __restrict__ q, int q_f32, const T* __restrict__ k_cache, const T* __restrict__ v_cache, long long head_stride,
                       const int* __restrict__ block_table, int table_stride, const int* __restrict__ token_seq, const int* __restrict__ positions,
                       const float* __restrict__ gate, long long ld_gate, T* __restrict__ out, long long ldo, int heads, int kv_heads, int dk, int page_size,
                       long long page_stride, int num_pages, int* status) {
    extern __shared__ float q_shared[];              // WARPS * kv_heads * dk
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * WARPS + warp;
    if (h >= heads) return;                           // no block-wide barrier below
    const int wide = kv_heads * dk;
    const int c_own = h / (heads / kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)token_seq[t] * table_stride;
    float* qs = q_shared + warp * wide;
    const size_t q_at = ((size_t)t * heads + h) * wide;
    for (int d = lane; d < wide; d += 32) qs[d] = q_f32 ? ((const float*)q)[q_at + d] : __bfloat162float(((const bf16*)q)[q_at + d]);
    __syncwarp();

    float m = -INFINITY, l = 0.0f;
    float acc[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] = 0.0f;
    for (int base = 0; base <= pos; base += 32) {
        const int kpos = base + lane;
        long long row_off = -1;
        if (kpos <= pos) {
            const int page = table[kpos / page_size];
            if (page < 0 || page >= num_pages) atomicOr(status, EG_STATUS_BAD_PAGE);
            else row_off = (long long)page * page_stride + (long long)(kpos % page_size) * dk;
        }
        float s = -INFINITY;
        if (row_off >= 0) {
            float dot = 0.0f;
            for (int c = 0; c < kv_heads; ++c) {
                const T* krow = k_cache + row_off + c * head_stride;
                const float* qc = qs + c * dk;
                for (int d = 0; d < dk; ++d) dot = fmaf(qc[d], to_f32<T>(krow[d]), dot);
            }
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float corr = expf(m - m_new);
        const float p = (row_off >= 0) ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] *= corr;
        const int nkeys = min(32, pos - base + 1);
        for (int j = 0; j < nkeys; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long off_j = __shfl_sync(0xffffffffu, row_off, j);
            if (off_j < 0) continue;
            const T* vrow = v_cache + off_j + c_own * head_stride;
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < dk) acc[i] = fmaf(pj, to_f32<T>(vrow[d]), acc[i]);
            }
        }
        m = m_new;
    }
    T* orow = out + (size_t)t * ldo + (size_t)h * dk;
    const float* grow = gate ? gate + (size_t)t * ld_gate + (size_t)h * dk : nullptr;
    const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < dk) {
            float v = acc[i] * inv_l;
            if (grow) v *= 1.0f / (1.0f + expf(-grow[d]));
            orow[d] = from_f32<T>(v);
        }
    }
}
}  // namespace

// proj float32 [tokens, ld]: query heads then key heads.  q_weight / k_weight float32 [dk] or null; eps < 0: no division by the
// root mean square.  table: cos/sin [tokens, rot_dims/2, 2] or null with rot_dims 0.  mix float32 [heads, heads].  k_cache null:
// nothing is stored.  The caches are in `dtype`, q_out [tokens, heads, kv_heads * dk] in q_dtype.
EG_API int eg_mixed_attention_prepare(cudaStream_t stream, int dtype, const float* proj, long long ld, const float* q_weight, const float* k_weight, float eps,
                                      const float* table, int rot_dims, float magnitude, const float* mix, float scale, const int* slot_map, void* k_cache,
                                      void* v_cache, long long head_stride, int page_size, long long page_stride, long long pool_slots, void* q_out, int q_dtype,
                                      int tokens, int heads, int kv_heads, int dk, int* status) {
    if (tokens <= 0) return 0;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > dk || (rot_dims > 0 && !table) || !mix || kv_heads <= 0 || heads % kv_heads) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)heads * dk * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    // a step of few tokens spreads a token's folded queries over several blocks (each norms and turns the token's heads itself)
    const int per_token = tokens >= 128 ? 1 : std::max(1, std::min(heads * kv_heads / 8, 128 / tokens));
    const dim3 grid(tokens, per_token);
    if (dtype == EG_BF16)
        mixed_prepare_kernel<bf16><<<grid, 256, smem, stream>>>(proj, ld, q_weight, k_weight, eps, (const float2*)table, rot_dims / 2, magnitude, mix, scale, slot_map,
                                                                  (bf16*)k_cache, (bf16*)v_cache, head_stride, page_size, page_stride, pool_slots, q_out, q_dtype == EG_F32,
                                                                  heads, kv_heads, dk, status);
    else
        mixed_prepare_kernel<float><<<grid, 256, smem, stream>>>(proj, ld, q_weight, k_weight, eps, (const float2*)table, rot_dims / 2, magnitude, mix, scale, slot_map,
                                                                   (float*)k_cache, (float*)v_cache, head_stride, page_size, page_stride, pool_slots, q_out,
                                                                   q_dtype == EG_F32, heads, kv_heads, dk, status);
    return eg_launch_status();
}

// q [tokens, heads, kv_heads * dk] (folded queries, in q_dtype); gate float32 [tokens, ld_gate] with head h at column h * dk, or null;
// out [tokens, ldo] with head h at column h * dk.  Returns cudaErrorInvalidValue for sizes it does not take.
EG_API int eg_mixed_attention(cudaStream_t stream, int dtype, const void* q, int q_dtype, const void* k_cache, const void* v_cache, long long head_stride,
                              const int* block_table, int table_stride, const int* token_seq, const int* positions, const float* gate, long long ld_gate,
                              void* out, long long ldo, int num_tokens, int heads, int kv_heads, int dk, int page_size, long long page_stride, int num_pages,
                              int* status) {
    if (num_tokens <= 0) return 0;
    if (dk <= 0 || dk > 32 * MAX_PER_LANE || kv_heads <= 0 || heads % kv_heads) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)WARPS * kv_heads * dk * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    dim3 grid(num_tokens, (heads + WARPS - 1) / WARPS);
    if (dtype == EG_BF16)
        mixed_attention_kernel<bf16><<<grid, WARPS * 32, smem, stream>>>(q, q_dtype == EG_F32, (const bf16*)k_cache, (const bf16*)v_cache, head_stride, block_table,
                                                                         table_stride, token_seq, positions, gate, ld_gate, (bf16*)out, ldo, heads, kv_heads, dk,
                                                                         page_size, page_stride, num_pages, status);
    else
        mixed_attention_kernel<float><<<grid, WARPS * 32, smem, stream>>>(q, q_dtype == EG_F32, (const float*)k_cache, (const float*)v_cache, head_stride, block_table,
                                                                          table_stride, token_seq, positions, gate, ld_gate, (float*)out, ldo, heads, kv_heads, dk,
                                                                          page_size, page_stride, num_pages, status);
    return eg_launch_status();
}
