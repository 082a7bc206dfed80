// Grouped-query attention with the mask, the score function and the softmax as parameters, over a paged cache that keeps
// either one row (keys | value) per token and KV head or, where a head has one key of the value's size, keys and values in
// planes of their own.  A key lies at k[page * page_stride + head * head_stride + offset * row_stride (+ map * dk)], its
// value at the same place from v.
//
// Heads.  H heads, each with `maps` queries (1, or 2 for an attention that takes one softmax map off another): the query
// rows are [tokens, H * maps, dk], row h * maps + m being map m of head h.  KV head g = h / (H / G) holds `maps` keys of dk
// values side by side and ONE value of dv values, which all maps share.  The output has a row per (head, map).
//
// With `planes` (keys and values in planes of their own, which holds for dk = dv only) both planes have G * maps heads: key
// head g * maps + m is map m's key of head g, and the value of head g is stored once per map, so that a kernel that knows
// nothing of maps sees G * maps ordinary key/value heads.
//
// Preparation, per token at position p (float32 throughout, from the float32 output of the projections):
//   norm_eps >= 0: every query and key (per head and map) is divided by its root mean square over dk (eps under the root)
//   and, with a gain [dk] given, multiplied by it channel by channel;
//   then the first rot_dims values are turned in pairs (i, i + rot_dims/2) by the angle p * f_i:
//   (u, v) -> (u c - v s, v c + u s) with (c, s) = magnitude * (cos, sin) from the step's table;
//   queries go to q_out, keys and values to the token's row of the cache.
//
// Attention.  The token at position p of its request sees key j <= p if
//   (window <= 0 or p - j < window) and (chunk <= 0 or floor(j / chunk) == floor(p / chunk)), or if j < keep_first;
//   score = (q . k) * scale, then with softcap > 0: softcap * tanh(score / softcap);
//   weight_j = exp(s_j) / (sum_i exp(s_i) + (sinks ? exp(sinks[head row]) : 0)), the sink a term without a value;
//   out = out_scale * sum_j weight_j v_j.
// One warp per (token, query row), a running softmax over chunks of 32 keys that start at the first kept key and then at the
// first key of the window or chunk: the order of the sums depends on the token's position and the mask alone, never on how
// the request was cut into steps, on the batch or on the page ids.
//
// Difference of maps: o = a_0 - lambda a_1 per head, divided by its root mean square over dv (eps under the root) and
// multiplied by `post`.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_PER_LANE = 8;      // value size <= 256

// one warp per (token, row): rows 0..Q-1 are queries (Q = heads * maps), Q..Q+K-1 keys (K = kv_heads * maps), then kv_heads values
template <typename T>
__global__ void __launch_bounds__(128) masked_prepare_kernel(const float* __restrict__ proj, long long ld, const float2* __restrict__ table, int half,
                                                             float magnitude, const int* __restrict__ slot_map, T* __restrict__ k_cache,
                                                             T* __restrict__ v_cache, int row_stride, long long head_stride, int page_size,
                                                             long long page_stride, long long pool_slots, T* __restrict__ q_out, int tokens, int heads,
                                                             int kv_heads, int maps, int dk, int dv, float norm_eps, const float* __restrict__ q_gain,
                                                             const float* __restrict__ k_gain, int planes, int* status) {
    const int lane = threadIdx.x & 31;
    const int Q = heads * maps, K = kv_heads * maps, rows = Q + K + kv_heads;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)tokens * rows) return;
    const int t = (int)(w / rows), r = (int)(w % rows);
    long long at = 0;
    if (r >= Q) {
        if (!k_cache) return;                       // the entry reads another entry's cache and stores nothing
        const long long slot = slot_map[t];
        if (slot < 0 || slot >= pool_slots) {
            if (lane == 0) atomicOr(status, EG_STATUS_BAD_SLOT);
            return;
        }
        // the cache head: the key/value head, or with planes the (head, map) pair (a value then starts at its head's first map)
        const int g = r < Q + K ? (planes ? r - Q : (r - Q) / maps) : (planes ? (r - Q - K) * maps : r - Q - K);
        at = (slot / page_size) * page_stride + g * head_stride + (slot % page_size) * (long long)row_stride;
    }
    if (r >= Q + K) {                               // a value: stored as it is (with planes once per map)
        const float* v = proj + (size_t)t * ld + (size_t)(Q + K) * dk + (size_t)(r - Q - K) * dv;
        for (int c = 0; c < (planes ? maps : 1); ++c)
            for (int d = lane; d < dv; d += 32) v_cache[at + c * head_stride + d] = from_f32<T>(v[d]);
        return;
    }
    const float* src = proj + (size_t)t * ld + (size_t)r * dk;          // queries then keys, row after row
    const float* gain = r < Q ? q_gain : k_gain;
    T* dst = r < Q ? q_out + ((size_t)t * Q + r) * dk : k_cache + at + (planes ? 0 : (size_t)((r - Q) % maps) * dk);
    float inv = 1.0f;
    if (norm_eps >= 0.f) {
        float ss = 0.f;
        for (int d = lane; d < dk; d += 32) ss = fmaf(src[d], src[d], ss);
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)dk + norm_eps);
    }
    const int rot = 2 * half;
    for (int d = lane; d < dk; d += 32) {
        float x = src[d] * inv;
        if (gain) x *= gain[d];
        if (d < rot) {
            const int i = d < half ? d : d - half, e = d < half ? d + half : d - half;
            float y = src[e] * inv;
            if (gain) y *= gain[e];
            const float2 cs = table[(size_t)t * half + i];
            const float c = cs.x * magnitude, s = cs.y * magnitude;
            x = d < half ? x * c - y * s : x * c + y * s;
        }
        dst[d] = from_f32<T>(x);
    }
}

template <typename T, typename TO>
__global__ void __launch_bounds__(WARPS * 32)
masked_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, int row_stride, long long head_stride,
                        const int* __restrict__ block_table, int table_stride, const int* __restrict__ token_seq, const int* __restrict__ positions,
                        const int* __restrict__ token_list, TO* __restrict__ out, long long ldo, int heads, int kv_heads, int maps, int dk, int dv,
                        int page_size, long long page_stride, int num_pages, int window, int chunk, int keep_first, float scale, float softcap,
                        const float* __restrict__ sinks, float out_scale, int planes, int* status) {
    extern __shared__ float q_shared[];              // WARPS * dk
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = token_list ? token_list[blockIdx.x] : blockIdx.x;
    const int r = blockIdx.y * WARPS + warp;          // the query row: head * maps + map
    if (r >= heads * maps) return;                    // no block-wide barrier below
    const int h = r / maps, map = r % maps;
    const int g = planes ? h / (heads / kv_heads) * maps + map : h / (heads / kv_heads);        // the cache head
    const int key_at = planes ? 0 : map * dk;
    const int pos = positions[t];
    const int* table = block_table + (size_t)token_seq[t] * table_stride;
    float* qs = q_shared + warp * dk;
    const T* qrow = q + ((size_t)t * heads * maps + r) * dk;
    for (int d = lane; d < dk; d += 32) qs[d] = to_f32<T>(qrow[d]);
    __syncwarp();

    int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (chunk > 0) first = max(first, pos / chunk * chunk);
    const int kept_end = min(keep_first, first);      // keys 0 .. kept_end - 1 are seen beside those from `first` on
    float m = -INFINITY, l = 0.0f;
    float acc[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] = 0.0f;
    const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
    for (int part = 0; part < 2; ++part) {
        const int lo = part == 0 ? 0 : first, hi = part == 0 ? kept_end : pos + 1;      // keys lo .. hi - 1
        for (int base = lo; base < hi; base += 32) {
            const int kpos = base + lane;
            long long row_off = -1;
            if (kpos < hi) {
                const int page = table[kpos / page_size];
                if (page < 0 || page >= num_pages) atomicOr(status, EG_STATUS_BAD_PAGE);
                else row_off = (long long)page * page_stride + g * head_stride + (long long)(kpos % page_size) * row_stride;
            }
            float s = -INFINITY;
            if (row_off >= 0) {
                const T* krow = k_cache + row_off + key_at;
                float dot = 0.0f;
                for (int d = 0; d < dk; ++d) dot = fmaf(qs[d], to_f32<T>(krow[d]), dot);
                s = dot * scale;
                if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
            }
            const float m_new = fmaxf(m, warp_max(s));
            if (m_new == -INFINITY) continue;
            const float corr = expf(m - m_new);
            const float p = (row_off >= 0) ? expf(s - m_new) : 0.0f;
            l = l * corr + warp_sum(p);
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] *= corr;
            const int nkeys = min(32, hi - base);
            for (int j = 0; j < nkeys; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
                const long long off_j = __shfl_sync(0xffffffffu, row_off, j);
                if (off_j < 0) continue;
                const T* vrow = v_cache + off_j;
#pragma unroll
                for (int i = 0; i < MAX_PER_LANE; ++i) {
                    const int d = lane + 32 * i;
                    if (d < dv) acc[i] = fmaf(pj, to_f32<T>(vrow[d]), acc[i]);
                }
            }
            m = m_new;
        }
    }
    if (sinks) {
        const float sink = sinks[r];
        const float m_new = fmaxf(m, sink);
        const float corr = expf(m - m_new);
        l = l * corr + expf(sink - m_new);
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] *= corr;
    }
    TO* orow = out + (size_t)t * ldo + (size_t)r * dv;
    const float inv_l = l > 0.0f ? out_scale / l : 0.0f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) orow[d] = from_f32<TO>(acc[i] * inv_l);
    }
}

// one warp per (token, head): maps float32 [tokens, heads, 2, dv] -> out [tokens, ldo], head h at column h * dv
template <typename TO>
__global__ void __launch_bounds__(128) map_difference_kernel(const float* __restrict__ maps, TO* __restrict__ out, long long ldo, int tokens, int heads, int dv,
                                                             float lambda, float eps, float post) {
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)tokens * heads) return;
    const int t = (int)(w / heads), h = (int)(w % heads);
    const float* a = maps + ((size_t)t * heads + h) * 2 * dv;
    float o[MAX_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        o[i] = d < dv ? a[d] - lambda * a[dv + d] : 0.f;
        ss = fmaf(o[i], o[i], ss);
    }
    ss = warp_sum(ss);
    const float f = post / sqrtf(ss / (float)dv + eps);
    TO* orow = out + (size_t)t * ldo + (size_t)h * dv;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) orow[d] = from_f32<TO>(o[i] * f);
    }
}
}  // namespace

// proj float32 [tokens, ld]: heads * maps queries, kv_heads * maps keys (dk values each), kv_heads values (dv each), side by
// side.  table: cos/sin [tokens, rot_dims/2, 2] or null with rot_dims 0.  norm_eps < 0: no norm; q_gain / k_gain float32 [dk] or
// null.  k_cache null: nothing is stored.  q_out [tokens, heads * maps, dk].  planes: see above.
EG_API int eg_masked_attention_prepare(cudaStream_t stream, int dtype, const float* proj, long long ld, const float* table, int rot_dims, float magnitude,
                                       const int* slot_map, void* k_cache, void* v_cache, int row_stride, long long head_stride, int page_size,
                                       long long page_stride, long long pool_slots, void* q_out, int tokens, int heads, int kv_heads, int maps, int dk, int dv,
                                       float norm_eps, const float* q_gain, const float* k_gain, int planes, int* status) {
    if (tokens <= 0) return 0;
    if (planes && dk != dv) return (int)cudaErrorInvalidValue;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > dk || (rot_dims > 0 && !table) || maps < 1 || kv_heads <= 0 || heads % kv_heads) return (int)cudaErrorInvalidValue;
    const long long warps = (long long)tokens * ((heads + kv_heads) * maps + kv_heads);
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    if (dtype == EG_BF16)
        masked_prepare_kernel<bf16><<<blocks, 128, 0, stream>>>(proj, ld, (const float2*)table, rot_dims / 2, magnitude, slot_map, (bf16*)k_cache, (bf16*)v_cache,
                                                                row_stride, head_stride, page_size, page_stride, pool_slots, (bf16*)q_out, tokens, heads, kv_heads,
                                                                maps, dk, dv, norm_eps, q_gain, k_gain, planes, status);
    else
        masked_prepare_kernel<float><<<blocks, 128, 0, stream>>>(proj, ld, (const float2*)table, rot_dims / 2, magnitude, slot_map, (float*)k_cache, (float*)v_cache,
                                                                 row_stride, head_stride, page_size, page_stride, pool_slots, (float*)q_out, tokens, heads, kv_heads,
                                                                 maps, dk, dv, norm_eps, q_gain, k_gain, planes, status);
    return eg_launch_status();
}

// q [tokens, heads * maps, dk] in dtype; out [tokens, ldo] in out_dtype (the cache's dtype, or float32) with row r at column
// r * dv.  token_list: the tokens to work on (num_tokens of them), or null for all.  sinks: float32 [heads * maps] or null.
// Returns cudaErrorInvalidValue for sizes it does not take.
EG_API int eg_masked_attention(cudaStream_t stream, int dtype, const void* q, const void* k_cache, const void* v_cache, int row_stride, long long head_stride,
                               const int* block_table, int table_stride, const int* token_seq, const int* positions, const int* token_list, void* out,
                               int out_dtype, long long ldo, int num_tokens, int heads, int kv_heads, int maps, int dk, int dv, int page_size,
                               long long page_stride, int num_pages, int window, int chunk, int keep_first, float scale, float softcap, const float* sinks,
                               float out_scale, int planes, int* status) {
    if (num_tokens <= 0) return 0;
    if (dv > 32 * MAX_PER_LANE || dv <= 0 || dk <= 0 || dk > 4096 || kv_heads <= 0 || heads % kv_heads || maps < 1 || keep_first < 0) return (int)cudaErrorInvalidValue;
    if (dtype == EG_F32 && out_dtype != EG_F32) return (int)cudaErrorInvalidValue;
    dim3 grid(num_tokens, (heads * maps + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * dk * sizeof(float);
#define EG_MASKED(T, TO)                                                                                                                                     \
    masked_attention_kernel<T, TO><<<grid, WARPS * 32, smem, stream>>>((const T*)q, (const T*)k_cache, (const T*)v_cache, row_stride, head_stride, block_table, \
                                                                       table_stride, token_seq, positions, token_list, (TO*)out, ldo, heads, kv_heads, maps, dk, \
                                                                       dv, page_size, page_stride, num_pages, window, chunk, keep_first, scale, softcap, sinks,  \
                                                                       out_scale, planes, status)
    if (dtype == EG_BF16 && out_dtype == EG_BF16) EG_MASKED(bf16, bf16);
    else if (dtype == EG_BF16) EG_MASKED(bf16, float);
    else EG_MASKED(float, float);
#undef EG_MASKED
    return eg_launch_status();
}

// maps float32 [tokens, heads, 2, dv]: out[t, h] = post * o / sqrt(mean(o^2) + eps) with o = maps[t, h, 0] - lambda * maps[t, h, 1]
EG_API int eg_attention_map_difference(cudaStream_t stream, const float* maps, void* out, int out_dtype, long long ldo, int tokens, int heads, int dv,
                                       float lambda, float eps, float post) {
    if (tokens <= 0) return 0;
    if (dv <= 0 || dv > 32 * MAX_PER_LANE) return (int)cudaErrorInvalidValue;
    const long long warps = (long long)tokens * heads;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    if (out_dtype == EG_BF16) map_difference_kernel<bf16><<<blocks, 128, 0, stream>>>(maps, (bf16*)out, ldo, tokens, heads, dv, lambda, eps, post);
    else map_difference_kernel<float><<<blocks, 128, 0, stream>>>(maps, (float*)out, ldo, tokens, heads, dv, lambda, eps, post);
    return eg_launch_status();
}
