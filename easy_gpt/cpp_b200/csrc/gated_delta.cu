// The gated delta rule: per head a matrix S [dk, dv] (float32, in the request's state slot) that every token lets decay,
// corrects towards its value along its key, and reads with its query:
//
//   q^ = q / sqrt(|q|^2 + unit_eps) * dk^(-1/2),  k^ = k / sqrt(|k|^2 + unit_eps)          (per key head, float32)
//   beta = sigmoid(b),  g = exp(-exp(A_log) * softplus(a + dt_bias))                          (per head, float32)
//   S <- g S;  u = beta (v - S^T k^);  S <- S + k^ u^T;  o = S^T q^
//   y = o / sqrt(mean(o^2) + eps) * w * silu(z)                                               (per head over dv)
//
// q, k, v are the convolved and activated projections (float32 [tokens, ...]), b, a and z columns of the projection's
// float32 output.  Head h reads key head h / (heads / kv_heads).
//
// A kernel over all tokens first makes the unit vectors and the per-token numbers (beta, g, k^ . q^).  Then one block per
// (head, batch entry, slice of the head's columns: the columns of S do not depend on one another).  Column j of S belongs
// to P neighbouring lanes, each with R = ceil(dk / P) of its rows in registers for the entry's whole run of tokens, so a
// token costs two dot products over the old S (with k^ and with q^, independent of each other: o = g S_old^T q^ +
// u (k^ . q^)), a few shuffles and one update per element.  The block walks the entry in tiles of tokens that arrive in
// shared memory by asynchronous copies, the next tile's behind this one's steps; outputs are normed per head and gated by
// the block itself where it holds whole heads, else by a kernel behind.  The slot keeps S as [head, dv, dk], so that a
// thread's rows are neighbours in memory.  The order of every sum depends on the sizes alone.
//
// A second form has a decay per head AND key channel, g [dk]: S <- diag(g) S (the rows of S decay each at its own rate), the
// rest as above.  With S' = diag(g) S_old:  u = beta (v - S'^T k^),  o = S'^T q^ + u (k^ . q^), so a token costs the same two
// dot products, over the decayed rows; the tile's decays are staged beside its keys and queries.  Its per-token numbers come
// from buffers of their own (beta's logits, the decays' step-size logits, the output gate), the gate is a sigmoid or a silu,
// and the output may carry a factor.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// exp(x) for x <= 0, with the last addition the only rounding that counts: a state that decays slowly is multiplied by
// thousands of such factors in a row, and an error with a sign of its own would add up over a long sequence.
__device__ __forceinline__ float decay_exp(float x) {
    if (x < -104.0f) return 0.0f;
    const float k = rintf(x * 1.442695041f);
    float r = fmaf(k, -0.693145751953125f, x);
    r = fmaf(k, -1.428606765330187e-06f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float e = 1.0f + fmaf(r * r, p, r);
    const int ki = (int)k;
    if (ki >= -125) return __int_as_float(__float_as_int(e) + (ki << 23));
    return __int_as_float(__float_as_int(e) + ((ki + 100) << 23)) * 7.888609052210118e-31f;
}

constexpr int TILE = 16;        // tokens staged at a time
constexpr int PAD = 4;          // floats between the parts' rows of a staged key or query: the parts' 16-byte loads then hit different banks

__device__ __forceinline__ void copy_async_16(float* smem_dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_4(float* smem_dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}

// Before the recurrence, for all tokens at once: a warp per (token, key head) makes the head's query and key unit vectors in
// place (the query also times dk^(-1/2)) and leaves, for every head of its group, (beta, g, k^ . q^) in aux [tokens, heads, 4].
__global__ void __launch_bounds__(128) delta_prepare_kernel(float* __restrict__ qkv, long long ldq, int q_col, int k_col, const float* __restrict__ proj,
                                                            long long ldp, int b_col, int a_col, const float* __restrict__ a_log,
                                                            const float* __restrict__ dt_bias, float* __restrict__ aux, int tokens, int heads,
                                                            int kv_heads, int dk, float unit_eps) {
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)tokens * kv_heads) return;
    const int t = (int)(w / kv_heads), g = (int)(w % kv_heads);
    float* q = qkv + (size_t)t * ldq + q_col + (size_t)g * dk;
    float* k = qkv + (size_t)t * ldq + k_col + (size_t)g * dk;
    float kk = 0.f, qq = 0.f, kq = 0.f;
    for (int d = lane; d < dk; d += 32) {
        const float a = k[d], b = q[d];
        kk = fmaf(a, a, kk);
        qq = fmaf(b, b, qq);
        kq = fmaf(a, b, kq);
    }
    kk = warp_sum(kk);
    qq = warp_sum(qq);
    kq = warp_sum(kq);
    const float ik = 1.0f / sqrtf(kk + unit_eps), iq = (1.0f / sqrtf((float)dk)) / sqrtf(qq + unit_eps);
    for (int d = lane; d < dk; d += 32) {
        k[d] *= ik;
        q[d] *= iq;
    }
    const int per = heads / kv_heads;
    const float* row = proj + (size_t)t * ldp;
    for (int i = lane; i < per; i += 32) {
        const int head = g * per + i;
        float* out = aux + ((size_t)t * heads + head) * 4;
        out[0] = 1.0f / (1.0f + expf(-row[b_col + head]));
        out[1] = decay_exp(-expf(a_log[head]) * softplus_f(row[a_col + head] + dt_bias[head]));
        out[2] = kq * ik * iq;
        out[3] = 0.f;
    }
}

// The same for the form with a decay per key channel: unit vectors and k^ . q^ per key head, beta per head, and the decays
// g = exp(-exp(A_log[head]) * softplus(a + dt_bias)) written over their logits a in `decay` [tokens, ldg] (heads x dk, dt_bias alike).
__global__ void __launch_bounds__(128) delta_prepare_channel_kernel(float* __restrict__ qkv, long long ldq, int q_col, int k_col, const float* __restrict__ b,
                                                                    long long ldb, int b_col, float* __restrict__ decay, long long ldg,
                                                                    const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                                                    float* __restrict__ aux, int tokens, int heads, int kv_heads, int dk, float unit_eps) {
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)tokens * kv_heads) return;
    const int t = (int)(w / kv_heads), g = (int)(w % kv_heads);
    float* q = qkv + (size_t)t * ldq + q_col + (size_t)g * dk;
    float* k = qkv + (size_t)t * ldq + k_col + (size_t)g * dk;
    float kk = 0.f, qq = 0.f, kq = 0.f;
    for (int d = lane; d < dk; d += 32) {
        const float a = k[d], c = q[d];
        kk = fmaf(a, a, kk);
        qq = fmaf(c, c, qq);
        kq = fmaf(a, c, kq);
    }
    kk = warp_sum(kk);
    qq = warp_sum(qq);
    kq = warp_sum(kq);
    const float ik = 1.0f / sqrtf(kk + unit_eps), iq = (1.0f / sqrtf((float)dk)) / sqrtf(qq + unit_eps);
    for (int d = lane; d < dk; d += 32) {
        k[d] *= ik;
        q[d] *= iq;
    }
    const int per = heads / kv_heads;
    for (int i = 0; i < per; ++i) {
        const int head = g * per + i;
        const float rate = -expf(a_log[head]);
        float* row = decay + (size_t)t * ldg + (size_t)head * dk;
        for (int d = lane; d < dk; d += 32) row[d] = decay_exp(rate * softplus_f(row[d] + dt_bias[(size_t)head * dk + d]));
        if (lane == 0) {
            float* out = aux + ((size_t)t * heads + head) * 4;
            out[0] = 1.0f / (1.0f + expf(-b[(size_t)t * ldb + b_col + head]));
            out[1] = 1.0f;
            out[2] = kq * ik * iq;
            out[3] = 0.f;
        }
    }
}

// grid (heads, entries, column slices): a block holds `cols` columns of a head's S.  With o_raw the block leaves its columns
// of o there (float32) and the norm over the head's columns is another kernel's; without, the block holds whole heads and
// norms and gates its outputs itself.  The tiles' keys, queries, values and (beta, g, k . q) come by asynchronous copies into
// one of two buffers, the next tile's while this one's steps run.
// CH: the form with a decay per key channel (`decay` [tokens, ldg], heads x dk), staged beside keys and queries.
template <typename TO, int R, int P, bool CH>
__global__ void __launch_bounds__(1024) gated_delta_kernel(const float* __restrict__ qkv, long long ldq, int q_col, int k_col, int v_col,
                                                           const float* __restrict__ proj, long long ldp, int z_col, const float* __restrict__ aux,
                                                           const float* __restrict__ norm_w, float* __restrict__ state, long long slot_floats,
                                                           long long state_offset, const int* __restrict__ seq_starts,
                                                           const int* __restrict__ seq_slots, TO* __restrict__ y, long long ldy,
                                                           float* __restrict__ o_raw, int cols, int heads, int kv_heads, int dk, int dv, float eps,
                                                           int wide, const float* __restrict__ decay, long long ldg, int gate_sigmoid, float out_scale) {
    extern __shared__ __align__(16) float smem[];
    constexpr int RS = R + PAD, DKS = RS * P;       // a part's stride, a staged row's length (rows beyond dk hold zeros)
    constexpr int VECS = CH ? 3 : 2;                // staged vectors of dk values a token: key, query and, with CH, decay
    const int vcols = (cols + 3) & ~3;
    const int stage_floats = TILE * (VECS * DKS + vcols + 4);
    float* s_o = smem + 2 * stage_floats;           // [TILE, cols]
    const int head = blockIdx.x, seq = blockIdx.y, j0 = blockIdx.z * cols;
    const int kvh = head / (heads / kv_heads);
    const int start = seq_starts[seq], count = seq_starts[seq + 1] - start;
    const int jl = threadIdx.x / P, j = j0 + jl, part = threadIdx.x % P;
    const int width = min(cols, dv - j0);           // this block's columns
    const bool active = jl < width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    float* S = state + (size_t)seq_slots[seq] * slot_floats + state_offset + ((size_t)head * dv + (active ? j : 0)) * dk;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = part * R + r;
        s[r] = (active && row < dk) ? S[row] : 0.f;
    }
    for (int i = threadIdx.x; i < 2 * stage_floats; i += blockDim.x) smem[i] = 0.f;      // rows beyond dk stay zero
    __syncthreads();
    // tile `ti` into buffer `b`: 16-byte pieces where every row starts on a 16-byte boundary (wide), else value by value
    auto fetch = [&](int ti, int b) {
        const int t0 = ti * TILE, n = min(TILE, count - t0);
        float* sk = smem + b * stage_floats;
        float* sq = sk + TILE * DKS;
        float* sg = sq + TILE * DKS;                // with CH only
        float* sv = sk + VECS * TILE * DKS;
        float* sa = sv + TILE * vcols;
        if (wide) {
            const int pieces = dk / 4;
            for (int i = threadIdx.x; i < n * pieces; i += blockDim.x) {
                const int t = i / pieces, d = (i % pieces) * 4;
                const float* row = qkv + (size_t)(start + t0 + t) * ldq;
                const int at = t * DKS + (d / R) * RS + d % R;
                copy_async_16(sk + at, row + k_col + kvh * dk + d);
                copy_async_16(sq + at, row + q_col + kvh * dk + d);
                if (CH) copy_async_16(sg + at, decay + (size_t)(start + t0 + t) * ldg + (size_t)head * dk + d);
            }
            const int vp = width / 4;
            for (int i = threadIdx.x; i < n * vp; i += blockDim.x) {
                const int t = i / vp, d = (i % vp) * 4;
                copy_async_16(sv + t * vcols + d, qkv + (size_t)(start + t0 + t) * ldq + v_col + head * dv + j0 + d);
            }
            for (int t = threadIdx.x; t < n; t += blockDim.x) copy_async_16(sa + t * 4, aux + ((size_t)(start + t0 + t) * heads + head) * 4);
        } else {
            for (int i = threadIdx.x; i < n * dk; i += blockDim.x) {
                const int t = i / dk, d = i % dk;
                const float* row = qkv + (size_t)(start + t0 + t) * ldq;
                const int at = t * DKS + (d / R) * RS + d % R;
                copy_async_4(sk + at, row + k_col + kvh * dk + d);
                copy_async_4(sq + at, row + q_col + kvh * dk + d);
                if (CH) copy_async_4(sg + at, decay + (size_t)(start + t0 + t) * ldg + (size_t)head * dk + d);
            }
            for (int i = threadIdx.x; i < n * width; i += blockDim.x) {
                const int t = i / width, d = i % width;
                copy_async_4(sv + t * vcols + d, qkv + (size_t)(start + t0 + t) * ldq + v_col + head * dv + j0 + d);
            }
            for (int i = threadIdx.x; i < n * 3; i += blockDim.x)
                copy_async_4(sa + (i / 3) * 4 + i % 3, aux + ((size_t)(start + t0 + i / 3) * heads + head) * 4 + i % 3);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    const int tiles = (count + TILE - 1) / TILE;
    if (tiles > 0) fetch(0, 0);
    for (int ti = 0; ti < tiles; ++ti) {
        const int t0 = ti * TILE, n = min(TILE, count - t0);
        if (ti + 1 < tiles) {
            fetch(ti + 1, (ti + 1) & 1);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();                            // this tile has arrived; the tile before is done with s_o
        const float* s_k = smem + (ti & 1) * stage_floats;
        const float* s_q = s_k + TILE * DKS;
        const float* s_g = s_q + TILE * DKS;        // with CH only
        const float* s_v = s_k + VECS * TILE * DKS;
        const float* s_a = s_v + TILE * vcols;
        auto step = [&](int t) {
            const float4* kt = reinterpret_cast<const float4*>(s_k + t * DKS + part * RS);
            const float4* qt = reinterpret_cast<const float4*>(s_q + t * DKS + part * RS);
            float kv[R];
            float sk0 = 0.f, sk1 = 0.f, sq0 = 0.f, sq1 = 0.f;
            if (CH) {                                   // the rows decay first, each at its own rate; the sums run over the decayed rows
                const float4* gt = reinterpret_cast<const float4*>(s_g + t * DKS + part * RS);
#pragma unroll
                for (int r = 0; r < R; r += 4) {
                    const float4 c = gt[r / 4];
                    s[r] *= c.x; s[r + 1] *= c.y; s[r + 2] *= c.z; s[r + 3] *= c.w;
                }
            }
#pragma unroll
            for (int r = 0; r < R; r += 4) {
                const float4 a = kt[r / 4], b = qt[r / 4];
                kv[r] = a.x; kv[r + 1] = a.y; kv[r + 2] = a.z; kv[r + 3] = a.w;
                sk0 = fmaf(s[r], a.x, sk0); sk1 = fmaf(s[r + 1], a.y, sk1); sk0 = fmaf(s[r + 2], a.z, sk0); sk1 = fmaf(s[r + 3], a.w, sk1);
                sq0 = fmaf(s[r], b.x, sq0); sq1 = fmaf(s[r + 1], b.y, sq1); sq0 = fmaf(s[r + 2], b.z, sq0); sq1 = fmaf(s[r + 3], b.w, sq1);
            }
            float sk = sk0 + sk1, sq = sq0 + sq1;
#pragma unroll
            for (int o = 1; o < P; o <<= 1) {
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
            }
            const float4 bgk = *reinterpret_cast<const float4*>(s_a + t * 4);      // beta, g, k . q
            const float g = CH ? 1.0f : bgk.y;
            const float u = bgk.x * ((active ? s_v[t * vcols + jl] : 0.f) - g * sk);
#pragma unroll
            for (int r = 0; r < R; ++r) s[r] = fmaf(kv[r], u, g * s[r]);
            if (active && part == 0) s_o[t * cols + jl] = fmaf(g, sq, u * bgk.z);
        };
        if (n == TILE) {                            // a whole tile: unrolled, so that the loads of the next tokens go out ahead of their steps
#pragma unroll 4
            for (int t = 0; t < TILE; ++t) step(t);
        } else {
            for (int t = 0; t < n; ++t) step(t);
        }
        __syncthreads();                            // the tile's outputs are complete; its buffer may be filled again
        if (o_raw) {
            for (int i = threadIdx.x; i < n * width; i += blockDim.x) {
                const int t = i / width, d = i % width;
                o_raw[(size_t)(start + t0 + t) * ((size_t)heads * dv) + head * dv + j0 + d] = s_o[t * cols + d];
            }
            continue;
        }
        // y = o / rms(o) * w * silu(z), a warp per token
        for (int t = warp; t < n; t += warps) {
            float ss = 0.f;
            for (int d = lane; d < dv; d += 32) ss = fmaf(s_o[t * cols + d], s_o[t * cols + d], ss);
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
            const float* z = proj + (size_t)(start + t0 + t) * ldp + z_col + head * dv;
            TO* out = y + (size_t)(start + t0 + t) * ldy + head * dv;
            for (int d = lane; d < dv; d += 32)
                out[d] = from_f32<TO>(s_o[t * cols + d] * inv * norm_w[d] * (gate_sigmoid ? 1.0f / (1.0f + expf(-z[d])) : silu_f(z[d])) * out_scale);
        }
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = part * R + r;
            if (row < dk) S[row] = s[r];
        }
    }
}

// y = o / rms(o) * w * silu(z) per (token, head), a warp each: behind a recurrence whose blocks held slices of a head
template <typename TO>
__global__ void delta_output_kernel(const float* __restrict__ o_raw, const float* __restrict__ proj, long long ldp, int z_col,
                                    const float* __restrict__ norm_w, TO* __restrict__ y, long long ldy, int tokens, int heads, int dv, float eps,
                                    int gate_sigmoid, float out_scale) {
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)tokens * heads) return;
    const int t = (int)(w / heads), head = (int)(w % heads);
    const float* o = o_raw + ((size_t)t * heads + head) * dv;
    float ss = 0.f;
    for (int d = lane; d < dv; d += 32) ss = fmaf(o[d], o[d], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    const float* z = proj + (size_t)t * ldp + z_col + head * dv;
    TO* out = y + (size_t)t * ldy + head * dv;
    for (int d = lane; d < dv; d += 32) out[d] = from_f32<TO>(o[d] * inv * norm_w[d] * (gate_sigmoid ? 1.0f / (1.0f + expf(-z[d])) : silu_f(z[d])) * out_scale);
}

// what the form with a decay per key channel brings beside the common arguments (decay null: the form with one decay a head)
struct ChannelForm {
    const float* b = nullptr;       // beta's logits [tokens, ldb], head h at b_col + h
    long long ldb = 0;
    float* decay = nullptr;         // [tokens, ldg], heads x dk: the decays' logits on entry, the decays after the preparation
    long long ldg = 0;
    int gate_sigmoid = 0;           // the output gate is sigmoid(z) instead of silu(z)
    float out_scale = 1.0f;
};

template <typename TO, int R, int P, bool CH>
int launch_delta(cudaStream_t stream, float* qkv, long long ldq, int q_col, int k_col, int v_col, const float* proj, long long ldp, int b_col,
                 int a_col, int z_col, const float* a_log, const float* dt_bias, const float* norm_w, float* state, long long slot_floats,
                 long long state_offset, const int* seq_starts, const int* seq_slots, void* y, long long ldy, float* aux, float* o_raw, int slices,
                 int tokens, int num_seqs, int heads, int kv_heads, int dk, int dv, float unit_eps, float eps, const ChannelForm& cf) {
    // columns per block: whole warps of them (32 / P columns a warp), and a multiple of four so that the slices' values start on 16-byte boundaries
    const int per_warp = 32 / P < 4 ? 4 : 32 / P;
    const int most_cols = 1024 / P / per_warp * per_warp;       // a block has at most 1024 threads
    if (!o_raw) slices = 1;
    int cols = (dv + slices - 1) / slices;
    cols = std::min((cols + per_warp - 1) / per_warp * per_warp, most_cols);
    slices = (dv + cols - 1) / cols;
    if (slices > 1 && !o_raw) return (int)cudaErrorInvalidValue;  // a head that no single block holds needs the buffer for its raw outputs
    if (slices == 1) o_raw = nullptr;
    const int threads = cols * P;
    const int vcols = (cols + 3) & ~3;
    const size_t smem = ((size_t)2 * TILE * ((CH ? 3 : 2) * (R + PAD) * P + vcols + 4) + (size_t)TILE * cols) * sizeof(float);
    if (threads > 1024 || smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    auto kernel = gated_delta_kernel<TO, R, P, CH>;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const long long prep = (long long)tokens * kv_heads;
    if (CH)
        delta_prepare_channel_kernel<<<(unsigned)((prep + 3) / 4), 128, 0, stream>>>(qkv, ldq, q_col, k_col, cf.b, cf.ldb, b_col, cf.decay, cf.ldg, a_log, dt_bias,
                                                                                     aux, tokens, heads, kv_heads, dk, unit_eps);
    else
        delta_prepare_kernel<<<(unsigned)((prep + 3) / 4), 128, 0, stream>>>(qkv, ldq, q_col, k_col, proj, ldp, b_col, a_col, a_log, dt_bias, aux, tokens, heads,
                                                                             kv_heads, dk, unit_eps);
    // 16-byte copies need every copied row to start on a 16-byte boundary
    const int wide = dk % 4 == 0 && dv % 4 == 0 && ldq % 4 == 0 && q_col % 4 == 0 && k_col % 4 == 0 && v_col % 4 == 0 && (uintptr_t)qkv % 16 == 0 &&
                     (uintptr_t)aux % 16 == 0 && (!CH || (cf.ldg % 4 == 0 && (uintptr_t)cf.decay % 16 == 0));
    kernel<<<dim3(heads, num_seqs, slices), threads, smem, stream>>>(qkv, ldq, q_col, k_col, v_col, proj, ldp, z_col, aux, norm_w, state, slot_floats,
                                                                     state_offset, seq_starts, seq_slots, (TO*)y, ldy, o_raw, cols, heads, kv_heads, dk, dv,
                                                                     eps, wide, cf.decay, cf.ldg, cf.gate_sigmoid, cf.out_scale);
    if (o_raw) {
        const long long warps = (long long)tokens * heads;
        delta_output_kernel<TO><<<(unsigned)((warps + 3) / 4), 128, 0, stream>>>(o_raw, proj, ldp, z_col, norm_w, (TO*)y, ldy, tokens, heads, dv, eps,
                                                                                 cf.gate_sigmoid, cf.out_scale);
    }
    return eg_launch_status();
}

template <typename TO>
int dispatch_delta(int R, int P, cudaStream_t stream, float* qkv, long long ldq, int q_col, int k_col, int v_col, const float* proj, long long ldp,
                   int b_col, int a_col, int z_col, const float* a_log, const float* dt_bias, const float* norm_w, float* state, long long slot_floats,
                   long long state_offset, const int* seq_starts, const int* seq_slots, void* y, long long ldy, float* aux, float* o_raw, int slices,
                   int tokens, int num_seqs, int heads, int kv_heads, int dk, int dv, float unit_eps, float eps, const ChannelForm& cf = ChannelForm()) {
#define EG_DELTA(RR, PP)                                                                                                                                  \
    if (R == RR && P == PP)                                                                                                                               \
        return cf.decay ? launch_delta<TO, RR, PP, true>(stream, qkv, ldq, q_col, k_col, v_col, proj, ldp, b_col, a_col, z_col, a_log, dt_bias, norm_w, state,  \
                                                         slot_floats, state_offset, seq_starts, seq_slots, y, ldy, aux, o_raw, slices, tokens, num_seqs, heads,  \
                                                         kv_heads, dk, dv, unit_eps, eps, cf)                                                                     \
                        : launch_delta<TO, RR, PP, false>(stream, qkv, ldq, q_col, k_col, v_col, proj, ldp, b_col, a_col, z_col, a_log, dt_bias, norm_w, state, \
                                                          slot_floats, state_offset, seq_starts, seq_slots, y, ldy, aux, o_raw, slices, tokens, num_seqs, heads, \
                                                          kv_heads, dk, dv, unit_eps, eps, cf)
    EG_DELTA(4, 4);
    EG_DELTA(8, 4);
    EG_DELTA(8, 8);
    EG_DELTA(8, 16);
    EG_DELTA(8, 32);
    EG_DELTA(4, 16);
    EG_DELTA(4, 32);
#undef EG_DELTA
    return (int)cudaErrorInvalidValue;
}
}  // namespace

// How a head's rows are spread for these sizes: P lanes a column with R rows each (R * P >= dk); 0 if the kernel does
// not take the sizes.  Few rows a lane and many lanes a column: a token's work is a chain of dependent steps, and a
// scheduler hides one warp's waits only behind other warps (measured on B200 with 128 x 128 states, 2,048 tokens: 16 rows
// a lane, 512 warps in all, 640 cycles a token, of which 92% waits).
EG_API int eg_gated_delta_plan(int dk, int dv, int* rows_per_lane, int* lanes) {
    if (dk <= 0 || dv <= 0 || dk > 256 || dv > 4096) return 0;
    *rows_per_lane = dk <= 16 ? 4 : 8;
    *lanes = dk <= 32 ? 4 : dk <= 64 ? 8 : dk <= 128 ? 16 : 32;
    static const int few = getenv("EASY_GPT_DELTA_ROWS") ? atoi(getenv("EASY_GPT_DELTA_ROWS")) : 0;      // for measurements: 4 rows a lane
    if (few == 4 && dk > 32 && dk <= 128) {
        *rows_per_lane = 4;
        *lanes = dk <= 64 ? 16 : 32;
    }
    return 1;
}

// qkv float32 [tokens, ldq]: convolved, activated queries (key heads x dk at q_col), keys (k_col) and values (heads x dv at
// v_col); queries and keys are made unit vectors in place.  proj float32 [tokens, ldp]: the projection's output with b
// (heads) at b_col, a (heads) at a_col and the output gate z (heads x dv) at z_col.  aux: float32 [tokens, heads, 4] of
// scratch.  state: the requests' slots; S of a request lies state_offset floats into its slot, as [heads, dv, dk].
// y [tokens, ldy] in y_dtype.  slices > 1 (with o_raw, float32 [tokens, heads * dv]): a head's columns are dealt to that
// many blocks, for steps with few (entry, head) pairs, and the outputs are normed by a kernel behind.
EG_API int eg_gated_delta(cudaStream_t stream, float* qkv, long long ldq, int q_col, int k_col, int v_col, const float* proj, long long ldp, int b_col,
                          int a_col, int z_col, const float* a_log, const float* dt_bias, const float* norm_w, float* state, long long slot_floats,
                          long long state_offset, const int* seq_starts, const int* seq_slots, void* y, int y_dtype, long long ldy, float* aux,
                          float* o_raw, int slices, int tokens, int num_seqs, int heads, int kv_heads, int dk, int dv, float unit_eps, float eps) {
    if (num_seqs <= 0 || tokens <= 0) return 0;
    int R = 0, P = 0;
    if (kv_heads <= 0 || heads % kv_heads || !eg_gated_delta_plan(dk, dv, &R, &P) || slices < 1 || !aux) return (int)cudaErrorInvalidValue;
    if (y_dtype == EG_BF16)
        return dispatch_delta<bf16>(R, P, stream, qkv, ldq, q_col, k_col, v_col, proj, ldp, b_col, a_col, z_col, a_log, dt_bias, norm_w, state, slot_floats,
                                    state_offset, seq_starts, seq_slots, y, ldy, aux, o_raw, slices, tokens, num_seqs, heads, kv_heads, dk, dv, unit_eps, eps);
    return dispatch_delta<float>(R, P, stream, qkv, ldq, q_col, k_col, v_col, proj, ldp, b_col, a_col, z_col, a_log, dt_bias, norm_w, state, slot_floats,
                                 state_offset, seq_starts, seq_slots, y, ldy, aux, o_raw, slices, tokens, num_seqs, heads, kv_heads, dk, dv, unit_eps, eps);
}

// The form with a decay per head and key channel.  qkv, aux, state, y, o_raw and slices as above.  b float32 [tokens, ldb] holds
// beta's logits (head h at b_col + h); decay float32 [tokens, ldg] holds, heads x dk, the logits a of the decays on entry and
// the decays g = exp(-exp(A_log[head]) softplus(a + dt_bias)) afterwards (dt_bias [heads x dk]); z float32 [tokens, ldz] the
// output gate's logits (heads x dv); the gate is sigmoid(z) (gate_sigmoid) or silu(z); y carries the factor out_scale.
EG_API int eg_gated_delta_channel(cudaStream_t stream, float* qkv, long long ldq, int q_col, int k_col, int v_col, const float* b, long long ldb, int b_col,
                                  float* decay, long long ldg, const float* z, long long ldz, const float* a_log, const float* dt_bias, const float* norm_w,
                                  float* state, long long slot_floats, long long state_offset, const int* seq_starts, const int* seq_slots, void* y,
                                  int y_dtype, long long ldy, float* aux, float* o_raw, int slices, int tokens, int num_seqs, int heads, int kv_heads, int dk,
                                  int dv, float unit_eps, float eps, int gate_sigmoid, float out_scale) {
    if (num_seqs <= 0 || tokens <= 0) return 0;
    int R = 0, P = 0;
    if (kv_heads <= 0 || heads % kv_heads || !eg_gated_delta_plan(dk, dv, &R, &P) || slices < 1 || !aux || !decay || !b || !z) return (int)cudaErrorInvalidValue;
    ChannelForm cf;
    cf.b = b;
    cf.ldb = ldb;
    cf.decay = decay;
    cf.ldg = ldg;
    cf.gate_sigmoid = gate_sigmoid;
    cf.out_scale = out_scale;
    if (y_dtype == EG_BF16)
        return dispatch_delta<bf16>(R, P, stream, qkv, ldq, q_col, k_col, v_col, z, ldz, b_col, 0, 0, a_log, dt_bias, norm_w, state, slot_floats, state_offset,
                                    seq_starts, seq_slots, y, ldy, aux, o_raw, slices, tokens, num_seqs, heads, kv_heads, dk, dv, unit_eps, eps, cf);
    return dispatch_delta<float>(R, P, stream, qkv, ldq, q_col, k_col, v_col, z, ldz, b_col, 0, 0, a_log, dt_bias, norm_w, state, slot_floats, state_offset,
                                 seq_starts, seq_slots, y, ldy, aux, o_raw, slices, tokens, num_seqs, heads, kv_heads, dk, dv, unit_eps, eps, cf);
}
