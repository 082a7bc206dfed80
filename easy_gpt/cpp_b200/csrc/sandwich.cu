// Pieces of a layer whose branches are normed on both sides, x <- x + norm_b(f(shift(norm_a(x)))):
//
//   token shift      out[t] = h[t] + (h[t-1] - h[t]) * mu            h[t-1]: the row before t in its request; the request's
//                                                                    slot holds the last row of earlier steps (zeros at the start)
//   norm + shift     the same with h = gain * x / sqrt(mean(x^2) + eps) computed here from the float32 stream
//   norm and add     x[t] += gain * y[t] / sqrt(mean(y[t]^2) + eps)  a branch's output joins the stream through its norm
//   xIELU            a(z) = ap z^2 + z / 2 (z > 0),  an (e^z - 1 - z) + z / 2 (z <= 0)
//   scaled gather    x[t] = scale * table[id[t]]
//
// Sums, roots and divisions are float32.  The slot is read by the block of an entry's first token alone, which then
// stores the entry's last row in it: read and write of a slot sit in one thread each, so no block waits for another.
#include "common.cuh"

namespace {

// inverse root mean square of `row` (+ nothing): every thread gets it
__device__ __forceinline__ float inv_rms(const float* __restrict__ row, int hidden, float eps, float* scratch) {
    float ss = 0.f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) ss = fmaf(row[j], row[j], ss);
    ss = block_sum(ss, scratch);
    return 1.0f / sqrtf(ss / (float)hidden + eps);
}

template <typename TO>
__global__ void token_shift_kernel(const float* __restrict__ rows, const float* __restrict__ mu, float* __restrict__ state, long long slot_floats,
                                   const int* __restrict__ token_seq, const int* __restrict__ seq_starts, const int* __restrict__ seq_slots,
                                   TO* __restrict__ out, int hidden) {
    const int t = blockIdx.x, seq = token_seq[t], start = seq_starts[seq];
    const bool first = t == start;
    float* slot = state + (size_t)seq_slots[seq] * slot_floats;
    const float* prev = first ? slot : rows + (size_t)(t - 1) * hidden;
    const float* x = rows + (size_t)t * hidden;
    const float* last = rows + (size_t)(seq_starts[seq + 1] - 1) * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float v = x[j], p = prev[j];
        out[(size_t)t * hidden + j] = from_f32<TO>(fmaf(p - v, mu[j], v));
        if (first) slot[j] = last[j];
    }
}

template <typename TO>
__global__ void rmsnorm_shift_kernel(const float* __restrict__ stream, const float* __restrict__ gain, float eps, const float* __restrict__ mu,
                                     float* __restrict__ state, long long slot_floats, const int* __restrict__ token_seq,
                                     const int* __restrict__ seq_starts, const int* __restrict__ seq_slots, TO* __restrict__ out, int hidden) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, seq = token_seq[t], start = seq_starts[seq];
    const bool first = t == start;
    float* slot = state + (size_t)seq_slots[seq] * slot_floats;
    const float* x = stream + (size_t)t * hidden;
    const float inv = inv_rms(x, hidden, eps, scratch);
    // the row in front: the stream's row t-1 normed again here, or the slot's row; the first token's block also norms the
    // entry's last row for the slot
    const float* other = stream + (size_t)(first ? seq_starts[seq + 1] - 1 : t - 1) * hidden;
    const float inv_other = (first && other == x) ? inv : inv_rms(other, hidden, eps, scratch);
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float g = gain[j];
        const float v = g * (x[j] * inv);
        const float o = g * (other[j] * inv_other);
        const float p = first ? slot[j] : o;
        out[(size_t)t * hidden + j] = from_f32<TO>(fmaf(p - v, mu[j], v));
        if (first) slot[j] = o;
    }
}

template <typename TD>
__global__ void rmsnorm_add_kernel(float* __restrict__ stream, const TD* __restrict__ y, long long ldy, const float* __restrict__ gain, float eps,
                                   int hidden) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const TD* row = y + (size_t)t * ldy;
    float ss = 0.f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float v = to_f32<TD>(row[j]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    float* x = stream + (size_t)t * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) x[j] += gain[j] * (to_f32<TD>(row[j]) * inv);
}

// ---- rows of up to 4096 (norm and add) or 2048 (norm and shift) values that are a multiple of 4 wide: a warp per row, the
// row in registers (VPL float4 a lane), so that it is read once with all of its loads in flight, and the sum is a shuffle.
// The sum's order (a lane's values in order, then the lanes by halving) depends on the width alone.
__device__ __forceinline__ float4 load4(const float* p, int q) { return reinterpret_cast<const float4*>(p)[q]; }
__device__ __forceinline__ float4 load4(const bf16* p, int q) {
    const uint2 raw = reinterpret_cast<const uint2*>(p)[q];
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, int q, float4 v) { reinterpret_cast<float4*>(p)[q] = v; }
__device__ __forceinline__ void store4(bf16* p, int q, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    reinterpret_cast<uint2*>(p)[q] = packed;
}
__device__ __forceinline__ float squares(float4 v) { return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }

template <typename TD, int VPL>
__global__ void __launch_bounds__(256) rmsnorm_add_warp_kernel(float* __restrict__ stream, const TD* __restrict__ y, long long ldy,
                                                               const float* __restrict__ gain, float eps, int tokens, int hidden) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const int quads = hidden / 4;
    const TD* row = y + (size_t)t * ldy;
    float* x = stream + (size_t)t * hidden;
    float4 v[VPL], r[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        v[i] = q < quads ? load4(row, q) : make_float4(0.f, 0.f, 0.f, 0.f);
        r[i] = q < quads ? load4(x, q) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) ss += squares(v[i]);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        if (q >= quads) continue;
        const float4 g = load4(gain, q);
        store4(x, q, make_float4(r[i].x + g.x * (v[i].x * inv), r[i].y + g.y * (v[i].y * inv), r[i].z + g.z * (v[i].z * inv), r[i].w + g.w * (v[i].w * inv)));
    }
}

// x[t] += gain * z / rms(z) with z = y[t] + bias (bias may be null), then (out given) out[t] = x[t] in out's type: a branch joins
// the stream through its norm, the bias of its last product on the way, and the stream's rows for a next branch that reads the
// stream itself follow from the row in registers
template <typename TD, typename TO, int VPL>
__global__ void __launch_bounds__(256) rmsnorm_add_rows_warp_kernel(float* __restrict__ stream, const TD* __restrict__ y, long long ldy,
                                                                    const float* __restrict__ bias, const float* __restrict__ gain, float eps,
                                                                    TO* __restrict__ out, int tokens, int hidden) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const int quads = hidden / 4;
    const TD* row = y + (size_t)t * ldy;
    float* x = stream + (size_t)t * hidden;
    float4 v[VPL], r[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        v[i] = q < quads ? load4(row, q) : make_float4(0.f, 0.f, 0.f, 0.f);
        r[i] = q < quads ? load4(x, q) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (bias) {                                 // a loop of its own: the rows' loads above are all in flight before anything waits
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int q = i * 32 + lane;
            if (q >= quads) continue;
            const float4 b = load4(bias, q);
            v[i] = make_float4(v[i].x + b.x, v[i].y + b.y, v[i].z + b.z, v[i].w + b.w);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) ss += squares(v[i]);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        if (q >= quads) continue;
        const float4 g = load4(gain, q);
        r[i] = make_float4(r[i].x + g.x * (v[i].x * inv), r[i].y + g.y * (v[i].y * inv), r[i].z + g.z * (v[i].z * inv), r[i].w + g.w * (v[i].w * inv));
        store4(x, q, r[i]);
        if (out) store4(out + (size_t)t * hidden, q, r[i]);
    }
}

// x[t] += gain * y[t] / rms(y[t]), then out[t] = gain2 * x[t] / rms(x[t]): a branch joins the stream through its norm and the
// norm in front of the next branch follows from the row in registers
template <typename TD, typename TO, int VPL>
__global__ void __launch_bounds__(256) rmsnorm_add_norm_warp_kernel(float* __restrict__ stream, const TD* __restrict__ y, long long ldy,
                                                                    const float* __restrict__ gain, float eps, const float* __restrict__ gain2,
                                                                    float eps2, TO* __restrict__ out, int tokens, int hidden) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const int quads = hidden / 4;
    const TD* row = y + (size_t)t * ldy;
    float* x = stream + (size_t)t * hidden;
    float4 v[VPL], r[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        v[i] = q < quads ? load4(row, q) : make_float4(0.f, 0.f, 0.f, 0.f);
        r[i] = q < quads ? load4(x, q) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) ss += squares(v[i]);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        if (q >= quads) continue;
        const float4 g = load4(gain, q);
        r[i] = make_float4(r[i].x + g.x * (v[i].x * inv), r[i].y + g.y * (v[i].y * inv), r[i].z + g.z * (v[i].z * inv), r[i].w + g.w * (v[i].w * inv));
        store4(x, q, r[i]);
        s2 += squares(r[i]);
    }
    s2 = warp_sum(s2);
    const float inv2 = 1.0f / sqrtf(s2 / (float)hidden + eps2);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        if (q >= quads) continue;
        const float4 g = load4(gain2, q);
        store4(out + (size_t)t * hidden, q, make_float4(g.x * (r[i].x * inv2), g.y * (r[i].y * inv2), g.z * (r[i].z * inv2), g.w * (r[i].w * inv2)));
    }
}

template <typename TO, int VPL>
__global__ void __launch_bounds__(256) rmsnorm_shift_warp_kernel(const float* __restrict__ stream, const float* __restrict__ gain, float eps,
                                                                 const float* __restrict__ mu, float* __restrict__ state, long long slot_floats,
                                                                 const int* __restrict__ token_seq, const int* __restrict__ seq_starts,
                                                                 const int* __restrict__ seq_slots, TO* __restrict__ out, int tokens, int hidden) {
    __shared__ float inv_of_warp[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    const bool live = t < tokens;
    const int quads = hidden / 4;
    const float* x = stream + (size_t)(live ? t : 0) * hidden;
    // the own row's loads go out first: their addresses need nothing of the batch's tables
    float4 v[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        v[i] = live && q < quads ? load4(x, q) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int seq = live ? token_seq[t] : 0, start = live ? seq_starts[seq] : 0;
    const bool first = live && t == start;
    float* slot = state + (size_t)(live ? seq_slots[seq] : 0) * slot_floats;
    // the row in front; the first token's warp norms the entry's last row for the slot instead
    const float* other = stream + (size_t)(live ? (first ? seq_starts[seq + 1] - 1 : t - 1) : 0) * hidden;
    // The own row stays in registers.  The inverse root mean square of the row in front is the warp in front's own (through
    // shared memory: the same instructions in the same order, so the same bits as when this warp computes it); only a
    // block's first warp and an entry's first token sum the other row's squares themselves.
    float ss = 0.f, so = 0.f;
    const bool own_sum = live && (first || warp == 0);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        ss += squares(v[i]);
        if (own_sum && q < quads) so += squares(load4(other, q));
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    if (lane == 0) inv_of_warp[warp] = inv;
    float inv_other = 0.f;
    if (own_sum) {
        so = warp_sum(so);
        inv_other = 1.0f / sqrtf(so / (float)hidden + eps);
    }
    __syncthreads();
    if (!live) return;
    if (!own_sum) inv_other = inv_of_warp[warp - 1];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        if (q >= quads) continue;
        const float4 g = load4(gain, q), m = load4(mu, q), o = load4(other, q);
        const float4 a = make_float4(g.x * (v[i].x * inv), g.y * (v[i].y * inv), g.z * (v[i].z * inv), g.w * (v[i].w * inv));
        const float4 b = make_float4(g.x * (o.x * inv_other), g.y * (o.y * inv_other), g.z * (o.z * inv_other), g.w * (o.w * inv_other));
        const float4 p = first ? load4(slot, q) : b;
        store4(out + (size_t)t * hidden, q, make_float4(fmaf(p.x - a.x, m.x, a.x), fmaf(p.y - a.y, m.y, a.y), fmaf(p.z - a.z, m.z, a.z), fmaf(p.w - a.w, m.w, a.w)));
        if (first) store4(slot, q, b);
    }
}

inline bool aligned16(const void* p) { return (uintptr_t)p % 16 == 0; }
inline void warp_rows_launch(int rows, int* blocks, int* threads) {
    const int warps = rows >= 2048 ? 8 : rows >= 512 ? 2 : 1;      // few rows: a warp a block, so that they are spread over the SMs
    *blocks = (rows + warps - 1) / warps;
    *threads = warps * 32;
}

__device__ __forceinline__ float xielu_f(float z, float ap, float an) {
    if (z > 0.f) return fmaf(ap * z, z, 0.5f * z);
    return fmaf(an, expm1f(z) - z, 0.5f * z);
}

template <typename TI, typename TO>
__global__ void xielu_kernel(const TI* __restrict__ x, long long ldx, TO* __restrict__ out, long long ldo, int tokens, int n, float ap, float an) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * n) return;
    const int t = (int)(i / n), c = (int)(i % n);
    out[(size_t)t * ldo + c] = from_f32<TO>(xielu_f(to_f32<TI>(x[(size_t)t * ldx + c]), ap, an));
}

template <typename T>
__global__ void embedding_scaled_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ stream, int hidden, int vocab,
                                        float scale, int* status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* out = stream + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, EG_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) out[j] = 0.0f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) out[j] = to_f32<T>(row[j]) * scale;
}

__global__ void scale_kernel(float* __restrict__ x, long long n, float s) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= s;
}

inline int row_threads(int hidden) {
    int threads = 64;
    while (threads < 512 && threads * 4 < hidden) threads <<= 1;
    return threads;
}

}  // namespace

// rows float32 [tokens, hidden], already normalised; out in out_dtype
EG_API int eg_token_shift(cudaStream_t stream, const float* rows, const float* mu, float* state, long long slot_floats, const int* token_seq,
                          const int* seq_starts, const int* seq_slots, void* out, int out_dtype, int tokens, int hidden) {
    if (tokens <= 0) return 0;
    const int threads = row_threads(hidden);
    if (out_dtype == EG_BF16)
        token_shift_kernel<bf16><<<tokens, threads, 0, stream>>>(rows, mu, state, slot_floats, token_seq, seq_starts, seq_slots, (bf16*)out, hidden);
    else
        token_shift_kernel<float><<<tokens, threads, 0, stream>>>(rows, mu, state, slot_floats, token_seq, seq_starts, seq_slots, (float*)out, hidden);
    return eg_launch_status();
}

// the norm of the float32 stream and the shift in one kernel
EG_API int eg_rmsnorm_shift(cudaStream_t stream, const float* residual, const float* gain, float eps, const float* mu, float* state,
                            long long slot_floats, const int* token_seq, const int* seq_starts, const int* seq_slots, void* out, int out_dtype,
                            int tokens, int hidden) {
    if (tokens <= 0) return 0;
    // (few rows: a block a row spreads a row's loads over more threads; measured at 8 rows of 2,048: 8 us against 18)
    if (tokens >= 256 && hidden % 4 == 0 && hidden <= 2048 && slot_floats % 4 == 0 && aligned16(residual) && aligned16(gain) && aligned16(mu) && aligned16(state) &&
        aligned16(out)) {
        // four warps a block: 512 blocks at 2,048 rows, all resident at once (measured cold: 16.5 us a launch; eight warps a block 17.1)
        const int nt = 128, blocks = (tokens + 3) / 4;
        const int vpl = (hidden / 4 + 31) / 32;
#define EG_SHIFT_WARP(TO, V) \
    rmsnorm_shift_warp_kernel<TO, V><<<blocks, nt, 0, stream>>>(residual, gain, eps, mu, state, slot_floats, token_seq, seq_starts, seq_slots, (TO*)out, tokens, hidden)
        if (out_dtype == EG_BF16) {
            if (vpl <= 4) EG_SHIFT_WARP(bf16, 4);
            else if (vpl <= 8) EG_SHIFT_WARP(bf16, 8);
            else EG_SHIFT_WARP(bf16, 16);
        } else {
            if (vpl <= 4) EG_SHIFT_WARP(float, 4);
            else if (vpl <= 8) EG_SHIFT_WARP(float, 8);
            else EG_SHIFT_WARP(float, 16);
        }
#undef EG_SHIFT_WARP
        return eg_launch_status();
    }
    const int threads = row_threads(hidden);
    if (out_dtype == EG_BF16)
        rmsnorm_shift_kernel<bf16><<<tokens, threads, 0, stream>>>(residual, gain, eps, mu, state, slot_floats, token_seq, seq_starts, seq_slots, (bf16*)out,
                                                                   hidden);
    else
        rmsnorm_shift_kernel<float><<<tokens, threads, 0, stream>>>(residual, gain, eps, mu, state, slot_floats, token_seq, seq_starts, seq_slots, (float*)out,
                                                                    hidden);
    return eg_launch_status();
}

// residual[t] += gain * y[t] / rms(y[t])
EG_API int eg_rmsnorm_add(cudaStream_t stream, float* residual, const void* y, int y_dtype, long long ldy, const float* gain, float eps, int tokens,
                          int hidden) {
    if (tokens <= 0) return 0;
    if (hidden % 4 == 0 && hidden <= 4096 && ldy % 4 == 0 && aligned16(residual) && aligned16(y) && aligned16(gain)) {
        int blocks, nt;
        warp_rows_launch(tokens, &blocks, &nt);
        const int vpl = (hidden / 4 + 31) / 32;
#define EG_ADD_WARP(TD, V) rmsnorm_add_warp_kernel<TD, V><<<blocks, nt, 0, stream>>>(residual, (const TD*)y, ldy, gain, eps, tokens, hidden)
        if (y_dtype == EG_BF16) {
            if (vpl <= 4) EG_ADD_WARP(bf16, 4);
            else if (vpl <= 8) EG_ADD_WARP(bf16, 8);
            else if (vpl <= 16) EG_ADD_WARP(bf16, 16);
            else EG_ADD_WARP(bf16, 32);
        } else {
            if (vpl <= 4) EG_ADD_WARP(float, 4);
            else if (vpl <= 8) EG_ADD_WARP(float, 8);
            else if (vpl <= 16) EG_ADD_WARP(float, 16);
            else EG_ADD_WARP(float, 32);
        }
#undef EG_ADD_WARP
        return eg_launch_status();
    }
    const int threads = row_threads(hidden);
    if (y_dtype == EG_BF16) rmsnorm_add_kernel<bf16><<<tokens, threads, 0, stream>>>(residual, (const bf16*)y, ldy, gain, eps, hidden);
    else rmsnorm_add_kernel<float><<<tokens, threads, 0, stream>>>(residual, (const float*)y, ldy, gain, eps, hidden);
    return eg_launch_status();
}

// residual[t] += gain * y[t] / rms(y[t]), then out[t] = gain2 * residual[t] / rms(residual[t]) (eps2), in one kernel.  Returns
// cudaErrorInvalidValue for sizes it does not take (rows of up to 2,048 values, a multiple of 4, 16-byte aligned).
EG_API int eg_rmsnorm_add_norm(cudaStream_t stream, float* residual, const void* y, int y_dtype, long long ldy, const float* gain, float eps,
                               const float* gain2, float eps2, void* out, int out_dtype, int tokens, int hidden) {
    if (tokens <= 0) return 0;
    if (hidden % 4 || hidden > 2048 || ldy % 4 || !aligned16(residual) || !aligned16(y) || !aligned16(gain) || !aligned16(gain2) || !aligned16(out))
        return (int)cudaErrorInvalidValue;
    int blocks, nt;
    warp_rows_launch(tokens, &blocks, &nt);
    const int vpl = (hidden / 4 + 31) / 32;
#define EG_ADD_NORM(TD, TO, V) \
    rmsnorm_add_norm_warp_kernel<TD, TO, V><<<blocks, nt, 0, stream>>>(residual, (const TD*)y, ldy, gain, eps, gain2, eps2, (TO*)out, tokens, hidden)
#define EG_ADD_NORM_V(TD, TO)               \
    if (vpl <= 4) EG_ADD_NORM(TD, TO, 4);   \
    else if (vpl <= 8) EG_ADD_NORM(TD, TO, 8); \
    else EG_ADD_NORM(TD, TO, 16)
    if (y_dtype == EG_BF16 && out_dtype == EG_BF16) { EG_ADD_NORM_V(bf16, bf16); }
    else if (y_dtype == EG_BF16) { EG_ADD_NORM_V(bf16, float); }
    else if (out_dtype == EG_BF16) { EG_ADD_NORM_V(float, bf16); }
    else { EG_ADD_NORM_V(float, float); }
#undef EG_ADD_NORM_V
#undef EG_ADD_NORM
    return eg_launch_status();
}

// residual[t] += gain * z / rms(z), z = y[t] + bias (bias float32 [hidden] or null); with out, also out[t] = residual[t] in
// out_dtype, in one kernel.  Returns cudaErrorInvalidValue for sizes it does not take (rows of up to 4,096 values, a multiple
// of 4, 16-byte aligned).
EG_API int eg_rmsnorm_add_rows(cudaStream_t stream, float* residual, const void* y, int y_dtype, long long ldy, const float* bias, const float* gain, float eps,
                               void* out, int out_dtype, int tokens, int hidden) {
    if (tokens <= 0) return 0;
    if (hidden % 4 || hidden > 4096 || ldy % 4 || !aligned16(residual) || !aligned16(y) || !aligned16(gain) || (bias && !aligned16(bias)) ||
        (out && !aligned16(out)))
        return (int)cudaErrorInvalidValue;
    int blocks, nt;
    warp_rows_launch(tokens, &blocks, &nt);
    const int vpl = (hidden / 4 + 31) / 32;
#define EG_ADD_ROWS(TD, TO, V) \
    rmsnorm_add_rows_warp_kernel<TD, TO, V><<<blocks, nt, 0, stream>>>(residual, (const TD*)y, ldy, bias, gain, eps, (TO*)out, tokens, hidden)
#define EG_ADD_ROWS_V(TD, TO)                  \
    if (vpl <= 4) EG_ADD_ROWS(TD, TO, 4);      \
    else if (vpl <= 8) EG_ADD_ROWS(TD, TO, 8); \
    else if (vpl <= 16) EG_ADD_ROWS(TD, TO, 16); \
    else EG_ADD_ROWS(TD, TO, 32)
    if (y_dtype == EG_BF16 && out_dtype == EG_BF16) { EG_ADD_ROWS_V(bf16, bf16); }
    else if (y_dtype == EG_BF16) { EG_ADD_ROWS_V(bf16, float); }
    else if (out_dtype == EG_BF16) { EG_ADD_ROWS_V(float, bf16); }
    else { EG_ADD_ROWS_V(float, float); }
#undef EG_ADD_ROWS_V
#undef EG_ADD_ROWS
    return eg_launch_status();
}

// out[t, c] = xielu(x[t, c]); ap and an are the finished coefficients (softplus applied by the caller)
EG_API int eg_xielu(cudaStream_t stream, const void* x, int x_dtype, long long ldx, void* out, int out_dtype, long long ldo, int tokens, int n, float ap,
                    float an) {
    const long long total = (long long)tokens * n;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (x_dtype == EG_F32 && out_dtype == EG_F32) xielu_kernel<float, float><<<blocks, 256, 0, stream>>>((const float*)x, ldx, (float*)out, ldo, tokens, n, ap, an);
    else if (x_dtype == EG_F32) xielu_kernel<float, bf16><<<blocks, 256, 0, stream>>>((const float*)x, ldx, (bf16*)out, ldo, tokens, n, ap, an);
    else if (out_dtype == EG_F32) xielu_kernel<bf16, float><<<blocks, 256, 0, stream>>>((const bf16*)x, ldx, (float*)out, ldo, tokens, n, ap, an);
    else xielu_kernel<bf16, bf16><<<blocks, 256, 0, stream>>>((const bf16*)x, ldx, (bf16*)out, ldo, tokens, n, ap, an);
    return eg_launch_status();
}

EG_API int eg_embedding_gather_scaled(cudaStream_t stream, int dtype, const int* ids, const void* table, float* residual, int tokens, int hidden,
                                      int vocab, float scale, int* status) {
    if (tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == EG_BF16) embedding_scaled_kernel<bf16><<<tokens, threads, 0, stream>>>(ids, (const bf16*)table, residual, hidden, vocab, scale, status);
    else embedding_scaled_kernel<float><<<tokens, threads, 0, stream>>>(ids, (const float*)table, residual, hidden, vocab, scale, status);
    return eg_launch_status();
}

EG_API int eg_scale_f32(cudaStream_t stream, float* x, long long n, float s) {
    if (n <= 0) return 0;
    scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, n, s);
    return eg_launch_status();
}
