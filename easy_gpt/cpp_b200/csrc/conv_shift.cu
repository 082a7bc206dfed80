// A causal convolution over time in front of a mixer, on the normed rows of the stream, channel by channel:
//
//   h[t]   = gain * x[t] / sqrt(mean(x[t]^2) + eps)                      (the norm in front, computed here from the float32 stream)
//   out[t] = h[t] + sum_{j < taps} w[:, j] * h[t - taps + 1 + j]         rows before the request's start are zero
//
// The last taps - 1 normed rows of a request are its state (float32, [taps - 1, hidden] in the request's slot, oldest
// first), so that a step continues where the one before ended.  Two kernels: the first reads the slots and writes both
// h (for a part that reads the plain norm) and out; the second, launched behind it, moves the slots on.  A row's norm is
// computed by the same instructions whether the row is a token's own or an earlier one, and the slot keeps float32
// values: a cut between two steps changes nothing.
//
//   eg_rmsnorm_conv_shift        both outputs from the stream (gain [hidden]; plain_out may be null)
//   eg_conv_shift                the same from rows that are normed already (float32)
//   eg_conv_shift_state          the slots of every entry move on by the entry's rows
#include "common.cuh"

namespace {
constexpr int MAX_TAPS = 8;

// inv[d] = 1 / sqrt(mean(x_d^2) + eps) for n <= MAX_TAPS rows x_d = first + d * step (in floats) at once: one pass over the rows
// and two barriers.  A row's sum is formed in the same order whichever of the n it is and whatever the others are.
__device__ __forceinline__ void rows_inverse_rms(const float* first, long long step, int n, int hidden, float eps, float (*scratch)[32], float* inv) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    float ss[MAX_TAPS];
#pragma unroll
    for (int d = 0; d < MAX_TAPS; ++d) ss[d] = 0.f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
#pragma unroll
        for (int d = 0; d < MAX_TAPS; ++d)
            if (d < n) {
                const float x = first[d * step + j];
                ss[d] = fmaf(x, x, ss[d]);
            }
    }
#pragma unroll
    for (int d = 0; d < MAX_TAPS; ++d)
        if (d < n) {
            const float v = warp_sum(ss[d]);
            if (lane == 0) scratch[d][warp] = v;
        }
    __syncthreads();
    for (int d = warp; d < n; d += nwarps) {
        const float v = warp_sum(lane < nwarps ? scratch[d][lane] : 0.f);
        if (lane == 0) inv[d] = 1.0f / sqrtf(v / (float)hidden + eps);
    }
    __syncthreads();
}

// NORMED: `rows` are h already; else they are the stream and h is computed here
template <typename TO, bool NORMED>
__global__ void conv_shift_kernel(const float* __restrict__ rows, const float* __restrict__ gain, float eps, const float* __restrict__ w,
                                  float* __restrict__ state, long long slot_floats, const int* __restrict__ token_seq,
                                  const int* __restrict__ seq_starts, const int* __restrict__ seq_slots, TO* __restrict__ out, TO* __restrict__ plain_out,
                                  int hidden, int taps, int single) {
    __shared__ float scratch[MAX_TAPS][32];
    __shared__ float inv[MAX_TAPS];
    const int t = blockIdx.x, seq = token_seq[t], start = seq_starts[seq];
    const int back = min(taps - 1, t - start);                  // earlier rows that lie in this step
    float* slot = taps > 1 ? state + (size_t)seq_slots[seq] * slot_floats : nullptr;      // one tap: no earlier rows, no slot
    if (!NORMED) rows_inverse_rms(rows + (size_t)t * hidden, -(long long)hidden, back + 1, hidden, eps, scratch, inv);     // inv[d]: d rows back
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float g = NORMED ? 1.0f : gain[j];
        float own = 0.f, acc = 0.f;
        // tap k weighs the row d = taps - 1 - k tokens back; oldest first, so that the sum's order is the same everywhere
        for (int k = 0; k < taps; ++k) {
            const int d = taps - 1 - k;
            float v;
            if (d <= back) {
                const float xv = rows[(size_t)(t - d) * hidden + j];
                v = NORMED ? xv : g * (xv * inv[d]);
            } else {
                // d - back - 1 rows before the step's first: the slot's row (taps - 1) - (d - back)
                v = slot[(size_t)(taps - 1 - (d - back)) * hidden + j];
            }
            if (d == 0) own = v;
            acc = fmaf(w[(size_t)j * taps + k], v, acc);
        }
        out[(size_t)t * hidden + j] = from_f32<TO>(own + acc);
        if (plain_out) plain_out[(size_t)t * hidden + j] = from_f32<TO>(own);
        if (single && taps > 1) {
            // every entry of the step is one token: its block is the slot's only reader, so it moves the slot on itself
            for (int r = 0; r + 2 < taps; ++r) slot[(size_t)r * hidden + j] = slot[(size_t)(r + 1) * hidden + j];
            slot[(size_t)(taps - 2) * hidden + j] = own;
        }
    }
}

// one block per entry; a thread owns its channels in every row of the slot, so the rows can move in place
template <bool NORMED>
__global__ void conv_shift_state_kernel(const float* __restrict__ rows, const float* __restrict__ gain, float eps, float* __restrict__ state,
                                        long long slot_floats, const int* __restrict__ seq_starts, const int* __restrict__ seq_slots, int hidden, int taps) {
    __shared__ float scratch[MAX_TAPS][32];
    __shared__ float inv[MAX_TAPS];
    const int seq = blockIdx.x, start = seq_starts[seq], len = seq_starts[seq + 1] - start;
    if (len <= 0) return;
    float* slot = state + (size_t)seq_slots[seq] * slot_floats;
    const int keep = taps - 1;
    const int fresh = min(keep, len);                           // the slot's last `fresh` rows come from this step
    if (!NORMED) rows_inverse_rms(rows + (size_t)(start + len - fresh) * hidden, hidden, fresh, hidden, eps, scratch, inv);
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        for (int r = 0; r < keep - fresh; ++r) slot[(size_t)r * hidden + j] = slot[(size_t)(r + fresh) * hidden + j];
        for (int r = 0; r < fresh; ++r) {
            const float xv = rows[(size_t)(start + len - fresh + r) * hidden + j];
            slot[(size_t)(keep - fresh + r) * hidden + j] = NORMED ? xv : gain[j] * (xv * inv[r]);
        }
    }
}

template <bool NORMED>
int launch_conv_shift(cudaStream_t stream, const float* rows, const float* gain, float eps, const float* w, float* state, long long slot_floats,
                      const int* token_seq, const int* seq_starts, const int* seq_slots, void* out, void* plain_out, int out_dtype, int tokens, int hidden,
                      int taps, int single) {
    if (tokens <= 0) return 0;
    if (taps < 1 || taps > MAX_TAPS || hidden <= 0 || (taps > 1 && slot_floats < (long long)(taps - 1) * hidden)) return (int)cudaErrorInvalidValue;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (out_dtype == EG_BF16)
        conv_shift_kernel<bf16, NORMED><<<tokens, threads, 0, stream>>>(rows, gain, eps, w, state, slot_floats, token_seq, seq_starts, seq_slots, (bf16*)out,
                                                                       (bf16*)plain_out, hidden, taps, single);
    else
        conv_shift_kernel<float, NORMED><<<tokens, threads, 0, stream>>>(rows, gain, eps, w, state, slot_floats, token_seq, seq_starts, seq_slots, (float*)out,
                                                                        (float*)plain_out, hidden, taps, single);
    return eg_launch_status();
}
}  // namespace

// stream float32 [tokens, hidden]; w float32 [hidden, taps] (the last tap weighs the token's own row); state float32
// [slots, slot_floats] with this part's (taps - 1) * hidden values first; out and plain_out [tokens, hidden] in out_dtype
// single != 0: every entry of the step is one token, and the slots move on here (no eg_conv_shift_state behind)
EG_API int eg_rmsnorm_conv_shift(cudaStream_t stream, const float* residual, const float* gain, float eps, const float* w, float* state,
                                 long long slot_floats, const int* token_seq, const int* seq_starts, const int* seq_slots, void* out, void* plain_out,
                                 int out_dtype, int tokens, int hidden, int taps, int single) {
    return launch_conv_shift<false>(stream, residual, gain, eps, w, state, slot_floats, token_seq, seq_starts, seq_slots, out, plain_out, out_dtype, tokens, hidden,
                                    taps, single);
}

EG_API int eg_conv_shift(cudaStream_t stream, const float* rows, const float* w, float* state, long long slot_floats, const int* token_seq,
                         const int* seq_starts, const int* seq_slots, void* out, int out_dtype, int tokens, int hidden, int taps, int single) {
    return launch_conv_shift<true>(stream, rows, nullptr, 0.f, w, state, slot_floats, token_seq, seq_starts, seq_slots, out, nullptr, out_dtype, tokens, hidden, taps,
                                   single);
}

// gain null: `rows` are normed already; else they are the stream and the slot receives gain * x / rms(x)
EG_API int eg_conv_shift_state(cudaStream_t stream, const float* rows, const float* gain, float eps, float* state, long long slot_floats, const int* seq_starts,
                               const int* seq_slots, int num_seqs, int hidden, int taps) {
    if (num_seqs <= 0 || taps <= 1) return 0;
    if (taps > MAX_TAPS || slot_floats < (long long)(taps - 1) * hidden) return (int)cudaErrorInvalidValue;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (gain) conv_shift_state_kernel<false><<<num_seqs, threads, 0, stream>>>(rows, gain, eps, state, slot_floats, seq_starts, seq_slots, hidden, taps);
    else conv_shift_state_kernel<true><<<num_seqs, threads, 0, stream>>>(rows, nullptr, 0.f, state, slot_floats, seq_starts, seq_slots, hidden, taps);
    return eg_launch_status();
}
