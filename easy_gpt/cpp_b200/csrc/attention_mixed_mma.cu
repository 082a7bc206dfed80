// Attention with mixed heads on the warp-level tensor cores (bfloat16 operands, float32 sums), over the paged cache that
// eg_mixed_attention_prepare fills.  With the mix folded into the queries (see attention_mixed.cu) a token has ONE key
// of `wide` = G * dk values for all H query heads (the normed and turned keys of its G key heads side by side), and the value
// of head h is the slice c(h) = h / (H / G) of the token's keys as projected (the cache's second plane):
//
//   s_h(i, j) = Q_h(i) . K(j)   over wide values;   o_h(i) = sum_j softmax_j(s_h(i, .)) k_c(h)(j);   out = o * sigmoid(gate)
//
//   eg_mixed_attention_tiles   prompt portions: a CTA takes 64 consecutive tokens of a listed tile and one head; its four
//                              warps hold 16 query rows each and walk the keys 32 at a time, the next 32 arriving by
//                              cp.async while these are used (flash-attention sums, a warp leaves out the tiles beyond its
//                              last row's position)
//   eg_mixed_attention_split   single tokens: a CTA takes one token, 16 heads (the rows of the tensor-core tile: all of them
//                              read the same keys) and one of `splits` ranges of the keys; each warp walks its own 16-key
//                              slices through a buffer of its own (no block-wide barrier in the loop).  The rows of a tile
//                              have different value heads: the product with the values is done once per value head of the
//                              tile with the other rows' weights set to zero.  The warps' sums are merged in shared memory and
//                              either finished (splits == 1) or stored for eg_mixed_attention_combine.
//
// Scores are in base 2 (the queries carry the scale; log2(e) is multiplied in here).  Sizes taken: dk a multiple of 16 up to
// 256 and shared memory up to the CTA's limit; everything else goes through eg_mixed_attention.
#include "mma_utils.cuh"

namespace {
constexpr int THREADS = 128;
constexpr int LISTED_ROWS = 128;   // tokens of a listed tile; a CTA of the prompt kernel takes 16 a warp of them
constexpr int BN = 32;             // keys a step of the prompt kernel
constexpr float LOG2E = 1.4426950408889634f;
constexpr int SMEM_LIMIT = 227 * 1024;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// S[16 MT x 8 NKT] = Q[16 MT x wide] K^T: q_rows 16 MT rows of stride qs in shared memory, k_rows 8 NKT keys of stride ks; a key
// fragment serves the MT row tiles
template <int MT, int NKT>
__device__ __forceinline__ void score_tile(float (&s)[MT][NKT][4], const bf16* q_rows, int qs, const bf16* k_rows, int ks, int wide, int lane) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < NKT; ++i) s[mt][i][0] = s[mt][i][1] = s[mt][i][2] = s[mt][i][3] = 0.f;
    const bf16* qa = q_rows + (lane & 15) * qs + (lane >> 4) * 8;
    const bf16* kb = k_rows + ((lane >> 4) * 8 + (lane & 7)) * ks + ((lane >> 3) & 1) * 8;
#pragma unroll 2
    for (int k0 = 0; k0 < wide; k0 += 16) {
        uint32_t a[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(a[mt], qa + mt * 16 * qs + k0);
#pragma unroll
        for (int np = 0; np < NKT / 2; ++np) {
            uint32_t b[4];
            ldmatrix_x4(b, kb + np * 16 * ks + k0);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_bf16_16816(s[mt][2 * np], a[mt], b[0], b[1]);
                mma_bf16_16816(s[mt][2 * np + 1], a[mt], b[2], b[3]);
            }
        }
    }
}

// the running maximum, sum and weights of the rows lane / 4 and lane / 4 + 8; key key0 + j is seen by a row up to its limit
template <int NKT>
__device__ __forceinline__ void softmax_tile(float (&s)[NKT][4], float (&m)[2], float (&l)[2], float (&corr)[2], int key0, int limit_lo, int limit_hi, int lane) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int limit = r ? limit_hi : limit_lo;
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int kpos = key0 + nt * 8 + 2 * (lane & 3) + e;
                const float v = kpos <= limit ? s[nt][2 * r + e] * LOG2E : -INFINITY;
                s[nt][2 * r + e] = v;
                mx = fmaxf(mx, v);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[r], mx);
        const float base = m_new == -INFINITY ? 0.f : m_new;
        corr[r] = ex2(m[r] - base);
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float pw = ex2(s[nt][2 * r + e] - base);
                s[nt][2 * r + e] = pw;
                sum += pw;
            }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[r] = l[r] * corr[r] + sum;
        m[r] = m_new;
    }
}

// O[16 MT x dk] += A[16 MT x 16] V[16 keys x dk]: v_rows 16 keys of stride vs, the head's first column already added
template <int MT, int NT>
__device__ __forceinline__ void value_step(float (&o)[MT][NT][4], const uint32_t (&a)[MT][4], const bf16* v_rows, int vs, int dk, int lane) {
    const bf16* vb = v_rows + (((lane >> 3) & 1) * 8 + (lane & 7)) * vs + (lane >> 4) * 8;
#pragma unroll
    for (int dp = 0; dp < NT / 2; ++dp) {
        if (dp * 16 < dk) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vb + dp * 16);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_bf16_16816(o[mt][2 * dp], a[mt], b[0], b[1]);
                mma_bf16_16816(o[mt][2 * dp + 1], a[mt], b[2], b[3]);
            }
        }
    }
}

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + __expf(-x)); }

struct TileParams {
    const bf16 *q, *k_cache, *v_cache;
    long long head_stride, page_stride;
    const int* block_table;
    int table_stride;
    const int *positions, *tiles;
    int num_subtiles;
    const float* gate;
    long long ld_gate;
    bf16* out;
    long long ldo;
    int heads, kv_heads, dk, page_size, num_pages;
    int* status;
};

// ---- prompt portions ---------------------------------------------------------------------------------------------------------
template <int NT, int WARPS, int MT>
__global__ void __launch_bounds__(WARPS * 32) mixed_tiles_kernel(const TileParams p) {
    constexpr int TILE_ROWS = 16 * MT * WARPS, SUBS = LISTED_ROWS / TILE_ROWS, NTHREADS = WARPS * 32;
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int dk = p.dk, wide = p.kv_heads * dk, qs = wide + 8, vs = dk + 8, cpr = wide / 8;
    const int sub = p.num_subtiles - 1 - (int)blockIdx.y;       // the last tiles of a prompt have the most keys: they start first, for all heads
    const int* tile = p.tiles + 3 * (sub / SUBS);
    const int first = tile[1] + TILE_ROWS * (sub % SUBS);
    const int count = min(TILE_ROWS, tile[2] - TILE_ROWS * (sub % SUBS));
    if (count <= 0) return;
    const int h = blockIdx.x;
    const int c_own = h / (p.heads / p.kv_heads);
    const int* table = p.block_table + (size_t)tile[0] * p.table_stride;

    bf16* q_s = (bf16*)smem;                                   // [TILE_ROWS][qs]
    bf16* k_s = q_s + TILE_ROWS * qs;                          // [2][BN][qs]
    bf16* v_s = k_s + 2 * BN * qs;                             // [2][BN][vs]
    long long* row_off = (long long*)(v_s + 2 * BN * vs);      // [2][BN]
    int* col_off = (int*)(row_off + 2 * BN);                   // [cpr]

    const int pos_last = p.positions[first + count - 1];
    const int steps = pos_last / BN + 1;
    auto find_rows = [&](int step, int buf) {
        if (tid < BN) {
            const int kpos = step * BN + tid;
            long long off = -1;
            if (kpos <= pos_last) {
                const int page = table[kpos / p.page_size];
                if (page < 0 || page >= p.num_pages) atomicOr(p.status, EG_STATUS_BAD_PAGE);
                else off = (long long)page * p.page_stride + (long long)(kpos % p.page_size) * dk;
            }
            row_off[buf * BN + tid] = off;
        }
    };
    auto fetch = [&](int buf) {
        for (int j = warp; j < BN; j += WARPS) {
            const long long off = row_off[buf * BN + j];
            const bool valid = off >= 0;
            bf16* kd = k_s + (buf * BN + j) * qs;
            for (int cc = lane; cc < cpr; cc += 32) cp_async_16(kd + cc * 8, p.k_cache + (valid ? off + col_off[cc] : 0), valid);
            bf16* vd = v_s + (buf * BN + j) * vs;
            for (int cc = lane; cc < dk / 8; cc += 32) cp_async_16(vd + cc * 8, p.v_cache + (valid ? off + c_own * p.head_stride + cc * 8 : 0), valid);
        }
    };

    for (int cc = tid; cc < cpr; cc += NTHREADS) col_off[cc] = (int)(((cc * 8) / dk) * p.head_stride + (cc * 8) % dk);
    find_rows(0, 0);
    for (int i = tid; i < TILE_ROWS * cpr; i += NTHREADS) {
        const int r = i / cpr, cc = i % cpr;
        const bool valid = r < count;
        cp_async_16(q_s + r * qs + cc * 8, p.q + (valid ? ((size_t)(first + r) * p.heads + h) * wide + cc * 8 : 0), valid);
    }
    __syncthreads();
    fetch(0);
    cp_async_commit();
    if (steps > 1) find_rows(1, 1);

    int limit[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = (warp * MT + mt) * 16 + (lane >> 2) + 8 * r;
            limit[mt][r] = row < count ? p.positions[first + row] : -1;
        }
    const int warp_limit = warp * MT * 16 < count ? p.positions[first + min(count - 1, warp * MT * 16 + MT * 16 - 1)] : -1;
    float m[MT][2], l[MT][2];
    float o[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        m[mt][0] = m[mt][1] = -INFINITY;
        l[mt][0] = l[mt][1] = 0.f;
#pragma unroll
        for (int i = 0; i < NT; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
    }

    for (int step = 0; step < steps; ++step) {
        const int buf = step & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (step + 1 < steps) fetch(buf ^ 1);
        cp_async_commit();
        if (step + 2 < steps) find_rows(step + 2, buf);
        const int key0 = step * BN;
        if (key0 > warp_limit) continue;
        float s[MT][BN / 8][4];
        score_tile<MT, BN / 8>(s, q_s + warp * MT * 16 * qs, qs, k_s + buf * BN * qs, qs, wide, lane);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float corr[2];
            softmax_tile<BN / 8>(s[mt], m[mt], l[mt], corr, key0, limit[mt][0], limit[mt][1], lane);
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                o[mt][i][0] *= corr[0];
                o[mt][i][1] *= corr[0];
                o[mt][i][2] *= corr[1];
                o[mt][i][3] *= corr[1];
            }
        }
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
            uint32_t a[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                a[mt][0] = pack_bf16(s[mt][2 * ks][0], s[mt][2 * ks][1]);
                a[mt][1] = pack_bf16(s[mt][2 * ks][2], s[mt][2 * ks][3]);
                a[mt][2] = pack_bf16(s[mt][2 * ks + 1][0], s[mt][2 * ks + 1][1]);
                a[mt][3] = pack_bf16(s[mt][2 * ks + 1][2], s[mt][2 * ks + 1][3]);
            }
            value_step<MT, NT>(o, a, v_s + (buf * BN + ks * 16) * vs, vs, dk, lane);
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = (warp * MT + mt) * 16 + (lane >> 2) + 8 * r;
            if (row >= count) continue;
            const float inv = l[mt][r] > 0.f ? 1.0f / l[mt][r] : 0.f;
            const size_t t = (size_t)(first + row);
            const float* g = p.gate ? p.gate + t * p.ld_gate + (size_t)h * dk : nullptr;
            bf16* dst = p.out + t * p.ldo + (size_t)h * dk;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int d = nt * 8 + 2 * (lane & 3);
                if (d < dk) {
                    float a = o[mt][nt][2 * r] * inv, b = o[mt][nt][2 * r + 1] * inv;
                    if (g) {
                        a *= sigmoid_f(g[d]);
                        b *= sigmoid_f(g[d + 1]);
                    }
                    *(__nv_bfloat162*)(dst + d) = __floats2bfloat162_rn(a, b);
                }
            }
        }
}

size_t tiles_smem(int wide, int dk, int rows) {
    return (size_t)(rows + 2 * BN) * (wide + 8) * 2 + (size_t)2 * BN * (dk + 8) * 2 + 2 * BN * 8 + (size_t)(wide / 8) * 4;
}

// ---- single tokens -----------------------------------------------------------------------------------------------------------
struct SplitParams {
    const bf16 *q, *k_cache, *v_cache;
    long long head_stride, page_stride;
    const int* block_table;
    int table_stride;
    const int *token_seq, *positions, *token_list;
    const float* gate;
    long long ld_gate;
    bf16* out;
    long long ldo;
    float *partial_acc, *partial_ml;      // [listed token, head, split, dk] and [.., 2] (maximum in base 2, sum)
    int heads, kv_heads, dk, page_size, num_pages, splits;
    int* status;
};

__host__ __device__ inline int split_chunk(int keys, int splits) {
    const int per = (keys + splits - 1) / splits;
    return max(128, (per + 63) / 64 * 64);
}

template <int NT>
__global__ void __launch_bounds__(THREADS) mixed_split_kernel(const SplitParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int dk = p.dk, wide = p.kv_heads * dk, qs = wide + 8, cpr = wide / 8, group = p.heads / p.kv_heads;
    const int listed = blockIdx.x, t = p.token_list ? p.token_list[listed] : listed;
    const int h0 = blockIdx.y * 16, z = blockIdx.z;
    const int pos = p.positions[t];
    const int* table = p.block_table + (size_t)p.token_seq[t] * p.table_stride;
    const int chunk = split_chunk(pos + 1, p.splits);
    const int k_begin = z * chunk, k_end = min(pos + 1, k_begin + chunk);

    bf16* q_s = (bf16*)smem;                                   // [16][qs]
    bf16* kv_s = q_s + 16 * qs;                                // per warp: 16 turned keys, then the 16 keys as projected, [qs] each
    bf16* k_w = kv_s + (size_t)warp * 32 * qs;
    bf16* v_w = k_w + 16 * qs;
    int* col_off = (int*)(kv_s + (size_t)(THREADS / 32) * 32 * qs);

    for (int cc = tid; cc < cpr; cc += THREADS) col_off[cc] = (int)(((cc * 8) / dk) * p.head_stride + (cc * 8) % dk);
    for (int i = tid; i < 16 * cpr; i += THREADS) {
        const int r = i / cpr, cc = i % cpr;
        const bool valid = h0 + r < p.heads;
        cp_async_16(q_s + r * qs + cc * 8, p.q + (valid ? ((size_t)t * p.heads + h0 + r) * wide + cc * 8 : 0), valid);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    const int row_lo = lane >> 2, row_hi = row_lo + 8;
    const int c_lo = (h0 + row_lo) / group, c_hi = (h0 + row_hi) / group;
    const int c_first = h0 / group, c_last = min(p.heads - 1, h0 + 15) / group;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o1[1][NT][4];
    float(&o)[NT][4] = o1[0];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int key0 = k_begin + warp * 16; key0 < k_end; key0 += 16 * (THREADS / 32)) {
        long long mine = -1;
        if (lane < 16 && key0 + lane < k_end) {
            const int kpos = key0 + lane;
            const int page = table[kpos / p.page_size];
            if (page < 0 || page >= p.num_pages) atomicOr(p.status, EG_STATUS_BAD_PAGE);
            else mine = (long long)page * p.page_stride + (long long)(kpos % p.page_size) * dk;
        }
        __syncwarp();                                          // the slices of the step before have been read
#pragma unroll 4
        for (int j = 0; j < 16; ++j) {
            const long long off = __shfl_sync(0xffffffffu, mine, j);
            const bool valid = off >= 0;
            for (int cc = lane; cc < cpr; cc += 32) {
                const long long at = valid ? off + col_off[cc] : 0;
                cp_async_16(k_w + j * qs + cc * 8, p.k_cache + at, valid);
                cp_async_16(v_w + j * qs + cc * 8, p.v_cache + at, valid);
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncwarp();
        float s1[1][2][4], corr[2];
        float(&s)[2][4] = s1[0];
        score_tile<1, 2>(s1, q_s, qs, k_w, qs, wide, lane);
        softmax_tile<2>(s, m, l, corr, key0, k_end - 1, k_end - 1, lane);
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
        const uint32_t a0 = pack_bf16(s[0][0], s[0][1]), a1 = pack_bf16(s[0][2], s[0][3]), a2 = pack_bf16(s[1][0], s[1][1]), a3 = pack_bf16(s[1][2], s[1][3]);
        for (int c = c_first; c <= c_last; ++c) {              // the rows of value head c, the others' weights zero
            const uint32_t a[1][4] = {{c_lo == c ? a0 : 0u, c_hi == c ? a1 : 0u, c_lo == c ? a2 : 0u, c_hi == c ? a3 : 0u}};
            value_step<1, NT>(o1, a, v_w + c * dk, qs, dk, lane);
        }
    }
    __syncthreads();                                           // every warp is done with its slices: the space is used again

    constexpr int OW = NT * 8 + 2;                             // a row's sums, then its maximum and its sum of weights
    float* merge = (float*)kv_s;                               // [warps][16][OW]
    {
        float* mine = merge + (size_t)warp * 16 * OW;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float* row = mine + (r ? row_hi : row_lo) * OW;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                row[nt * 8 + 2 * (lane & 3)] = o[nt][2 * r];
                row[nt * 8 + 2 * (lane & 3) + 1] = o[nt][2 * r + 1];
            }
            if ((lane & 3) == 0) {
                row[NT * 8] = m[r];
                row[NT * 8 + 1] = l[r];
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < 16 * dk; i += THREADS) {
        const int r = i / dk, d = i % dk, h = h0 + r;
        if (h >= p.heads) continue;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < THREADS / 32; ++w) top = fmaxf(top, merge[((size_t)w * 16 + r) * OW + NT * 8]);
        float acc = 0.f, sum = 0.f;
        if (top > -INFINITY) {
#pragma unroll
            for (int w = 0; w < THREADS / 32; ++w) {
                const float* row = merge + ((size_t)w * 16 + r) * OW;
                const float f = ex2(row[NT * 8] - top);
                acc = fmaf(f, row[d], acc);
                sum = fmaf(f, row[NT * 8 + 1], sum);
            }
        }
        if (p.splits == 1) {
            float v = sum > 0.f ? acc / sum : 0.f;
            if (p.gate) v *= sigmoid_f(p.gate[(size_t)t * p.ld_gate + (size_t)h * dk + d]);
            p.out[(size_t)t * p.ldo + (size_t)h * dk + d] = __float2bfloat16_rn(v);
        } else {
            const size_t at = ((size_t)listed * p.heads + h) * p.splits + z;
            p.partial_acc[at * dk + d] = acc;
            if (d == 0) {
                p.partial_ml[at * 2] = top;
                p.partial_ml[at * 2 + 1] = sum;
            }
        }
    }
}

// one block per (listed token, head): the ranges' sums become the head's output
__global__ void __launch_bounds__(128) mixed_combine_kernel(const SplitParams p) {
    const int listed = blockIdx.x, h = blockIdx.y, t = p.token_list ? p.token_list[listed] : listed;
    const size_t at = ((size_t)listed * p.heads + h) * p.splits;
    float top = -INFINITY;
    for (int z = 0; z < p.splits; ++z) top = fmaxf(top, p.partial_ml[(at + z) * 2]);
    for (int d = threadIdx.x; d < p.dk; d += blockDim.x) {
        float acc = 0.f, sum = 0.f;
        if (top > -INFINITY)
            for (int z = 0; z < p.splits; ++z) {
                const float f = ex2(p.partial_ml[(at + z) * 2] - top);
                acc = fmaf(f, p.partial_acc[(at + z) * p.dk + d], acc);
                sum = fmaf(f, p.partial_ml[(at + z) * 2 + 1], sum);
            }
        float v = sum > 0.f ? acc / sum : 0.f;
        if (p.gate) v *= sigmoid_f(p.gate[(size_t)t * p.ld_gate + (size_t)h * p.dk + d]);
        p.out[(size_t)t * p.ldo + (size_t)h * p.dk + d] = __float2bfloat16_rn(v);
    }
}

size_t split_smem(int wide, int dk_padded) {
    const size_t slices = (size_t)(THREADS / 32) * 32 * (wide + 8) * 2;
    const size_t merge = (size_t)(THREADS / 32) * 16 * (dk_padded + 2) * 4;
    return (size_t)16 * (wide + 8) * 2 + (slices > merge ? slices : merge) + (size_t)(wide / 8) * 4 + 16;
}

int padded_dk(int dk) { return dk <= 64 ? 64 : dk <= 128 ? 128 : 256; }
bool sizes_taken(int heads, int kv_heads, int dk) { return dk > 0 && dk <= 256 && dk % 16 == 0 && kv_heads > 0 && heads % kv_heads == 0; }
}  // namespace

template <class K>
static int raise_smem(K kernel, size_t bytes) {
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

// 1 when the two kernels take these sizes (bfloat16 only), else 0
EG_API int eg_mixed_attention_mma_takes(int heads, int kv_heads, int dk) {
    if (!sizes_taken(heads, kv_heads, dk)) return 0;
    const int wide = kv_heads * dk;
    return tiles_smem(wide, dk, 64) <= (size_t)SMEM_LIMIT && split_smem(wide, padded_dk(dk)) <= (size_t)SMEM_LIMIT;
}

// q bfloat16 [tokens, heads, kv_heads * dk] (folded queries); tiles int32 [num_tiles, 3] = (entry, first token, count <= 128);
// gate float32 [tokens, ld_gate] with head h at column h * dk, or null; out bfloat16 [tokens, ldo]
EG_API int eg_mixed_attention_tiles(cudaStream_t stream, const void* q, const void* k_cache, const void* v_cache, long long head_stride, const int* block_table,
                                    int table_stride, const int* positions, const int* tiles, int num_tiles, const float* gate, long long ld_gate, void* out,
                                    long long ldo, int heads, int kv_heads, int dk, int page_size, long long page_stride, int num_pages, int* status) {
    if (num_tiles <= 0) return 0;
    if (!eg_mixed_attention_mma_takes(heads, kv_heads, dk)) return (int)cudaErrorInvalidValue;
    TileParams p{(const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, head_stride, page_stride, block_table, table_stride, positions, tiles, 2 * num_tiles,
                 gate, ld_gate, (bf16*)out, ldo, heads, kv_heads, dk, page_size, num_pages, status};
    // all 128 tokens of a listed tile in one CTA where their queries fit beside the keys (a warp holds 32 rows, so that a key
    // fragment from shared memory serves two row tiles; heads of more than 128 values: 16 rows a warp), else 64 tokens
    const int wide = kv_heads * dk;
    const bool whole = tiles_smem(wide, dk, LISTED_ROWS) <= (size_t)SMEM_LIMIT;
    const int rows = whole ? LISTED_ROWS : 64;
    const size_t smem = tiles_smem(wide, dk, rows);
    const int subtiles = num_tiles * (LISTED_ROWS / rows);
    p.num_subtiles = subtiles;
    const dim3 grid(heads, subtiles);
    int rc = 0;
#define EG_MIXED_TILES(NT, W, MT)                                                   \
    do {                                                                            \
        if ((rc = raise_smem(mixed_tiles_kernel<NT, W, MT>, smem))) return rc;      \
        mixed_tiles_kernel<NT, W, MT><<<grid, W * 32, smem, stream>>>(p);           \
    } while (0)
    if (whole) {
        if (dk <= 64) EG_MIXED_TILES(8, 4, 2);
        else if (dk <= 128) EG_MIXED_TILES(16, 4, 2);
        else EG_MIXED_TILES(32, 8, 1);
    } else {
        if (dk <= 64) EG_MIXED_TILES(8, 4, 1);
        else if (dk <= 128) EG_MIXED_TILES(16, 4, 1);
        else EG_MIXED_TILES(32, 4, 1);
    }
#undef EG_MIXED_TILES
    return eg_launch_status();
}

// The listed tokens (token_list int32 [num_tokens], or null: tokens 0 .. num_tokens - 1), each against its own keys in `splits`
// ranges.  splits > 1 needs partial_acc float32 [num_tokens, heads, splits, dk] and partial_ml [num_tokens, heads, splits, 2].
EG_API int eg_mixed_attention_split(cudaStream_t stream, const void* q, const void* k_cache, const void* v_cache, long long head_stride, const int* block_table,
                                    int table_stride, const int* token_seq, const int* positions, const int* token_list, int num_tokens, const float* gate,
                                    long long ld_gate, void* out, long long ldo, float* partial_acc, float* partial_ml, int splits, int heads, int kv_heads, int dk,
                                    int page_size, long long page_stride, int num_pages, int* status) {
    if (num_tokens <= 0) return 0;
    if (!eg_mixed_attention_mma_takes(heads, kv_heads, dk) || splits < 1 || (splits > 1 && (!partial_acc || !partial_ml)) || splits > 65535)
        return (int)cudaErrorInvalidValue;
    SplitParams p{(const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, head_stride, page_stride, block_table, table_stride, token_seq, positions, token_list,
                  gate, ld_gate, (bf16*)out, ldo, partial_acc, partial_ml, heads, kv_heads, dk, page_size, num_pages, splits, status};
    const size_t smem = split_smem(kv_heads * dk, padded_dk(dk));
    const dim3 grid(num_tokens, (heads + 15) / 16, splits);
    int rc = 0;
    if (dk <= 64) {
        if ((rc = raise_smem(mixed_split_kernel<8>, smem))) return rc;
        mixed_split_kernel<8><<<grid, THREADS, smem, stream>>>(p);
    } else if (dk <= 128) {
        if ((rc = raise_smem(mixed_split_kernel<16>, smem))) return rc;
        mixed_split_kernel<16><<<grid, THREADS, smem, stream>>>(p);
    } else {
        if ((rc = raise_smem(mixed_split_kernel<32>, smem))) return rc;
        mixed_split_kernel<32><<<grid, THREADS, smem, stream>>>(p);
    }
    if ((rc = eg_launch_status())) return rc;
    if (splits > 1) {
        mixed_combine_kernel<<<dim3(num_tokens, heads), 128, 0, stream>>>(p);
        rc = eg_launch_status();
    }
    return rc;
}
