// Paged grouped-query attention on the warp-level tensor cores (bfloat16), for
// every token of a step: decoded tokens and, until a tiled prefill kernel takes
// them, the tokens of prompt portions too.
//
// One CTA works on (token, KV head, split): the G = NH/NKV query heads that share
// the KV head are the rows of the MMA (padded to 16), so a key tile is read once
// for all of them.  The token's visible keys [first, pos] are cut into tiles of
// 64 keys (aligned to 64, so a tile's 16-key quarters never straddle a page of
// 16, 32, 64, ... tokens); the tiles are dealt to `splits` CTAs in contiguous
// runs, each CTA streams its run through a cp.async pipeline, its four warps take
// a quarter of every tile each, and keep a running softmax (m, l, acc) in
// float32 (src/cuda/ops/self_attn_detail.cuh:325-382).  The warps' states are
// merged in shared memory; with one split the result is written at once, else a
// partial (m, l, acc) goes to scratch memory and the CTA of that (token, KV head)
// that finishes last (a ticket counter; nobody waits) merges the splits in order.
//
// score = (q . k) * scale in float32; the running softmax works in base 2 (scores times
// log2 e, exp2f: one hardware instruction, 2 ulp); P is rounded to bfloat16 for the
// P V product (as V is bfloat16 anyway); sums and the accumulator stay float32.
#include <cstdlib>

#include "mma_utils.cuh"

namespace {

constexpr int TILE_KEYS = 64;
constexpr int THREADS = 128;
constexpr int QUARTER_TILES = 64;      // tiles whose cache addresses are kept in shared memory at a time

// DEEP: as many stages as fit about 96 KB (up to five tiles in flight per CTA, two CTAs per SM): for steps with few
// CTAs, where each has to keep its own loads going.  Otherwise three stages, so that four CTAs share an SM: with
// many CTAs it is their number in flight that hides a tile's latency.
constexpr int MAX_SPLITS = 128;

// TPI: the CTA's warps in fours; TI: key tiles that they work on at a time (a warp takes 16 or 32 keys of a tile)
template <int HD, bool DEEP = true, int TPI = 1, int TI = TPI>
struct Layout {
    static constexpr int CHUNKS = HD / 8;                         // 16-byte chunks per key row
    static constexpr int SWZ = CHUNKS >= 8 ? 7 : CHUNKS - 1;
    static constexpr int TILE_BYTES = TILE_KEYS * HD * 2;          // K or V
    static constexpr int GROUP_BYTES = 2 * TILE_BYTES;             // K and V of one tile
    static constexpr int STAGE_BYTES = TI * GROUP_BYTES;
    // up to five tiles in flight per CTA, within about 96 KB of shared memory (two stages at least)
    static constexpr int DEEP_STAGES = (TPI * 96 * 1024 / STAGE_BYTES) >= 5 ? 5 : ((TPI * 96 * 1024 / STAGE_BYTES) >= 2 ? (TPI * 96 * 1024 / STAGE_BYTES) : 2);
    static constexpr int STAGES = DEEP ? DEEP_STAGES : (DEEP_STAGES < 3 ? DEEP_STAGES : 3);
    static constexpr int WARP_MERGE_BYTES = TPI * 4 * 16 * (HD + 2) * 4;      // the warps' partial results
    static constexpr int SPLIT_MERGE_BYTES = (2 * 16 * MAX_SPLITS + 16) * 4;  // (m, l) of every row and split, 1/l per row
    static constexpr int MERGE_BYTES = WARP_MERGE_BYTES > SPLIT_MERGE_BYTES ? WARP_MERGE_BYTES : SPLIT_MERGE_BYTES;
    static constexpr int SMEM = (STAGES * STAGE_BYTES > MERGE_BYTES) ? STAGES * STAGE_BYTES : MERGE_BYTES;
    __device__ static __forceinline__ int offset(int row, int chunk) {      // bytes inside a K or V tile
        return (row * CHUNKS + (chunk ^ (row & SWZ))) * 16;
    }
};

// tanh by one exponent and one division: absolute error about 1e-7, which a score that goes into an exponent next can bear
__device__ __forceinline__ float tanh_by_exp(float x) {
    const float e = __expf(2.0f * fminf(x, 15.0f));
    return 1.0f - __fdividef(2.0f, e + 1.0f);
}

struct Params {
    const bf16* q;
    int ldq;
    const bf16* k_cache;
    const bf16* v_cache;
    long long page_stride, head_stride;
    const int* block_table;
    int table_stride;
    const int* token_seq;
    const int* positions;
    const int* seq_context;   // [sequences] keys cached before this step (those from it on are written by the kernel in front); may be null
    bf16* out;
    int ldo;
    float* partial_acc;       // [T, NH, splits, HD]
    float* partial_ml;        // [T, NH, splits, 2]
    int num_heads, num_kv_heads, page_size, num_pages, window, splits;
    float scale;
    int* status;
    const void* prefetch;         // weights of a kernel that runs soon: pulled into L2 meanwhile
    long long prefetch_bytes;
    int* counters;                // [tokens of this launch * gridDim.y] tickets, zero before and after every launch
    int use_pdl;
    unsigned long long* trace;    // optional: [2] earliest start / latest end of this launch's CTAs (%globaltimer, ns)
    const int* token_list;        // optional: the tokens this launch works on (blockIdx.x indexes it); null: all, in order
    int cluster_merge;            // the splits of a (token, KV head) are one cluster and are merged in its first CTA's shared memory
    float sink2 = -INFINITY;      // a sink's logit times log2(e): one more term of the softmax's denominator; -inf: none
    // Further masks and score functions (all off by default; PrefillParams has the same).  chunk: a query sees keys of its own
    // block of `chunk` positions only; keep_first: keys 0 .. keep_first - 1 stay visible whatever window and chunk say (their
    // key tiles are walked first); softcap c: the scaled score becomes c tanh(score / c); sinks: a logit per query row
    // (natural log) in place of sink2; maps m: query rows head * m + map read key head (head / group) * m + map (both planes
    // hold num_kv_heads heads; num_heads counts rows); out_scale: a factor on the output; out_f32: float32 output [tokens, ldo].
    int chunk = 0, keep_first = 0, maps = 1;
    float softcap = 0.f, out_scale = 1.f;
    const float* sinks = nullptr;
    float* out_f32 = nullptr;
};

// acc * this = the softmax's output, with (m, l) the reference (base 2) and sum of the weights that acc holds, and the
// sink's term 2^(sink2 - m) joining the sum (in a form that cannot overflow whatever m is)
__device__ __forceinline__ float norm_with_sink(float m, float l, float sink2) {
    if (!(l > 0.f)) return 0.f;
    if (sink2 == -INFINITY) return 1.0f / l;
    const float top = fmaxf(m, sink2), c = exp2f(m - top);
    return c / fmaf(l, c, exp2f(sink2 - top));
}

// MASKED: the further masks and score functions of Params are read; without it they are constants ("none"), and the kernel is the
// plain one to the instruction.
template <int HD, bool DEEP, int TPI, int KW, bool MASKED>
__global__ void __launch_bounds__(TPI * THREADS) attention_paged_kernel(const Params p) {
    const int x_chunk = MASKED ? p.chunk : 0, x_keep = MASKED ? p.keep_first : 0, x_maps = MASKED ? p.maps : 1;
    const float x_softcap = MASKED ? p.softcap : 0.f, x_out_scale = MASKED ? p.out_scale : 1.f;
    const float* const x_sinks = MASKED ? p.sinks : nullptr;
    float* const x_out_f32 = MASKED ? p.out_f32 : nullptr;
    constexpr int TI = TPI * KW / 16;                                // key tiles of an iteration
    constexpr int KB = KW / 16;                                      // blocks of 16 keys a warp takes of its tile
    using L = Layout<HD, DEEP, TPI, TI>;
    constexpr int NT = TPI * THREADS;                                // threads of the CTA
    constexpr int WARPS = TPI * 4;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int is_last;
    TraceScope trace_scope(p.trace);
    const int t = p.token_list ? p.token_list[blockIdx.x] : blockIdx.x;
    const int G = p.num_heads / p.num_kv_heads;
    const int gblocks = (G + 15) / 16;
    const int kvh = blockIdx.y / gblocks;
    const int g0 = (blockIdx.y % gblocks) * 16;                   // first query head of the group handled here
    const int split = blockIdx.z;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const float cap_pre = x_softcap > 0.f ? p.scale / x_softcap : 0.f, cap_post = x_softcap * 1.4426950408889634f;
    // the query row (and output row) of row r of this key head's group, and its sink (base 2)
    auto head_of = [&](int r) { return x_maps == 1 ? kvh * G + r : ((kvh / x_maps) * G + r) * x_maps + kvh % x_maps; };
    auto sink_of = [&](int r) { return x_sinks ? x_sinks[head_of(r)] * 1.4426950408889634f : p.sink2; };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;

    if (p.prefetch) {
        constexpr long long PIECE = 4096;
        const long long pieces = (p.prefetch_bytes + PIECE - 1) / PIECE;
        const long long cta = ((long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        const long long ctas = (long long)gridDim.x * gridDim.y * gridDim.z;
        for (long long i = cta * NT + threadIdx.x; i < pieces; i += ctas * NT) {
            const long long off = i * PIECE;
            const long long n = p.prefetch_bytes - off < PIECE ? p.prefetch_bytes - off : PIECE;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(static_cast<const char*>(p.prefetch) + off),
                         "r"((unsigned)(n & ~15LL)) : "memory");
        }
    }
    // Positions and block tables were uploaded before the step and the cached keys were written by earlier
    // steps, so everything up to the first fresh key can be fetched before the kernel in front has finished.
    if (p.use_pdl == 1) asm volatile("griddepcontrol.launch_dependents;\n" ::);
    const int pos = p.positions[t];
    const int fresh_from = p.seq_context ? p.seq_context[p.token_seq[t]] : 0;
    int first = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    if (x_chunk > 0) first = max(first, pos / x_chunk * x_chunk);
    const int* table = p.block_table + (size_t)p.token_seq[t] * p.table_stride;
    const int tile_lo = first / TILE_KEYS, tile_hi = pos / TILE_KEYS;           // inclusive
    // Key tiles in the order they are walked: those of the kept first keys that lie wholly in front of the others, then the
    // tiles from the first visible key on.  my_lo, my_hi and every tile index below count in that order; tile_of gives the tile.
    const int kept_tiles = x_keep > 0 ? min((x_keep + TILE_KEYS - 1) / TILE_KEYS, tile_lo) : 0;
    const int all_tiles = kept_tiles + tile_hi - tile_lo + 1;
    auto tile_of = [&](int w) { return w < kept_tiles ? w : tile_lo + w - kept_tiles; };
    auto visible = [&](int kpos) { return (kpos >= first || kpos < x_keep) && kpos <= pos; };
    const int per = (all_tiles + p.splits - 1) / p.splits;
    const int my_lo = split * per;
    const int my_hi = min(all_tiles - 1, my_lo + per - 1);
    const int ntiles = my_hi - my_lo + 1;                                       // may be <= 0

    // Where every 16-key quarter of this CTA's tiles starts in the cache (element offset, -1: nothing to read):
    // looked up once through the block table, so that the tile loads below touch no global metadata.
    __shared__ long long quarter_base[QUARTER_TILES * 4];
    int quarter_tile0 = my_lo;
    auto fill_quarters = [&](int tile0) {
        quarter_tile0 = tile0;
        const int count = min(QUARTER_TILES, my_hi - tile0 + 1);
        for (int e = threadIdx.x; e < count * 4; e += NT) {
            const int kpos0 = tile_of(tile0 + e / 4) * TILE_KEYS + (e % 4) * 16;
            long long base = -1;
            if (kpos0 <= pos && (kpos0 + 15 >= first || kpos0 < x_keep)) {
                const int page = table[kpos0 / p.page_size];
                if (page < 0 || page >= p.num_pages) atomicOr(p.status, EG_STATUS_BAD_PAGE);
                else base = (long long)page * p.page_stride + (long long)kvh * p.head_stride + (long long)(kpos0 % p.page_size) * HD;
            }
            quarter_base[e] = base;
        }
    };
    if (ntiles > 0) fill_quarters(my_lo);
    __syncthreads();

    // mode 0: every row; 1 (before the wait): all but the fresh keys; 2 (after it): the fresh keys only
    auto load_one = [&](int tile, unsigned char* ks, int mode) {
        unsigned char* vs = ks + L::TILE_BYTES;
        const long long* qb = quarter_base + (tile - quarter_tile0) * 4;
        for (int e = threadIdx.x; e < TILE_KEYS * L::CHUNKS; e += NT) {
            const int row = e / L::CHUNKS, chunk = e % L::CHUNKS;
            const int kpos = tile_of(tile) * TILE_KEYS + row;
            const long long base = qb[row >> 4];
            const bool valid = visible(kpos) && base >= 0;
            const bool fresh = visible(kpos) && kpos >= fresh_from;
            if ((mode == 1 && fresh) || (mode == 2 && !fresh)) continue;
            const long long off = valid ? base + (long long)(row & 15) * HD + chunk * 8 : 0;
            cp_async_16(ks + L::offset(row, chunk), p.k_cache + off, valid);
            cp_async_16(vs + L::offset(row, chunk), p.v_cache + off, valid);
        }
    };
    // the TPI tiles of iteration `it` into stage `stage` (those that exist); fresh_only: only tiles that hold fresh keys
    auto load_tile = [&](int it_tile0, int stage, int mode) {
#pragma unroll
        for (int g = 0; g < TI; ++g) {
            const int tile = it_tile0 + g;
            if (tile > my_hi) break;
            if (mode == 2 && (tile_of(tile) + 1) * TILE_KEYS <= fresh_from) continue;
            load_one(tile, smem + stage * L::STAGE_BYTES + g * L::GROUP_BYTES, mode);
        }
    };
    const int niter = ntiles > 0 ? (ntiles + TI - 1) / TI : 0;

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;                 // rows gid and gid + 8
    float acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

#pragma unroll
    for (int s = 0; s < L::STAGES - 1; ++s) {
        if (s < niter) load_tile(my_lo + s * TI, s, 1);
        cp_async_commit();
    }
    trace_scope.mark(0);
    if (p.use_pdl) asm volatile("griddepcontrol.wait;\n" ::: "memory");     // q and the fresh keys come from the kernel in front
    if (p.use_pdl == 2) asm volatile("griddepcontrol.launch_dependents;\n" ::);
    trace_scope.mark(1);
#pragma unroll
    for (int s = 0; s < L::STAGES - 1; ++s)
        if (s < niter) load_tile(my_lo + s * TI, s, 2);
    cp_async_commit();

    // ---- query rows as A fragments: row r <-> head kvh*G + g0 + r
    uint32_t qf[HD / 16][4];
    {
        const int r0 = g0 + gid, r1 = g0 + gid + 8;
        const bf16* q0 = p.q + (size_t)t * p.ldq + (size_t)head_of(r0) * HD;
        const bf16* q1 = p.q + (size_t)t * p.ldq + (size_t)head_of(r1) * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            const int d = ks * 16 + 2 * tig;
            qf[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
            qf[ks][1] = r1 < G ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
            qf[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
            qf[ks][3] = r1 < G ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
        }
    }


    constexpr int WARPS_PER_TILE = TILE_KEYS / KW;
    const int group = warp / WARPS_PER_TILE, key0 = (warp % WARPS_PER_TILE) * KW;   // which tile of the iteration, which keys of it
    for (int it = 0; it < niter; ++it) {
        if (it == 0) cp_async_wait<0>();                                          // the first tiles and their fresh rows
        else cp_async_wait<L::STAGES - 2>();
        __syncthreads();
        if (it == 0) trace_scope.mark(2);
        {   // prefetch the tile STAGES-1 ahead into the stage freed by the previous iteration
            const int nxt = it + L::STAGES - 1;
            if (nxt < niter && (nxt * TI) % QUARTER_TILES == 0) {                 // the next stretch of the block table
                fill_quarters(my_lo + nxt * TI);
                __syncthreads();
            }
            if (nxt < niter) load_tile(my_lo + nxt * TI, nxt % L::STAGES, 0);
            cp_async_commit();
        }
        const unsigned char* ks = smem + (it % L::STAGES) * L::STAGE_BYTES + group * L::GROUP_BYTES;
        const unsigned char* vs = ks + L::TILE_BYTES;
        if (it * TI + group >= ntiles) continue;                                  // the run has no tile for this group of warps any more
        const int key_base = tile_of(my_lo + it * TI + group) * TILE_KEYS + key0; // this warp's KW keys
        if (key_base > pos || (key_base + KW - 1 < first && key_base >= x_keep)) continue;   // nothing visible in them

        // S = Q K^T for 16 rows x KW keys
        float s[2 * KB][4];
#pragma unroll
        for (int j = 0; j < 2 * KB; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                uint32_t b[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4(b, ks + L::offset(key0 + kb * 16 + (mi >> 1) * 8 + r, kk * 2 + (mi & 1)));
                mma_bf16_16816(s[2 * kb], qf[kk], b[0], b[1]);
                mma_bf16_16816(s[2 * kb + 1], qf[kk], b[2], b[3]);
            }
        }
        // scale, mask, running softmax
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2 * KB; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kpos = key_base + j * 8 + 2 * tig + (e & 1);
                const bool ok = visible(kpos);
                s[j][e] = ok ? (x_softcap > 0.f ? cap_post * tanh_by_exp(s[j][e] * cap_pre) : s[j][e] * scale_log2) : -INFINITY;
                if (e < 2) tmax0 = fmaxf(tmax0, s[j][e]); else tmax1 = fmaxf(tmax1, s[j][e]);
            }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        const float mn0 = fmaxf(m0, tmax0), mn1 = fmaxf(m1, tmax1);               // finite: a key of these is visible
        const float c0 = exp2f(m0 - mn0), c1 = exp2f(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        uint32_t pf[KB][4];
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
            const float (&sa)[4] = s[2 * kb];
            const float (&sb)[4] = s[2 * kb + 1];
            const float e00 = exp2f(sa[0] - mn0), e01 = exp2f(sa[1] - mn0), e02 = exp2f(sa[2] - mn1), e03 = exp2f(sa[3] - mn1);
            const float e10 = exp2f(sb[0] - mn0), e11 = exp2f(sb[1] - mn0), e12 = exp2f(sb[2] - mn1), e13 = exp2f(sb[3] - mn1);
            ps0 += (e00 + e01) + (e10 + e11);
            ps1 += (e02 + e03) + (e12 + e13);
            pf[kb][0] = pack_bf16(e00, e01);
            pf[kb][1] = pack_bf16(e02, e03);
            pf[kb][2] = pack_bf16(e10, e11);
            pf[kb][3] = pack_bf16(e12, e13);
        }
        l0 = l0 * c0 + ps0;
        l1 = l1 * c1 + ps1;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            acc[i][0] *= c0;
            acc[i][1] *= c0;
            acc[i][2] *= c1;
            acc[i][3] *= c1;
        }
        // acc += P V
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
            for (int nt = 0; nt < HD / 8; nt += 2) {
                uint32_t b[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4_trans(b, vs + L::offset(key0 + kb * 16 + (mi & 1) * 8 + r, nt + (mi >> 1)));
                mma_bf16_16816(acc[nt], pf[kb], b[0], b[1]);
                mma_bf16_16816(acc[nt + 1], pf[kb], b[2], b[3]);
            }
    }
    cp_async_wait<0>();
    trace_scope.mark(3, true);
    __syncthreads();                                                              // the pipeline's memory is free now

    // ---- merge the four warps: rows r = gid, gid + 8
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* wm = reinterpret_cast<float*>(smem);                                   // [WARPS][16]
    float* wl = wm + WARPS * 16;                                                  // [WARPS][16]
    float* wacc = wl + WARPS * 16;                                                // [WARPS][16][HD]
    if (tig == 0) {
        wm[warp * 16 + gid] = m0;
        wm[warp * 16 + gid + 8] = m1;
        wl[warp * 16 + gid] = l0;
        wl[warp * 16 + gid + 8] = l1;
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + 2 * tig;
        float* a0 = wacc + ((warp * 16 + gid) * HD + d);
        float* a1 = wacc + ((warp * 16 + gid + 8) * HD + d);
        a0[0] = acc[i][0];
        a0[1] = acc[i][1];
        a1[0] = acc[i][2];
        a1[1] = acc[i][3];
    }
    // Splits as a cluster: every CTA of it is past its key tiles here, so the first CTA's pipeline memory is free for
    // the others' results (behind the part that its own warps' merge still uses).
    unsigned cluster_rank = 0;
    uint32_t incoming = 0;                                                         // [splits][rows][HD + 2] in the first CTA
    if (p.cluster_merge) {
        asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(cluster_rank));
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(incoming) : "r"(smem_u32(smem + L::WARP_MERGE_BYTES)), "r"(0));
        asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    } else {
        __syncthreads();
    }
    const int rows = min(16, G - g0);
    for (int e = threadIdx.x; e < rows * HD; e += NT) {
        const int r = e / HD, d = e % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, wm[w * 16 + r]);
        float l = 0.f, a = 0.f;
        if (m > -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float f = exp2f(wm[w * 16 + r] - m);                          // -inf -> 0
                l += wl[w * 16 + r] * f;
                a += wacc[(w * 16 + r) * HD + d] * f;
            }
        }
        const int h = kvh * G + g0 + r;
        if (p.splits == 1) {
            const float s2 = sink_of(g0 + r);
            const float v = (s2 == -INFINITY ? (l > 0.f ? a / l : 0.f) : a * norm_with_sink(m, l, s2)) * x_out_scale;
            const size_t at = (size_t)t * p.ldo + (size_t)head_of(g0 + r) * HD + d;
            if (x_out_f32) x_out_f32[at] = v;
            else p.out[at] = __float2bfloat16_rn(v);
        } else if (p.cluster_merge) {
            const uint32_t at = incoming + (uint32_t)((cluster_rank * rows + r) * (HD + 2)) * 4u;
            asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at + (uint32_t)d * 4u), "f"(a) : "memory");
            if (d == 0) {
                asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at + (uint32_t)HD * 4u), "f"(m) : "memory");
                asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at + (uint32_t)(HD + 1) * 4u), "f"(l) : "memory");
            }
        } else {
            const size_t slot = ((size_t)t * p.num_heads + h) * p.splits + split;
            p.partial_acc[slot * HD + d] = a;
            if (d == 0) {
                p.partial_ml[slot * 2] = m;
                p.partial_ml[slot * 2 + 1] = l;
            }
        }
    }
    trace_scope.mark(4);
    if (p.splits == 1) return;
    if (p.cluster_merge) {
        asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
        trace_scope.mark(5);
        if (cluster_rank != 0) return;
        // out = sum_s acc_s e^{m_s - m} / sum_s l_s e^{m_s - m}, the splits in order, from this CTA's own shared memory
        const float* inc = reinterpret_cast<const float*>(smem + L::WARP_MERGE_BYTES);
        constexpr int QUADS = HD / 4;
        for (int q = threadIdx.x; q < rows * QUADS; q += NT) {
            const int r = q / QUADS, dq = q % QUADS;
            float m = -INFINITY;
            for (int s2 = 0; s2 < p.splits; ++s2) m = fmaxf(m, inc[(size_t)(s2 * rows + r) * (HD + 2) + HD]);
            float l = 0.f;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s2 = 0; s2 < p.splits; ++s2) {
                const float* part = inc + (size_t)(s2 * rows + r) * (HD + 2);
                const float w = m > -INFINITY ? exp2f(part[HD] - m) : 0.f;
                l += part[HD + 1] * w;
                const float2 lo = *reinterpret_cast<const float2*>(part + dq * 4), hi = *reinterpret_cast<const float2*>(part + dq * 4 + 2);
                a.x += lo.x * w; a.y += lo.y * w; a.z += hi.x * w; a.w += hi.y * w;
            }
            const float il = norm_with_sink(m, l, sink_of(g0 + r)) * x_out_scale;
            const size_t at = (size_t)t * p.ldo + (size_t)head_of(g0 + r) * HD + dq * 4;
            if (x_out_f32) *reinterpret_cast<float4*>(x_out_f32 + at) = make_float4(a.x * il, a.y * il, a.z * il, a.w * il);
            else *reinterpret_cast<uint2*>(p.out + at) = make_uint2(pack_bf16(a.x * il, a.y * il), pack_bf16(a.z * il, a.w * il));
        }
        return;
    }

    // ---- the last CTA of this (token, KV head) to get here merges the splits, in order:
    // out = sum_s acc_s e^{m_s - m} / sum_s l_s e^{m_s - m}
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = p.counters + (size_t)blockIdx.x * gridDim.y + blockIdx.y;   // by the token's place in this launch
        const int ticket = atomicAdd(counter, 1);
        is_last = ticket == p.splits - 1;
        if (is_last) *counter = 0;                                                // all have arrived: ready for the next launch
    }
    __syncthreads();
    trace_scope.mark(5);
    if (!is_last) return;
    __threadfence();
    // Every load of the merge is issued before anything waits: (m, l) of all (row, split) pairs, and the first
    // MERGE_BATCH splits of the accumulators, a float4 of one row per thread.  One trip to the L2 instead of several.
    constexpr int MERGE_BATCH = 16;
    constexpr int QUADS = HD / 4;
    float* fac = reinterpret_cast<float*>(smem);                                  // [rows][splits]: m_s, then e^{m_s - m}
    float* lpart = fac + 16 * p.splits;                                            // [rows][splits]: l_s
    float* inv_l = lpart + 16 * p.splits;                                          // [rows]
    const size_t head0 = (size_t)t * p.num_heads + kvh * G + g0;
    for (int e = threadIdx.x; e < rows * p.splits; e += NT) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.partial_ml) + head0 * p.splits + e);   // rows are consecutive heads
        fac[e] = ml.x;
        lpart[e] = ml.y;
    }
    for (int q0 = 0; q0 < rows * QUADS; q0 += NT) {
        const int q = q0 + threadIdx.x;
        const bool mine = q < rows * QUADS;
        const int r = mine ? q / QUADS : 0, dq = mine ? q % QUADS : 0;
        const float4* src = reinterpret_cast<const float4*>(p.partial_acc + (head0 + r) * p.splits * HD) + dq;
        float4 part[MERGE_BATCH];
#pragma unroll
        for (int i = 0; i < MERGE_BATCH; ++i)
            if (mine && i < p.splits) part[i] = __ldcg(src + (size_t)i * QUADS);
        if (q0 == 0) {
            __syncthreads();
            if (threadIdx.x < rows) {
                float* f = fac + threadIdx.x * p.splits;
                const float* lp = lpart + threadIdx.x * p.splits;
                float m = -INFINITY;
                for (int s2 = 0; s2 < p.splits; ++s2) m = fmaxf(m, f[s2]);
                float l = 0.f;
                for (int s2 = 0; s2 < p.splits; ++s2) {                             // in order
                    const float w = m > -INFINITY ? exp2f(f[s2] - m) : 0.f;
                    f[s2] = w;
                    l += lp[s2] * w;
                }
                inv_l[threadIdx.x] = norm_with_sink(m, l, sink_of(g0 + threadIdx.x)) * x_out_scale;
            }
            __syncthreads();
        }
        if (!mine) continue;
        const float* f = fac + r * p.splits;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < MERGE_BATCH; ++i)
            if (i < p.splits) {
                const float w = f[i];
                a.x += part[i].x * w; a.y += part[i].y * w; a.z += part[i].z * w; a.w += part[i].w * w;
            }
        for (int s0 = MERGE_BATCH; s0 < p.splits; s0 += MERGE_BATCH) {             // further splits, a batch in flight at a time
#pragma unroll
            for (int i = 0; i < MERGE_BATCH; ++i)
                if (s0 + i < p.splits) part[i] = __ldcg(src + (size_t)(s0 + i) * QUADS);
#pragma unroll
            for (int i = 0; i < MERGE_BATCH; ++i)
                if (s0 + i < p.splits) {
                    const float w = f[s0 + i];
                    a.x += part[i].x * w; a.y += part[i].y * w; a.z += part[i].z * w; a.w += part[i].w * w;
                }
        }
        const float il = inv_l[r];
        const size_t at = (size_t)t * p.ldo + (size_t)head_of(g0 + r) * HD + dq * 4;
        if (x_out_f32) *reinterpret_cast<float4*>(x_out_f32 + at) = make_float4(a.x * il, a.y * il, a.z * il, a.w * il);
        else *reinterpret_cast<uint2*>(p.out + at) = make_uint2(pack_bf16(a.x * il, a.y * il), pack_bf16(a.z * il, a.w * il));
    }
}

template <int HD, bool DEEP, bool MASKED, int TPI = 1, int KW = 16>
int launch_with(cudaStream_t stream, const Params& p, dim3 grid, bool must_cluster = false) {
    using L = Layout<HD, DEEP, TPI, TPI * KW / 16>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_paged_kernel<HD, DEEP, TPI, KW, MASKED>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(TPI * THREADS);
    cfg.dynamicSmemBytes = L::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    if (p.use_pdl) {
        attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[nattr].val.programmaticStreamSerializationAllowed = 1;
        ++nattr;
    }
    // The splits of a (token, KV head) as one cluster (up to 16 CTAs, which needs the kernel's leave for a cluster of
    // more than 8), merged through the first CTA's shared memory instead of scratch memory and a ticket: for the
    // launches of fewer CTAs than SMs, and for those of many small CTAs.
    Params q = p;
    static const bool cluster_allowed = !(getenv("EASY_GPT_CLUSTER_MERGE") && atoi(getenv("EASY_GPT_CLUSTER_MERGE")) == 0);
    const int G = p.num_heads / p.num_kv_heads;
    const size_t incoming_bytes = (size_t)p.splits * (G < 16 ? G : 16) * (HD + 2) * sizeof(float);
    // (Measured on B200, 16 splits, context 4096: at batch 1 the step takes 0.708 ms with it against 0.749, at batch 4
    // 0.753 against 0.777; at batch 8, 256 CTAs in 16 clusters, 0.966 against 0.826: so many clusters of 16 find room
    // only when the kernel in front has left the SMs, and the early start is lost.)
    int sms = 0, device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long long ctas = (long long)grid.x * grid.y * grid.z;
    // Launches of many CTAs (four an SM): clusters of up to 8 (batch 24 / 32 / 64: 1.288 / 1.370 / 1.604 ms a step with
    // them, 1.307 / 1.394 / 1.65 without).
    if (cluster_allowed && ((DEEP && ctas <= sms) || (!DEEP && p.splits <= 8)) && p.splits > 1 && p.splits <= 16 &&
        L::WARP_MERGE_BYTES + incoming_bytes <= (size_t)L::SMEM) {
        static int leave = 0;                                                      // 0 not asked yet, 1 given, -1 refused
        if (!leave) leave = cudaFuncSetAttribute(attention_paged_kernel<HD, DEEP, TPI, KW, MASKED>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess ? 1 : -1;
        if (p.splits <= 8 || leave == 1) {
            attr[nattr].id = cudaLaunchAttributeClusterDimension;
            attr[nattr].val.clusterDim.x = 1;
            attr[nattr].val.clusterDim.y = 1;
            attr[nattr].val.clusterDim.z = (unsigned)p.splits;
            cfg.attrs = attr;
            cfg.numAttrs = nattr + 1;
            int clusters = 0;
            // all clusters have to be on the GPU together, or the last ones run as a second wave (measured: batch 8, 16
            // clusters of 8 CTAs, of which 15 found room: the step took 0.92 ms instead of 0.80)
            if (cudaOccupancyMaxActiveClusters(&clusters, attention_paged_kernel<HD, DEEP, TPI, KW, MASKED>, &cfg) == cudaSuccess &&
                clusters >= (int)(grid.x * grid.y)) {
                q.cluster_merge = 1;
                ++nattr;
            } else {
                (void)cudaGetLastError();
            }
        }
    }
    if (must_cluster && !q.cluster_merge) return -1;                              // the caller has another way
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    return (int)cudaLaunchKernelEx(&cfg, attention_paged_kernel<HD, DEEP, TPI, KW, MASKED>, q);
}

template <int HD, bool MASKED>
int launch(cudaStream_t stream, const Params& p, int tokens) {
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    const int G = p.num_heads / p.num_kv_heads;
    const dim3 grid(tokens, p.num_kv_heads * ((G + 15) / 16), p.splits);
    const long long ctas = (long long)grid.x * grid.y * grid.z;
    // Up to twice as many CTAs as SMs: eight warps a CTA take two key tiles at a time and half as many splits (the same
    // warps, tiles in flight and trips through the keys as with four warps), so that the splits of a (token, KV head)
    // are at most 8 CTAs, one an SM, and can be merged as a cluster.  All clusters have to find room at once; if they
    // do not, a split or two fewer may.  (Measured on B200, context 4096, ms a decode step with / without: batch 1
    // 0.681 / 0.749, batch 4 0.702 / 0.777, batch 7 0.732; batch 8: 16 clusters of 8 do not find room.)
    // A long run of key tiles is a stream, and streams want all SMs: at the 0.5B sizes, batch 8, context 32k, 7 splits in
    // 16 clusters are 112 CTAs and the step takes 1.59 ms with them, 1.45 with 256 four-warp CTAs.
    constexpr int WIDE_KEYS = HD <= 64 ? 32 : 16;                                // keys a warp of the eight-warp form takes of a tile
    const long long most_tiles = ((long long)p.table_stride * p.page_size + TILE_KEYS - 1) / TILE_KEYS;
    if constexpr (HD <= 128) if (ctas <= 2ll * sm_count && p.splits >= 4 && p.splits % 2 == 0) {
        for (int fewer = 0; fewer <= 2; ++fewer) {
            Params half = p;
            half.splits = p.splits / 2 - fewer;
            if (half.splits < 2) break;
            // long runs: only if the clusters still cover most of the SMs (7B sizes, batch 8, context 8k: 4.05 ms a step with
            // 32 clusters of 4, 5.08 with 256 four-warp CTAs and tickets)
            if (most_tiles > 16ll * half.splits && (long long)grid.x * grid.y * half.splits * 100 < 85ll * sm_count) break;
            const int rc = launch_with<HD, true, MASKED, 2, WIDE_KEYS>(stream, half, dim3(grid.x, grid.y, half.splits), true);
            if (rc != -1) return rc;
        }
    }
    return ctas <= 2ll * sm_count ? launch_with<HD, true, MASKED>(stream, p, grid) : launch_with<HD, false, MASKED>(stream, p, grid);
}


// ---------------------------------------------------------------------------
// Prompt portions: 64 consecutive query tokens of one request (half of a listed
// tile) and one query head per CTA (four warps of 16 rows), against key tiles of 64 from the
// paged cache — the portion's own keys were stored there just before.  The K/V
// tiles of a KV head are read by the CTAs of its G query heads at about the same
// time and come from the L2 after the first.  Causal and window limits are
// applied per element; the running softmax is the same as above.
// ---------------------------------------------------------------------------

// 2^x by the hardware's approximation (relative error about 2^-22; results below 2^-126 become 0, and -inf gives 0).
__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct PrefillParams {
    const bf16* q;
    int ldq;
    const bf16* k_cache;
    const bf16* v_cache;
    long long page_stride, head_stride;
    const int* block_table;
    int table_stride;
    const int* positions;      // [T]
    const int* tiles;          // [num_tiles][3]: sequence (row of the block table), first token, tokens in the tile (<= 128)
    bf16* out;
    int ldo;
    int num_heads, num_kv_heads, page_size, num_pages, window;
    float scale;
    int* status;
    float sink2 = -INFINITY;      // as in Params
    // Further masks and score functions (all off by default).  chunk: a query sees keys of its own block of `chunk` positions
    // only; keep_first: keys 0 .. keep_first - 1 stay visible whatever window and chunk say; softcap c: the scaled score becomes
    // c tanh(score / c); sinks: a logit per query row in place of sink2; maps m: rows h = head * m + map read key head
    // (head / group) * m + map (both planes hold num_kv_heads heads); out_scale: a factor on the output; out_f32: the
    // output goes there as float32 [tokens, ldo] instead of to `out`.
    int chunk = 0, keep_first = 0, maps = 1;
    float softcap = 0.f, out_scale = 1.f;
    const float* sinks = nullptr;
    float* out_f32 = nullptr;
};

template <int HD>
struct PrefillLayout {
    static constexpr int CHUNKS = HD / 8;
    static constexpr int TILE_BYTES = TILE_KEYS * HD * 2;
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int STAGES = 3;
    static constexpr int SMEM = STAGES * STAGE_BYTES;
};

template <int HD, bool MASKED>
__global__ void __launch_bounds__(THREADS, HD <= 64 ? 4 : 2) attention_prefill_kernel(const PrefillParams p) {
    const int x_chunk = MASKED ? p.chunk : 0, x_keep = MASKED ? p.keep_first : 0, x_maps = MASKED ? p.maps : 1;
    const float x_softcap = MASKED ? p.softcap : 0.f, x_out_scale = MASKED ? p.out_scale : 1.f;
    const float* const x_sinks = MASKED ? p.sinks : nullptr;
    float* const x_out_f32 = MASKED ? p.out_f32 : nullptr;
    using L = Layout<HD>;
    using PL = PrefillLayout<HD>;
    extern __shared__ __align__(128) unsigned char smem[];
    // later tiles of a request see more keys: start them first
    const int item = gridDim.x - 1 - blockIdx.x;
    const int tile = item >> 1, half = item & 1;                 // a listed tile has up to 128 tokens: two CTAs
    const int h = blockIdx.y;
    const int kvh = (h / x_maps) / (p.num_heads / p.num_kv_heads) * x_maps + h % x_maps;
    // with a soft cap the scores are scaled and capped as they come out of the product; else the scale rides in the exponent
    const float scale_log2 = x_softcap > 0.f ? 1.4426950408889634f : p.scale * 1.4426950408889634f;
    const float sink2 = x_sinks ? x_sinks[h] * 1.4426950408889634f : p.sink2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int seq = p.tiles[tile * 3], t0 = p.tiles[tile * 3 + 1] + half * TILE_KEYS;
    const int count = min(TILE_KEYS, p.tiles[tile * 3 + 2] - half * TILE_KEYS);
    if (count <= 0) return;
    const int* table = p.block_table + (size_t)seq * p.table_stride;
    const int pos_lo = p.positions[t0], pos_hi = pos_lo + count - 1;           // positions in a tile are consecutive
    // the first key that the window and the chunk of a query at `pos` leave visible (never decreasing in pos)
    auto first_of = [&](int pos) {
        const int w = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
        return x_chunk > 0 ? max(w, pos / x_chunk * x_chunk) : w;
    };
    const int first = first_of(pos_lo);
    const int tile_lo = first / TILE_KEYS;
    // key tiles in the order they are walked: those of the kept first keys that lie wholly in front of the others, then the
    // tiles from the first visible key on
    const int kept_tiles = x_keep > 0 ? min((x_keep + TILE_KEYS - 1) / TILE_KEYS, tile_lo) : 0;
    const int ntiles = kept_tiles + pos_hi / TILE_KEYS - tile_lo + 1;
    auto tile_of = [&](int it) { return it < kept_tiles ? it : tile_lo + it - kept_tiles; };

    // rows of this warp: r0 = warp*16 + gid, r1 = r0 + 8
    const int r0 = warp * 16 + gid, r1 = r0 + 8;
    const bool v0 = r0 < count, v1 = r1 < count;
    const int qp0 = pos_lo + r0, qp1 = pos_lo + r1;
    uint32_t qf[HD / 16][4];
    {
        const bf16* q0 = p.q + (size_t)(t0 + (v0 ? r0 : 0)) * p.ldq + (size_t)h * HD;
        const bf16* q1 = p.q + (size_t)(t0 + (v1 ? r1 : 0)) * p.ldq + (size_t)h * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            const int d = ks * 16 + 2 * tig;
            qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
            qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
            qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
            qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
        }
    }

    __shared__ long long quarter_base[QUARTER_TILES * 4];         // as in the decode kernel
    int quarter_tile0 = 0;                                        // in walking order
    auto fill_quarters = [&](int tile0) {
        quarter_tile0 = tile0;
        const int count = min(QUARTER_TILES, ntiles - tile0);
        for (int e = threadIdx.x; e < count * 4; e += THREADS) {
            const int kpos0 = tile_of(tile0 + e / 4) * TILE_KEYS + (e % 4) * 16;
            long long base = -1;
            if (kpos0 <= pos_hi && (kpos0 + 15 >= first || kpos0 < x_keep)) {
                const int page = table[kpos0 / p.page_size];
                if (page < 0 || page >= p.num_pages) atomicOr(p.status, EG_STATUS_BAD_PAGE);
                else base = (long long)page * p.page_stride + (long long)kvh * p.head_stride + (long long)(kpos0 % p.page_size) * HD;
            }
            quarter_base[e] = base;
        }
    };
    fill_quarters(0);
    __syncthreads();

    auto load_tile = [&](int it, int stage) {                     // `it` in walking order
        unsigned char* ks = smem + stage * PL::STAGE_BYTES;
        unsigned char* vs = ks + PL::TILE_BYTES;
        const long long* qb = quarter_base + (it - quarter_tile0) * 4;
        const int kt = tile_of(it);
        for (int e = threadIdx.x; e < TILE_KEYS * L::CHUNKS; e += THREADS) {
            const int row = e / L::CHUNKS, chunk = e % L::CHUNKS;
            const int kpos = kt * TILE_KEYS + row;
            const long long base = qb[row >> 4];
            const bool valid = (kpos >= first || kpos < x_keep) && kpos <= pos_hi && base >= 0;
            const long long off = valid ? base + (long long)(row & 15) * HD + chunk * 8 : 0;
            cp_async_16(ks + L::offset(row, chunk), p.k_cache + off, valid);
            cp_async_16(vs + L::offset(row, chunk), p.v_cache + off, valid);
        }
    };

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

#pragma unroll
    for (int s = 0; s < PL::STAGES - 1; ++s) {
        if (s < ntiles) load_tile(s, s);
        cp_async_commit();
    }
    for (int it = 0; it < ntiles; ++it) {
        cp_async_wait<PL::STAGES - 2>();
        __syncthreads();
        {
            const int nxt = it + PL::STAGES - 1;
            if (nxt < ntiles && nxt % QUARTER_TILES == 0) {
                fill_quarters(nxt);
                __syncthreads();
            }
            if (nxt < ntiles) load_tile(nxt, nxt % PL::STAGES);
            cp_async_commit();
        }
        const unsigned char* ks = smem + (it % PL::STAGES) * PL::STAGE_BYTES;
        const unsigned char* vs = ks + PL::TILE_BYTES;
        const int key_base = tile_of(it) * TILE_KEYS;
        // this warp's rows see keys up to qp1 (or qp0): skip a key tile that lies wholly behind or before them (kept first keys are never before them)
        const int warp_hi = pos_lo + min(count - 1, warp * 16 + 15), warp_lo = pos_lo + warp * 16;
        const int warp_first = first_of(warp_lo);
        if (warp * 16 >= count || key_base > warp_hi || (key_base + TILE_KEYS - 1 < warp_first && key_base >= x_keep)) continue;

        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {                                    // 16 keys each
                uint32_t b[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4(b, ks + L::offset(kb * 16 + (mi >> 1) * 8 + r, kk * 2 + (mi & 1)));
                mma_bf16_16816(s[2 * kb], qf[kk], b[0], b[1]);
                mma_bf16_16816(s[2 * kb + 1], qf[kk], b[2], b[3]);
            }
        }
        // Scores stay unscaled here; the scale goes into the exponent's multiply-add.  Only a tile that crosses the
        // diagonal, the window's far edge or the end of the portion needs the per-element limits.
        if (x_softcap > 0.f) {
            const float pre = p.scale / x_softcap;
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = x_softcap * tanh_by_exp(s[j][e] * pre);
        }
        const bool limits = key_base + TILE_KEYS - 1 > warp_lo || warp * 16 + 15 >= count || key_base < first_of(warp_lo + 15);
        if (limits) {
            const int f0 = first_of(qp0), f1 = first_of(qp1);
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int kpos = key_base + j * 8 + 2 * tig + (e & 1);
                    const int qp = e < 2 ? qp0 : qp1;
                    const bool ok = (e < 2 ? v0 : v1) && kpos <= qp && (kpos >= (e < 2 ? f0 : f1) || kpos < x_keep);
                    if (!ok) s[j][e] = -INFINITY;
                }
        }
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            tmax0 = fmaxf(tmax0, fmaxf(s[j][0], s[j][1]));
            tmax1 = fmaxf(tmax1, fmaxf(s[j][2], s[j][3]));
        }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        // m0, m1: running maxima in scaled (base-2) units
        const float mn0 = fmaxf(m0, tmax0 * scale_log2), mn1 = fmaxf(m1, tmax1 * scale_log2);
        // a row that sees nothing yet keeps m = -inf: use 0 as the reference so that exp(-inf - 0) = 0
        const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
        const float c0 = exp2_approx(m0 - ref0), c1 = exp2_approx(m1 - ref1);
        m0 = mn0;
        m1 = mn1;
        uint32_t pf[4][4];
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            const float e00 = exp2_approx(fmaf(s[2 * kb][0], scale_log2, -ref0)), e01 = exp2_approx(fmaf(s[2 * kb][1], scale_log2, -ref0));
            const float e02 = exp2_approx(fmaf(s[2 * kb][2], scale_log2, -ref1)), e03 = exp2_approx(fmaf(s[2 * kb][3], scale_log2, -ref1));
            const float e10 = exp2_approx(fmaf(s[2 * kb + 1][0], scale_log2, -ref0)), e11 = exp2_approx(fmaf(s[2 * kb + 1][1], scale_log2, -ref0));
            const float e12 = exp2_approx(fmaf(s[2 * kb + 1][2], scale_log2, -ref1)), e13 = exp2_approx(fmaf(s[2 * kb + 1][3], scale_log2, -ref1));
            ps0 += e00 + e01 + e10 + e11;
            ps1 += e02 + e03 + e12 + e13;
            pf[kb][0] = pack_bf16(e00, e01);
            pf[kb][1] = pack_bf16(e02, e03);
            pf[kb][2] = pack_bf16(e10, e11);
            pf[kb][3] = pack_bf16(e12, e13);
        }
        l0 = l0 * c0 + ps0;
        l1 = l1 * c1 + ps1;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            acc[i][0] *= c0;
            acc[i][1] *= c0;
            acc[i][2] *= c1;
            acc[i][3] *= c1;
        }
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
#pragma unroll
            for (int nt = 0; nt < HD / 8; nt += 2) {
                uint32_t b[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4_trans(b, vs + L::offset(kb * 16 + (mi & 1) * 8 + r, nt + (mi >> 1)));
                mma_bf16_16816(acc[nt], pf[kb], b[0], b[1]);
                mma_bf16_16816(acc[nt + 1], pf[kb], b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = norm_with_sink(m0, l0, sink2) * x_out_scale, i1 = norm_with_sink(m1, l1, sink2) * x_out_scale;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + 2 * tig;
        if (x_out_f32) {
            if (v0) *reinterpret_cast<float2*>(x_out_f32 + (size_t)(t0 + r0) * p.ldo + (size_t)h * HD + d) = make_float2(acc[i][0] * i0, acc[i][1] * i0);
            if (v1) *reinterpret_cast<float2*>(x_out_f32 + (size_t)(t0 + r1) * p.ldo + (size_t)h * HD + d) = make_float2(acc[i][2] * i1, acc[i][3] * i1);
            continue;
        }
        if (v0) *reinterpret_cast<uint32_t*>(p.out + (size_t)(t0 + r0) * p.ldo + (size_t)h * HD + d) = pack_bf16(acc[i][0] * i0, acc[i][1] * i0);
        if (v1) *reinterpret_cast<uint32_t*>(p.out + (size_t)(t0 + r1) * p.ldo + (size_t)h * HD + d) = pack_bf16(acc[i][2] * i1, acc[i][3] * i1);
    }
}

template <int HD, bool MASKED = false>
int launch_prefill(cudaStream_t stream, const PrefillParams& p, int num_tiles) {
    using PL = PrefillLayout<HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD, MASKED>, cudaFuncAttributeMaxDynamicSharedMemorySize, PL::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(2 * num_tiles, p.num_heads);
    attention_prefill_kernel<HD, MASKED><<<grid, THREADS, PL::SMEM, stream>>>(p);
    return eg_launch_status();
}

}  // namespace

// Head sizes 32, 64, 128, 256 and page sizes that are multiples of 16; anything else
// returns cudaErrorInvalidValue and the caller uses the generic kernel.
// partial_acc / partial_ml: scratch of tokens*heads*splits*(head_dim + 2) floats, and counters: one zeroed int
// per (token, KV head block) (left zero), needed when splits > 1.  seq_context (may be null): per block-table row, the
// number of keys that were in the cache before this step; those may be fetched before the kernel in front has finished.
// token_list (may be null): `tokens` indices of the tokens to work on (scratch and counters are indexed by token index,
// so they cover all tokens of the step either way).
static int attention_paged_any(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache,
                               const int* block_table, int table_stride, const int* token_seq, const int* positions,
                               const int* seq_context, void* out, int ldo, float* partial_acc, float* partial_ml, int tokens, int num_heads,
                               int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride,
                               int num_pages, int window, float scale, int splits, int* status, const void* prefetch,
                               long long prefetch_bytes, int* counters, int use_pdl, unsigned long long* trace, const int* token_list, float sink2,
                               const Params* extras = nullptr) {
    if (tokens <= 0) return 0;
    if (page_size % 16 || num_kv_heads <= 0 || num_heads % num_kv_heads || splits < 1 || tokens > 0x7fffffff ||
        splits > MAX_SPLITS || (splits > 1 && (!partial_acc || !partial_ml || !counters || ldo % 4 || (uintptr_t)out % 8)))
        return (int)cudaErrorInvalidValue;
    Params p{(const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, head_stride, block_table,
             table_stride, token_seq, positions, seq_context, (bf16*)out, ldo, partial_acc, partial_ml, num_heads, num_kv_heads,
             page_size, num_pages, window, splits, scale, status, prefetch_bytes >= 16 ? prefetch : nullptr, prefetch_bytes,
             counters, use_pdl, trace, token_list};
    p.sink2 = sink2;
    if (extras) {
        p.chunk = extras->chunk;
        p.keep_first = (window > 0 || extras->chunk > 0) ? extras->keep_first : 0;
        p.maps = extras->maps;
        p.softcap = extras->softcap;
        p.out_scale = extras->out_scale;
        p.sinks = extras->sinks;
        p.out_f32 = extras->out_f32;
    }
    if (extras) {
        switch (head_dim) {
            case 32: return launch<32, true>(stream, p, tokens);
            case 64: return launch<64, true>(stream, p, tokens);
            case 128: return launch<128, true>(stream, p, tokens);
            default: return (int)cudaErrorInvalidValue;
        }
    }
    switch (head_dim) {
        case 32: return launch<32, false>(stream, p, tokens);
        case 64: return launch<64, false>(stream, p, tokens);
        case 128: return launch<128, false>(stream, p, tokens);
        case 256: return launch<256, false>(stream, p, tokens);
        default: return (int)cudaErrorInvalidValue;
    }
}

EG_API int eg_attention_paged(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache,
                              const int* block_table, int table_stride, const int* token_seq, const int* positions,
                              const int* seq_context, void* out, int ldo, float* partial_acc, float* partial_ml, int tokens, int num_heads,
                              int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride,
                              int num_pages, int window, float scale, int splits, int* status, const void* prefetch,
                              long long prefetch_bytes, int* counters, int use_pdl, unsigned long long* trace, const int* token_list) {
    return attention_paged_any(stream, q, ldq, k_cache, v_cache, block_table, table_stride, token_seq, positions, seq_context, out, ldo, partial_acc,
                               partial_ml, tokens, num_heads, num_kv_heads, head_dim, page_size, page_stride, head_stride, num_pages, window, scale, splits,
                               status, prefetch, prefetch_bytes, counters, use_pdl, trace, token_list, -INFINITY);
}

// The same with a sink: one more term exp(sink_logit) in every softmax's denominator, which has no value.
EG_API int eg_attention_paged_sink(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache,
                                   const int* block_table, int table_stride, const int* token_seq, const int* positions,
                                   const int* seq_context, void* out, int ldo, float* partial_acc, float* partial_ml, int tokens, int num_heads,
                                   int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride,
                                   int num_pages, int window, float scale, int splits, int* status, int* counters, int use_pdl,
                                   const int* token_list, float sink_logit) {
    return attention_paged_any(stream, q, ldq, k_cache, v_cache, block_table, table_stride, token_seq, positions, seq_context, out, ldo, partial_acc,
                               partial_ml, tokens, num_heads, num_kv_heads, head_dim, page_size, page_stride, head_stride, num_pages, window, scale, splits,
                               status, nullptr, 0, counters, use_pdl, nullptr, token_list, sink_logit * 1.4426950408889634f);
}

// Prompt portions in tiles of 64 query tokens: tiles[num_tiles][3] = (block table row, first token, count <= 64);
// the tokens of a tile are consecutive positions of one request.  Head sizes 32, 64, 128; pages of a multiple of 16.
static int attention_prefill_any(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache,
                                 const int* block_table, int table_stride, const int* positions, const int* tiles,
                                 int num_tiles, void* out, int ldo, int num_heads, int num_kv_heads, int head_dim,
                                 int page_size, long long page_stride, long long head_stride, int num_pages, int window,
                                 float scale, int* status, float sink2) {
    if (num_tiles <= 0) return 0;
    if (page_size % 16 || num_kv_heads <= 0 || num_heads % num_kv_heads || num_heads > 65535) return (int)cudaErrorInvalidValue;
    PrefillParams p{(const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, head_stride, block_table,
                    table_stride, positions, tiles, (bf16*)out, ldo, num_heads, num_kv_heads, page_size, num_pages, window,
                    scale, status};
    p.sink2 = sink2;
    switch (head_dim) {
        case 32: return launch_prefill<32>(stream, p, num_tiles);
        case 64: return launch_prefill<64>(stream, p, num_tiles);
        case 128: return launch_prefill<128>(stream, p, num_tiles);
        default: return (int)cudaErrorInvalidValue;
    }
}

EG_API int eg_attention_prefill(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* positions, const int* tiles,
                                int num_tiles, void* out, int ldo, int num_heads, int num_kv_heads, int head_dim,
                                int page_size, long long page_stride, long long head_stride, int num_pages, int window,
                                float scale, int* status) {
    return attention_prefill_any(stream, q, ldq, k_cache, v_cache, block_table, table_stride, positions, tiles, num_tiles, out, ldo, num_heads, num_kv_heads,
                                 head_dim, page_size, page_stride, head_stride, num_pages, window, scale, status, -INFINITY);
}

// The same with a sink: one more term exp(sink_logit) in every softmax's denominator, which has no value.
EG_API int eg_attention_prefill_sink(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache,
                                     const int* block_table, int table_stride, const int* positions, const int* tiles,
                                     int num_tiles, void* out, int ldo, int num_heads, int num_kv_heads, int head_dim,
                                     int page_size, long long page_stride, long long head_stride, int num_pages, int window,
                                     float scale, int* status, float sink_logit) {
    return attention_prefill_any(stream, q, ldq, k_cache, v_cache, block_table, table_stride, positions, tiles, num_tiles, out, ldo, num_heads, num_kv_heads,
                                 head_dim, page_size, page_stride, head_stride, num_pages, window, scale, status, sink_logit * 1.4426950408889634f);
}

// Prompt portions in tiles, with the further masks and score functions of PrefillParams: chunk (keys of the query's own block
// of that many positions), keep_first (the first keys stay visible), softcap, sinks (float32 [num_heads], natural-log logits,
// or null), maps (query row head * maps + map reads key head (head / group) * maps + map; num_heads and num_kv_heads count
// rows and key heads, both planes hold num_kv_heads heads), out_scale; out_dtype EG_BF16, or EG_F32 for float32 rows.
EG_API int eg_attention_prefill_masked(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache, const int* block_table,
                                       int table_stride, const int* positions, const int* tiles, int num_tiles, void* out, int out_dtype, int ldo,
                                       int num_heads, int num_kv_heads, int maps, int head_dim, int page_size, long long page_stride, long long head_stride,
                                       int num_pages, int window, int chunk, int keep_first, float scale, float softcap, const float* sinks, float out_scale,
                                       int* status) {
    if (num_tiles <= 0) return 0;
    if (page_size % 16 || num_kv_heads <= 0 || num_heads % num_kv_heads || num_heads > 65535 || maps < 1 || num_kv_heads % maps || chunk < 0 || keep_first < 0 ||
        softcap < 0.f)
        return (int)cudaErrorInvalidValue;
    PrefillParams p{(const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, head_stride, block_table,
                    table_stride, positions, tiles, (bf16*)out, ldo, num_heads, num_kv_heads, page_size, num_pages, window,
                    scale, status};
    p.chunk = chunk;
    p.keep_first = (window > 0 || chunk > 0) ? keep_first : 0;
    p.maps = maps;
    p.softcap = softcap;
    p.sinks = sinks;
    p.out_scale = out_scale;
    if (out_dtype == EG_F32) p.out_f32 = (float*)out;
    switch (head_dim) {
        case 32: return launch_prefill<32, true>(stream, p, num_tiles);
        case 64: return launch_prefill<64, true>(stream, p, num_tiles);
        case 128: return launch_prefill<128, true>(stream, p, num_tiles);
        default: return (int)cudaErrorInvalidValue;
    }
}

// Single tokens split over their keys, with the further masks and score functions of Params: chunk, keep_first, softcap, sinks
// (float32 [num_heads], natural-log logits, or null), maps (num_heads and num_kv_heads count rows and key heads; both planes
// hold num_kv_heads heads), out_scale; out_dtype EG_BF16, or EG_F32 for float32 rows (ldo a multiple of four then too).
EG_API int eg_attention_paged_masked(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache, const int* block_table,
                                     int table_stride, const int* token_seq, const int* positions, const int* seq_context, void* out, int out_dtype, int ldo,
                                     float* partial_acc, float* partial_ml, int tokens, int num_heads, int num_kv_heads, int maps, int head_dim, int page_size,
                                     long long page_stride, long long head_stride, int num_pages, int window, int chunk, int keep_first, float scale,
                                     float softcap, const float* sinks, float out_scale, int splits, int* status, int* counters, int use_pdl,
                                     const int* token_list) {
    if (maps < 1 || num_kv_heads % maps || chunk < 0 || keep_first < 0 || softcap < 0.f || (out_dtype == EG_F32 && (ldo % 4 || (uintptr_t)out % 16)))
        return (int)cudaErrorInvalidValue;
    Params extras{};
    extras.chunk = chunk;
    extras.keep_first = keep_first;
    extras.maps = maps;
    extras.softcap = softcap;
    extras.out_scale = out_scale;
    extras.sinks = sinks;
    extras.out_f32 = out_dtype == EG_F32 ? (float*)out : nullptr;
    return attention_paged_any(stream, q, ldq, k_cache, v_cache, block_table, table_stride, token_seq, positions, seq_context, out, ldo, partial_acc,
                               partial_ml, tokens, num_heads, num_kv_heads, head_dim, page_size, page_stride, head_stride, num_pages, window, scale, splits,
                               status, nullptr, 0, counters, use_pdl, nullptr, token_list, -INFINITY, &extras);
}
