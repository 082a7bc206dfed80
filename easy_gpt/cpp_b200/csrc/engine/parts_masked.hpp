// Further parts: attention whose mask (window, blocks of positions, kept first tokens), score function (soft cap), softmax (a
// learned sink per head) and heads (two softmax maps a head, one taken off the other) are parameters; a gated delta-rule
// mixer whose decay has a rate per key channel and whose per-token numbers come through low-rank maps; and a mixer that runs
// two mixers side by side on the same input and adds their outputs.  Each takes its sizes, constants and tensor-name
// suffixes from its parameters and knows nothing of the model around it.
#pragma once
#include "parts_delta.hpp"

namespace easygpt::engine {

// ---- attention with mask, score function and softmax as parameters ---------------------------------------------------------
// H heads with `maps` queries each (1 or 2) of `dim` values, G key/value heads (head h reads head h / (H / G)), each with
// `maps` keys of `dim` values and one value of `vdim` values:  q, k, v = W_q h, W_k h, W_v h as ONE product (rows stacked),
// float32 out;  with qk_norm "unit" or "gain", q and k are divided by their root mean square per head and map (norm_eps under
// the root) and, for "gain", multiplied by the tensors .q.norm / .k.norm [dim];  then they are turned by the layer's position
// encoding (a half rotation over its first dimensions);  score = (q . k) * scale, with softcap c: c tanh(score / c);
// position p sees j <= p with p - j < window (if given) and floor(j / chunk) = floor(p / chunk) (if given), and every
// j < keep_first;  the softmax's denominator has one more term exp(sink_h) with `sinks` (tensor .sink [H]);
// with maps = 2 and lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (tensors .lq1 .lk1 .lq2 .lk2 [dim]):
// o = a_1 - lambda a_2, divided by its root mean square over vdim (norm_eps) and multiplied by (1 - diff);
// out = W_o (heads' outputs side by side, times out_scale).  The cache keeps one row (keys | value) per token and key head;
// where dim = vdim it keeps keys and values in planes of their own with a head per (key head, map), the value stored once per
// map: G * maps ordinary key/value heads, which in bfloat16 (heads of 32, 64 or 128) the engine's tensor-core kernels walk: the
// tcgen05 one for prompt portions of 33 tokens and more (heads of 64 and 128, no soft cap), the tiled mma.sync one for shorter
// portions, heads of 32 and capped scores, the split-key one for single tokens; everything else runs on the generic kernel.  With a window
// or a chunk the cache manager gives pages back that no coming token can see, except those of the kept first positions.
// Parameters: hidden_size, heads, kv_heads, dim, vdim, scale, maps, window, chunk, keep_first, softcap, sinks, qk_norm,
// norm_eps, diff, out_scale.  Tensors: .q .k .v .o (+ .q.norm .k.norm, .sink, .lq1 .lk1 .lq2 .lk2).
class MaskedAttention : public Mixer {
public:
    MaskedAttention(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
        : Mixer(p, prefix, std::move(position)), hidden_((int)p.integer("hidden_size")), heads_((int)p.integer("heads")), kv_heads_((int)p.integer("kv_heads")),
          dk_((int)p.integer("dim")), dv_((int)p.integer("vdim")), maps_((int)p.integer("maps", 1)), scale_((float)p.real("scale")),
          window_(p.integer("window", 0)), chunk_(p.integer("chunk", 0)), keep_first_(p.integer("keep_first", 0)), softcap_((float)p.real("softcap", 0.0)),
          sinks_(p.integer("sinks", 0) != 0), norm_kind_(p.text("qk_norm", "none")), norm_eps_((float)p.real("norm_eps", 0.0)), diff_(p.real("diff", 0.0)),
          out_scale_((float)p.real("out_scale", 1.0)) {
        if (hidden_ <= 0 || heads_ <= 0 || kv_heads_ <= 0 || dk_ <= 0 || dv_ <= 0) throw std::invalid_argument("masked attention: sizes must be positive");
        if (heads_ % kv_heads_) throw std::invalid_argument("masked attention: heads must be a multiple of kv_heads");
        if (maps_ != 1 && maps_ != 2) throw std::invalid_argument("masked attention: a head has one map, or two of which the second is taken off the first");
        if (window_ < 0 || chunk_ < 0 || keep_first_ < 0 || softcap_ < 0.f) throw std::invalid_argument("masked attention: window, chunk, keep_first and softcap must not be negative");
        if (keep_first_ > 0 && window_ <= 0 && chunk_ <= 0) keep_first_ = 0;          // all keys are seen anyway
        if (norm_kind_ != "none" && norm_kind_ != "unit" && norm_kind_ != "gain") throw std::invalid_argument("masked attention: qk_norm is 'none', 'unit' or 'gain'");
        if (sinks_ && maps_ != 1) throw std::invalid_argument("masked attention: sinks go with one map a head");
        if (dv_ > 256 || dk_ > 4096) throw std::invalid_argument("masked attention: vdim up to 256 and dim up to 4096 are what the kernels take");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        std::vector<TensorRequest> r = {TensorRequest::matrix(prefix + ".q", (long long)heads_ * maps_ * dk_, hidden_),
                                        TensorRequest::matrix(prefix + ".k", (long long)kv_heads_ * maps_ * dk_, hidden_),
                                        TensorRequest::matrix(prefix + ".v", (long long)kv_heads_ * dv_, hidden_),
                                        TensorRequest::matrix(prefix + ".o", hidden_, (long long)heads_ * dv_)};
        if (norm_kind_ == "gain") {
            r.push_back(TensorRequest::vector(prefix + ".q.norm", dk_).with_init("one"));
            r.push_back(TensorRequest::vector(prefix + ".k.norm", dk_).with_init("one"));
        }
        if (sinks_) r.push_back(TensorRequest::vector(prefix + ".sink", heads_).with_init("zero"));
        if (maps_ == 2)
            for (const char* n : {".lq1", ".lk1", ".lq2", ".lk2"}) r.push_back(TensorRequest::vector(prefix + n, dk_));
        return r;
    }
    void load(const HostTensors& file, DType dtype) override {
        std::vector<float> w;
        for (const char* n : {".q", ".k", ".v"}) {
            const std::vector<float> part = host_floats(need_tensor(file, prefix + n));
            w.insert(w.end(), part.begin(), part.end());
        }
        qkv_ = Linear(w.data(), (heads_ + kv_heads_) * maps_ * dk_ + kv_heads_ * dv_, hidden_, nullptr, dtype);
        out_ = Linear(need_tensor(file, prefix + ".o"), nullptr, dtype);
        if (norm_kind_ == "gain") {
            q_gain_ = upload_f32(file, prefix + ".q.norm");
            k_gain_ = upload_f32(file, prefix + ".k.norm");
        }
        if (sinks_) sink_ = upload_f32(file, prefix + ".sink");
        if (maps_ == 2) {
            auto dot = [&](const char* a, const char* b) {
                const std::vector<float> x = host_floats(need_tensor(file, prefix + a)), y = host_floats(need_tensor(file, prefix + b));
                double s = 0.0;
                for (size_t i = 0; i < x.size(); ++i) s += (double)x[i] * (double)y[i];
                return s;
            };
            lambda_ = (float)(std::exp(dot(".lq1", ".lk1")) - std::exp(dot(".lq2", ".lk2")) + diff_);
        }
        if (position) position->load(file, dtype);
    }
    size_t weight_bytes() const override { return qkv_.weight_bytes() + out_.weight_bytes(); }
    size_t arena_bytes(long long T) const override {
        // partial results of single tokens whose keys are dealt to several CTAs: bounded by the CTAs of a few waves
        const size_t partials = planes() ? plans::PREFILL_PARTS_SCRATCH_BYTES + (size_t)(4 * plans::sm_count() + 64) * 128 * (size_t)(dv_ + 2) * 4 : 0;
        return (size_t)T * ((size_t)qkv_.out_features * 4 + (size_t)heads_ * maps_ * (dk_ + dv_) * 4 + (size_t)heads_ * dv_ * 4 + (size_t)hidden_ * 4) + partials + (1u << 16);
    }
    bool capturable() const override { return true; }
    // keys and values in planes of their own where they have one size (a head per map), else side by side in one row
    bool planes() const { return dk_ == dv_; }
    // the cache may let go of what no coming token sees: the window, or (a chunk never reaches further back than its size) the chunk
    long long kept_back() const {
        if (window_ > 0 && chunk_ > 0) return std::min(window_, chunk_);
        return window_ > 0 ? window_ : chunk_ > 0 ? chunk_ : -1;
    }
    CacheNeed cache_need() const override {
        const CacheNeed n = planes() ? CacheNeed::paged(kv_heads_ * maps_, dk_, kept_back()) : CacheNeed::paged_joint(kv_heads_, maps_ * dk_, dv_, kept_back());
        return n.keeping_first(keep_first_);
    }

    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm*) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        if (cache.group < 0) throw DeviceError("masked attention was handed no paged cache");
        const GroupTables& tables = ctx.groups.at(cache.group);
        const Rows h = in.pending ? in.pending->materialize() : in.rows;
        const Rows proj = qkv_(ctx, h, /*out_f32=*/true);
        HalfRotation rot;
        const bool rotates = position && position->half_rotation(&rot);
        if (position && !rotates) throw DeviceError("masked attention takes a half rotation or no position encoding");
        if (rotates && rot.rotary_dim > dk_) throw DeviceError("masked attention: the rotation covers more than a head");
        const float* table = rotates ? step_rotation_table(ctx, rot) : nullptr;
        const int rows = heads_ * maps_;
        Rows q{ctx.take_rows(T, rows * dk_, dtype), dtype, T, rows * dk_, rows * dk_};
        // where a key's row lies: planes of their own, or keys and value behind one another in a row
        void* values = planes() ? cache.v : (char*)cache.k + (size_t)maps_ * dk_ * dtype_size(dtype);
        const int row_stride = planes() ? dk_ : maps_ * dk_ + dv_;
        launch_check(eg_masked_attention_prepare(ctx.stream, (int)dtype, (const float*)proj.p, proj.ld, table, rotates ? rot.rotary_dim : 0, rot.magnitude,
                                                 tables.slot_map, cache.writes ? cache.k : nullptr, values, row_stride, cache.head_stride, cache.page_size,
                                                 cache.page_stride, (long long)cache.num_pages * cache.page_size, q.p, T, heads_, kv_heads_, maps_, dk_, dv_,
                                                 norm_kind_ == "none" ? -1.f : norm_eps_, norm_kind_ == "gain" ? q_gain_.as<float>() : nullptr,
                                                 norm_kind_ == "gain" ? k_gain_.as<float>() : nullptr, planes() ? 1 : 0, ctx.status), "masked_attention_prepare");
        Rows attn{ctx.take_rows(T, heads_ * dv_, dtype), dtype, T, heads_ * dv_, heads_ * dv_};
        // one map: the heads' outputs at once; two: both maps of every head in float32, then their difference, its norm and its
        // factor in one kernel
        float* both = maps_ == 2 ? ctx.take<float>((size_t)T * rows * dv_) : nullptr;
        void* out = both ? (void*)both : attn.p;
        const DType out_dtype = both ? DType::F32 : dtype;
        const long long ldo = both ? (long long)rows * dv_ : attn.ld;
        const float* sinks = sinks_ ? sink_.as<float>() : nullptr;
        const float factor = both ? 1.0f : out_scale_;
        if (dtype == DType::BF16 && planes() && (dk_ == 32 || dk_ == 64 || dk_ == 128) && cache.page_size % 16 == 0) {
            auto tiled = [&](const int* tiles, int count) {
                launch_check(eg_attention_prefill_masked(ctx.stream, q.p, (int)q.ld, cache.k, cache.v, tables.block_table, tables.table_width, ctx.positions, tiles,
                                                         count, out, (int)out_dtype, (int)ldo, rows, kv_heads_ * maps_, maps_, dk_, cache.page_size, cache.page_stride,
                                                         cache.head_stride, cache.num_pages, (int)window_, (int)chunk_, (int)keep_first_, scale_, softcap_, sinks,
                                                         factor, ctx.status), "attention_prefill_masked");
            };
            // prompt portions in tiles of query tokens, on tcgen05 when they are long enough to fill its 128-row tiles; single
            // tokens (decoding, short entries) split over their keys
            const long long reach = kept_back() < 0 ? ctx.max_context_len : std::min<long long>(ctx.max_context_len, kept_back() + keep_first_ + 255);
            const int key_heads = kv_heads_ * maps_;
            // (with a soft cap the tiled kernel: the cap is a second exponent a score, and the tcgen05 kernel's softmax threads run at
            // the exponent unit's rate already; measured on B200, 8 heads of 128, 2,048 tokens, window 1,024, 64 kept keys: 56 us
            // tiled, 57 us + 11 us for the merge of its parts on tcgen05)
            if (ctx.query_tiles && softcap_ == 0.f && ctx.max_query_len >= plans::TCGEN05_ATTENTION_MIN_QUERY &&
                plans::attention_prefill_tcgen05_takes(dtype, dk_, cache.page_size)) {
                int parts, part_tiles;
                plans::attention_prefill_parts(ctx.num_tiles, rows, dk_, reach, &parts, &part_tiles);
                const size_t slots = (size_t)ctx.num_tiles * rows;
                while (parts > 1 && slots * parts * 128 * (dk_ + 2) * 4 > plans::PREFILL_PARTS_SCRATCH_BYTES) --parts;
                float *partial_o = nullptr, *partial_ml = nullptr;
                if (parts > 1) {
                    partial_o = ctx.take<float>(slots * parts * 128 * dk_);
                    partial_ml = ctx.take<float>(slots * parts * 128 * 2);
                }
                launch_check(eg_attention_prefill_tcgen05_masked(ctx.stream, q.p, q.ld, T, cache.k, cache.v, tables.block_table, tables.table_width, ctx.positions,
                                                                 ctx.query_tiles, ctx.num_tiles, out, (int)out_dtype, ldo, rows, key_heads, maps_, dk_, cache.page_size,
                                                                 cache.page_stride, cache.head_stride, cache.num_pages, (int)window_, (int)chunk_, (int)keep_first_,
                                                                 scale_, sinks, factor, ctx.status, parts, part_tiles, partial_o, partial_ml,
                                                                 ctx.scratch->prefill_queue.as<int>()), "attention_prefill_tcgen05_masked");
            } else if (ctx.query_tiles) {
                tiled(ctx.query_tiles, ctx.num_tiles);
            }
            const int singles = ctx.query_tiles ? ctx.num_small : T;
            if (singles > 0) {
                const int splits = plans::attention_paged_splits(singles, rows, key_heads, reach, dk_);
                float *acc = nullptr, *ml = nullptr;
                int* counters = nullptr;
                if (splits > 1) {
                    acc = ctx.take<float>((size_t)T * rows * splits * dv_);
                    ml = ctx.take<float>((size_t)T * rows * splits * 2);
                    if ((size_t)singles * key_heads * ((rows / key_heads + 15) / 16) > KernelScratch::ATTENTION_COUNTERS)
                        throw DeviceError("a step has more (token, KV head) pairs than the attention's ticket counters");
                    counters = ctx.scratch->attention_counters.as<int>();
                }
                launch_check(eg_attention_paged_masked(ctx.stream, q.p, (int)q.ld, cache.k, cache.v, tables.block_table, tables.table_width, ctx.token_seq,
                                                       ctx.positions, ctx.query_tiles ? nullptr : ctx.seq_context, out, (int)out_dtype, (int)ldo, acc, ml, singles,
                                                       rows, key_heads, maps_, dk_, cache.page_size, cache.page_stride, cache.head_stride, cache.num_pages,
                                                       (int)window_, (int)chunk_, (int)keep_first_, scale_, softcap_, sinks, factor, splits, ctx.status, counters,
                                                       plans::use_pdl(), ctx.query_tiles ? ctx.small_tokens : nullptr), "attention_paged_masked");
            }
        } else {
            launch_check(eg_masked_attention(ctx.stream, (int)dtype, q.p, cache.k, values, row_stride, cache.head_stride, tables.block_table, tables.table_width,
                                             ctx.token_seq, ctx.positions, nullptr, out, (int)out_dtype, ldo, T, heads_, kv_heads_, maps_, dk_, dv_, cache.page_size,
                                             cache.page_stride, cache.num_pages, (int)window_, (int)chunk_, (int)keep_first_, scale_, softcap_, sinks, factor,
                                             planes() ? 1 : 0, ctx.status), "masked_attention");
        }
        if (both)
            launch_check(eg_attention_map_difference(ctx.stream, both, attn.p, (int)dtype, attn.ld, T, heads_, dv_, lambda_, norm_eps_,
                                                     (float)(1.0 - diff_) * out_scale_), "attention_map_difference");
        const Rows o = out_(ctx, attn, /*out_f32=*/true);
        Delta d;
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    int hidden_, heads_, kv_heads_, dk_, dv_, maps_;
    float scale_;
    long long window_, chunk_, keep_first_;
    float softcap_;
    bool sinks_;
    std::string norm_kind_;
    float norm_eps_;
    double diff_;
    float out_scale_, lambda_ = 0.f;
    Linear qkv_, out_;
    DeviceBuffer q_gain_, k_gain_, sink_;
};

// ---- gated delta rule with a decay per key channel ---------------------------------------------------------------------------
// With h the input, H heads of `vdim` values, G key heads of `dim` values (head i reads key head i / (H / G)), K taps:
//   (q | k | v | b | a' | z') = W h as ONE product, float32 out, with a' = A1 h and z' = G1 h the inner values of two low-rank
//   maps;  q, k, v <- silu(conv_K(.)) per channel, causal, continuing from the request's last K-1 inputs;  q^, k^ unit vectors
//   per key head (unit_eps under the root), q^ times dim^(-1/2);  beta = sigmoid(b);
//   g = exp(-exp(A_log_h) softplus(A2 a' + dt_bias)) per head and key channel;  z = G2 z' per head and value channel;
//   S <- diag(g) S;  u = beta (v - S^T k^);  S <- S + k^ u^T;  o = S^T q^   (S [dim, vdim] per head, float32, in the request's slot)
//   out = W_o (o / rms(o) * w * gate(z) * out_scale), rms per head over vdim with eps, gate = sigmoid (or silu).
// The slot holds the convolution's last K-1 inputs [(K-1), channels] and then S [H, vdim, dim], all float32.  The inner sizes of
// the low-rank maps are what the file's tensors have (parameter rank: what random-weights mode writes).
// Parameters: hidden_size, heads, kv_heads, dim, vdim, conv, eps, unit_eps, gate, out_scale, rank.  Tensors: .q .k .v [out, hidden]
// with .q.conv .k.conv .v.conv [channels, K], .b [H, hidden], .A_log [H], .a1 [r, hidden], .a2 [H dim, r], .dt_bias [H dim],
// .g1 [r', hidden], .g2 [H vdim, r'], .norm [vdim], .o [hidden, H vdim].
class ChannelDeltaMixer : public Mixer {
public:
    ChannelDeltaMixer(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
        : Mixer(p, prefix, std::move(position)), hidden_((int)p.integer("hidden_size")), heads_((int)p.integer("heads")), kv_heads_((int)p.integer("kv_heads")),
          dk_((int)p.integer("dim")), dv_((int)p.integer("vdim")), taps_((int)p.integer("conv")), eps_((float)p.real("eps")),
          unit_eps_((float)p.real("unit_eps", 1e-6)), gate_sigmoid_(p.text("gate", "sigmoid") == "sigmoid"), out_scale_((float)p.real("out_scale", 1.0)),
          rank_((int)p.integer("rank", 16)) {
        if (hidden_ <= 0 || heads_ <= 0 || kv_heads_ <= 0 || dk_ <= 0 || dv_ <= 0 || taps_ < 1 || rank_ < 1) throw std::invalid_argument("channel delta: sizes must be positive");
        if (heads_ % kv_heads_) throw std::invalid_argument("channel delta: heads must be a multiple of kv_heads");
        if (p.text("gate", "sigmoid") != "sigmoid" && p.text("gate", "sigmoid") != "silu") throw std::invalid_argument("channel delta: gate is 'sigmoid' or 'silu'");
        int r = 0, l = 0;
        if (!eg_gated_delta_plan(dk_, dv_, &r, &l))
            throw std::invalid_argument("channel delta: dim " + std::to_string(dk_) + " with vdim " + std::to_string(dv_) +
                                        " is beyond what the kernel takes (dim up to 256, vdim up to 4096)");
    }
    int channels() const { return 2 * kv_heads_ * dk_ + heads_ * dv_; }
    std::vector<TensorRequest> tensor_requests() const override {
        const long long qk = (long long)kv_heads_ * dk_, v = (long long)heads_ * dv_, decays = (long long)heads_ * dk_;
        return {TensorRequest::matrix(prefix + ".q", qk, hidden_), TensorRequest::matrix(prefix + ".q.conv", qk, taps_),
                TensorRequest::matrix(prefix + ".k", qk, hidden_), TensorRequest::matrix(prefix + ".k.conv", qk, taps_),
                TensorRequest::matrix(prefix + ".v", v, hidden_), TensorRequest::matrix(prefix + ".v.conv", v, taps_),
                TensorRequest::matrix(prefix + ".b", heads_, hidden_), TensorRequest::vector(prefix + ".A_log", heads_).with_init("log_decay"),
                TensorRequest::matrix(prefix + ".a1", rank_, hidden_).with_free_dim(0), TensorRequest::matrix(prefix + ".a2", decays, rank_).with_free_dim(1),
                TensorRequest::vector(prefix + ".dt_bias", decays).with_init("step_bias"),
                TensorRequest::matrix(prefix + ".g1", rank_, hidden_).with_free_dim(0), TensorRequest::matrix(prefix + ".g2", v, rank_).with_free_dim(1),
                TensorRequest::vector(prefix + ".norm", dv_).with_init("one"), TensorRequest::matrix(prefix + ".o", hidden_, v)};
    }
    void load(const HostTensors& file, DType dtype) override {
        const StoredTensor &a1 = need_tensor(file, prefix + ".a1"), &a2 = need_tensor(file, prefix + ".a2"), &g1 = need_tensor(file, prefix + ".g1"),
                           &g2 = need_tensor(file, prefix + ".g2");
        ra_ = (int)a1.shape[0];
        rg_ = (int)g1.shape[0];
        if (a2.shape[1] != ra_ || g2.shape[1] != rg_)
            throw WeightError("the two halves of a low-rank map under '" + prefix + "' differ in their inner size");
        std::vector<float> w, cw;
        for (const char* n : {".q", ".k", ".v", ".b", ".a1", ".g1"}) {
            const std::vector<float> part = host_floats(need_tensor(file, prefix + n));
            w.insert(w.end(), part.begin(), part.end());
        }
        in_ = Linear(w.data(), channels() + heads_ + ra_ + rg_, hidden_, nullptr, dtype);
        // the second halves read rows padded to a multiple of eight values (a 16-byte boundary for every row): their weights are padded alike
        auto padded_second = [&](const StoredTensor& t, int r, int rp) {
            const std::vector<float> src = host_floats(t);
            const size_t rows = (size_t)t.shape[0];
            std::vector<float> dst(rows * rp, 0.f);
            for (size_t i = 0; i < rows; ++i) std::memcpy(&dst[i * rp], &src[i * r], (size_t)r * 4);
            return Linear(dst.data(), (int)rows, rp, nullptr, dtype);
        };
        a2_ = padded_second(a2, ra_, padded(ra_));
        g2_ = padded_second(g2, rg_, padded(rg_));
        for (const char* n : {".q.conv", ".k.conv", ".v.conv"}) {
            const std::vector<float> part = host_floats(need_tensor(file, prefix + n));
            cw.insert(cw.end(), part.begin(), part.end());
        }
        conv_w_ = upload(cw.data(), cw.size(), DType::F32);
        a_log_ = upload_f32(file, prefix + ".A_log");
        dt_bias_ = upload_f32(file, prefix + ".dt_bias");
        norm_w_ = upload_f32(file, prefix + ".norm");
        out_ = Linear(need_tensor(file, prefix + ".o"), nullptr, dtype);
    }
    static int padded(int r) { return (r + 7) / 8 * 8; }
    size_t weight_bytes() const override {
        return in_.weight_bytes() + a2_.weight_bytes() + g2_.weight_bytes() + out_.weight_bytes() + (size_t)channels() * taps_ * 4;
    }
    size_t arena_bytes(long long T) const override {
        return (size_t)T * ((size_t)in_.out_features * 4 + (size_t)channels() * 4 + (size_t)(padded(ra_) + padded(rg_)) * 4 + (size_t)heads_ * dk_ * 4 +
                            (size_t)heads_ * dv_ * 12 + (size_t)heads_ * 16 + (size_t)hidden_ * 4) + (1u << 16);
    }
    bool capturable() const override { return true; }
    long long conv_floats() const { return (long long)(taps_ - 1) * channels(); }
    long long slot_floats() const { return conv_floats() + (long long)heads_ * dv_ * dk_; }
    CacheNeed cache_need() const override { return CacheNeed::state({slot_floats()}); }

    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm*) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        if (!cache.state || cache.state_bytes_per_slot != (size_t)slot_floats() * 4) throw DeviceError("a channel delta mixer was handed no state of its shape");
        if (!cache.writes) throw DeviceError("a channel delta mixer cannot read another entry's state without advancing it");
        const Rows h = in.pending ? in.pending->materialize() : in.rows;
        const Rows proj = in_(ctx, h, /*out_f32=*/true);                            // [T, q | k | v | b | a' | z'] float32
        float* state = (float*)cache.state;
        const long long slot = slot_floats();
        const int C = channels();
        float* u = ctx.take<float>((size_t)T * C);                                  // convolved and activated q | k | v
        launch_check(eg_conv_silu(ctx.stream, (int)DType::F32, proj.p, proj.ld, conv_w_.as<float>(), nullptr, state, slot, ctx.token_seq, ctx.seq_starts,
                                  ctx.seq_slots, u, C, T, C, taps_), "conv_silu");
        launch_check(eg_conv_state(ctx.stream, (int)DType::F32, proj.p, proj.ld, state, slot, ctx.seq_starts, ctx.seq_slots, ctx.num_seqs, C, taps_), "conv_state");
        // the low-rank maps' second halves: their inputs are columns of the first product's float32 output
        const int b_col = C, a_col = C + heads_, z_col = a_col + ra_;
        const Rows decay = second_half(ctx, a2_, (const float*)proj.p + a_col, proj.ld, ra_, T);     // [T, H dim]: logits, then the decays
        const Rows gate = second_half(ctx, g2_, (const float*)proj.p + z_col, proj.ld, rg_, T);      // [T, H vdim]
        Rows y{ctx.take_rows(T, heads_ * dv_, dtype), dtype, T, heads_ * dv_, heads_ * dv_};
        const int qk = kv_heads_ * dk_;
        const int slices = plans::delta_column_slices(ctx.num_seqs, heads_, dv_);
        float* o_raw = ctx.take<float>((size_t)T * heads_ * dv_);
        float* aux = ctx.take<float>((size_t)T * heads_ * 4);
        launch_check(eg_gated_delta_channel(ctx.stream, u, C, 0, qk, 2 * qk, (const float*)proj.p, proj.ld, b_col, (float*)decay.p, decay.ld, (const float*)gate.p,
                                            gate.ld, a_log_.as<float>(), dt_bias_.as<float>(), norm_w_.as<float>(), state, slot, conv_floats(), ctx.seq_starts,
                                            ctx.seq_slots, y.p, (int)dtype, y.ld, aux, o_raw, slices, T, ctx.num_seqs, heads_, kv_heads_, dk_, dv_, unit_eps_, eps_,
                                            gate_sigmoid_ ? 1 : 0, out_scale_), "gated_delta_channel");
        const Rows o = out_(ctx, y, /*out_f32=*/true);
        Delta d;
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    // second (cols float32 values a row, lds apart) -> float32 [T, second.out_features]: the columns become rows of the compute
    // dtype, padded with zeros to the product's inner size
    Rows second_half(const StepContext& ctx, const Linear& second, const float* cols, long long lds, int r, int T) const {
        const int rp = second.in_features;
        Rows x{ctx.take_rows(T, rp, ctx.dtype), ctx.dtype, T, rp, rp};
        launch_check(eg_convert_columns(ctx.stream, cols, lds, x.p, (int)ctx.dtype, rp, T, r, rp), "convert_columns");
        return second(ctx, x, /*out_f32=*/true);
    }

    int hidden_, heads_, kv_heads_, dk_, dv_, taps_;
    float eps_, unit_eps_;
    bool gate_sigmoid_;
    float out_scale_;
    int rank_, ra_ = 0, rg_ = 0;
    Linear in_, a2_, g2_, out_;
    DeviceBuffer conv_w_, a_log_, dt_bias_, norm_w_;
};

// ---- two mixers side by side --------------------------------------------------------------------------------------------------
// out = left(h) + right(h): both read the same rows; their weights on the sum are parameters of the two mixers themselves
// (out_scale), so the sum costs one addition.  The two are built from the registry by kind; the first may keep pages, the
// second a state (or either nothing): the cache manager gives the pair pages AND a slot.
// Parameters: left_kind, right_kind, and the two mixers' own parameters under "left." and "right.".  Tensors: the two mixers'
// under <prefix>.left and <prefix>.right.
class SideBySideMixer : public Mixer {
public:
    SideBySideMixer(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position);
    std::vector<TensorRequest> tensor_requests() const override {
        std::vector<TensorRequest> r = left_->tensor_requests();
        for (auto& t : right_->tensor_requests()) r.push_back(t);
        return r;
    }
    void load(const HostTensors& file, DType dtype) override {
        left_->load(file, dtype);
        right_->load(file, dtype);
    }
    size_t weight_bytes() const override { return left_->weight_bytes() + right_->weight_bytes(); }
    size_t arena_bytes(long long T) const override { return left_->arena_bytes(T) + right_->arena_bytes(T); }
    bool capturable() const override { return left_->capturable() && right_->capturable(); }
    CacheNeed cache_need() const override {
        const CacheNeed l = left_->cache_need(), r = right_->cache_need();
        if (l.kind == CacheNeed::None) return r;
        if (r.kind == CacheNeed::None) return l;
        if (l.kind == CacheNeed::PagedKV && r.kind == CacheNeed::State && l.state_shape.empty()) return l.with_state(r.state_shape, r.state_dtype);
        throw std::invalid_argument("two mixers side by side: the first may keep pages and the second a state");
    }
    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm*) override {
        const Rows h = in.pending ? in.pending->materialize() : in.rows;
        PartInput rows;
        rows.rows = h;
        // each half sees its own part of the cache: the pages, or the slot
        CacheView paged = cache, slot = cache;
        paged.state = nullptr;
        paged.state_bytes_per_slot = 0;
        slot.group = -1;
        slot.k = slot.v = nullptr;
        const bool left_paged = left_->cache_need().kind == CacheNeed::PagedKV;
        Delta a = left_->forward(ctx, rows, left_paged ? paged : slot, nullptr);
        Delta b = right_->forward(ctx, rows, left_paged ? slot : paged, nullptr);
        if (a.has_pre() || b.has_pre() || a.scale || b.scale || a.dtype != DType::F32) throw DeviceError("two mixers side by side hand back plain float32 outputs");
        launch_check(eg_add_into_f32(ctx.stream, (float*)a.p, b.p, (int)b.dtype, (long long)ctx.num_tokens * h.cols), "add");
        return a;
    }

private:
    std::shared_ptr<Mixer> left_, right_;
};

inline SideBySideMixer::SideBySideMixer(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
    : Mixer(p, prefix, position) {
    PartRegistry& reg = PartRegistry::instance();
    left_ = PartRegistry::find(reg.mixers, "mixer", p.text("left_kind"))(p.sub("left."), prefix + ".left", position);
    right_ = PartRegistry::find(reg.mixers, "mixer", p.text("right_kind"))(p.sub("right."), prefix + ".right", position);
}

inline void register_masked_parts() {
    PartRegistry& r = PartRegistry::instance();
    if (r.mixers.count("masked_attention")) return;
    r.mixers["masked_attention"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<MaskedAttention>(p, prefix, std::move(pos));
    };
    r.mixers["channel_delta"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<ChannelDeltaMixer>(p, prefix, std::move(pos));
    };
    r.mixers["side_by_side"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<SideBySideMixer>(p, prefix, std::move(pos));
    };
}

}  // namespace easygpt::engine
