// Further parts: a token shift in front of a mixer, attention over a sliding window with a sink in its softmax and keys
// and values of sizes of their own, a gated delta-rule mixer (a matrix of state per head instead of cached keys), and a
// dense feed-forward with the xIELU activation.  Each takes its sizes, constants and tensor-name suffixes from its
// parameters and knows nothing of the model around it.
#pragma once
#include "parts.hpp"

namespace easygpt::engine {

inline DeviceBuffer upload_f32(const HostTensors& file, const std::string& name) {
    const std::vector<float> v = host_floats(need_tensor(file, name));
    return upload(v.data(), v.size(), DType::F32);
}

// ---- token shift ---------------------------------------------------------------------------------------------------------
// out[t] = h[t] + (h[t-1] - h[t]) * mu, element by element, h[t-1] the normed row of the token in front of t in its request
// (zeros in front of the first); the request's slot keeps the last row between steps, in float32.
// Parameters: size.  The tensor is the one named by the prefix itself, [size].
class TokenShift : public Shift {
public:
    TokenShift(const Params& p, const std::string& prefix) : Shift(p, prefix), size_((int)p.integer("size")) {
        if (size_ <= 0) throw std::invalid_argument("a token shift's size must be positive");
    }
    std::vector<TensorRequest> tensor_requests() const override { return {TensorRequest::vector(prefix, size_).with_init("half")}; }
    void load(const HostTensors& file, DType) override { mu_ = upload_f32(file, prefix); }
    size_t weight_bytes() const override { return (size_t)size_ * 4; }
    bool capturable() const override { return true; }
    long long state_floats() const override { return size_; }
    void forward(const StepContext& ctx, const float* rows, float* state, long long slot_floats, void* out, DType out_dtype) const override {
        launch_check(eg_token_shift(ctx.stream, rows, mu_.as<float>(), state, slot_floats, ctx.token_seq, ctx.seq_starts, ctx.seq_slots, out, (int)out_dtype,
                                    ctx.num_tokens, size_), "token_shift");
    }
    bool forward_rms(const StepContext& ctx, const float* residual, const float* gain, float eps, float* state, long long slot_floats, void* out,
                     void* plain_out, DType out_dtype) const override {
        if (plain_out) return false;        // the fused kernel leaves the mixed rows only
        launch_check(eg_rmsnorm_shift(ctx.stream, residual, gain, eps, mu_.as<float>(), state, slot_floats, ctx.token_seq, ctx.seq_starts, ctx.seq_slots, out,
                                      (int)out_dtype, ctx.num_tokens, size_), "rmsnorm_shift");
        return true;
    }

private:
    int size_;
    DeviceBuffer mu_;
};

// ---- attention over a window, with a sink ------------------------------------------------------------------------------------
// H query heads of `dim` values, G key/value heads (query head h reads head h / (H / G)) with keys of `dim` and values of
// `vdim` values:  q, k, v = W_q h, W_k h, W_v h as ONE product (rows stacked), float32 out;  q and k are turned by the layer's
// position encoding (a half rotation over its first dimensions, with the encoding's factor on cos and sin) and then, with
// unit_eps given, divided by their root mean square per head;  score = (q . k) * scale over the last `window` positions
// (all, if none is given);  weights = exp(s_j) / (exp(sink_logit) + sum exp(s_i)) if a sink logit is given, else the plain
// softmax;  out = W_o (heads' values side by side).  The cache keeps one row (key | value) per token and key head; where
// dim == vdim it keeps keys and values in planes of their own, the layout of the engine's tensor-core attention kernels,
// which then do the work in bfloat16 (prompt portions on tcgen05 or mma.sync tiles, single tokens split over their keys),
// with the sink as one more term of their final sums.
// Parameters: hidden_size, heads, kv_heads, dim, vdim, scale, window, sink_logit, unit_eps.  Tensors: .q .k .v .o.
class SinkAttention : public Mixer {
public:
    SinkAttention(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
        : Mixer(p, prefix, std::move(position)), hidden_((int)p.integer("hidden_size")), heads_((int)p.integer("heads")), kv_heads_((int)p.integer("kv_heads")),
          dk_((int)p.integer("dim")), dv_((int)p.integer("vdim")), scale_((float)p.real("scale")), window_(p.has("window") ? p.integer("window") : -1),
          has_sink_(p.has("sink_logit")), sink_(p.has("sink_logit") ? (float)p.real("sink_logit") : 0.f),
          unit_eps_(p.has("unit_eps") ? (float)p.real("unit_eps") : -1.f) {
        if (hidden_ <= 0 || heads_ <= 0 || kv_heads_ <= 0 || dk_ <= 0 || dv_ <= 0) throw std::invalid_argument("sink attention: sizes must be positive");
        if (heads_ % kv_heads_) throw std::invalid_argument("sink attention: heads must be a multiple of kv_heads");
        if (p.has("window") && window_ <= 0) throw std::invalid_argument("sink attention: window must be positive");
        if (dv_ > 256 || dk_ > 4096) throw std::invalid_argument("sink attention: vdim up to 256 and dim up to 4096 are what the kernels take");
        if (p.has("unit_eps") && unit_eps_ < 0.f) throw std::invalid_argument("sink attention: unit_eps must not be negative");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        return {TensorRequest::matrix(prefix + ".q", (long long)heads_ * dk_, hidden_), TensorRequest::matrix(prefix + ".k", (long long)kv_heads_ * dk_, hidden_),
                TensorRequest::matrix(prefix + ".v", (long long)kv_heads_ * dv_, hidden_), TensorRequest::matrix(prefix + ".o", hidden_, (long long)heads_ * dv_)};
    }
    void load(const HostTensors& file, DType dtype) override {
        std::vector<float> w;
        for (const char* n : {".q", ".k", ".v"}) {
            const std::vector<float> part = host_floats(need_tensor(file, prefix + n));
            w.insert(w.end(), part.begin(), part.end());
        }
        qkv_ = Linear(w.data(), (heads_ + kv_heads_) * dk_ + kv_heads_ * dv_, hidden_, nullptr, dtype);
        out_ = Linear(need_tensor(file, prefix + ".o"), nullptr, dtype);
        if (position) position->load(file, dtype);
    }
    size_t weight_bytes() const override { return qkv_.weight_bytes() + out_.weight_bytes(); }
    size_t arena_bytes(long long T) const override {
        // partial results of an attention whose keys are shared by several CTAs: as the engine's attention sizes them
        const size_t partials = plans::PREFILL_PARTS_SCRATCH_BYTES + (size_t)(4 * plans::sm_count() + 64) * 128 * (size_t)(dv_ + 2) * 4;
        return (size_t)T * ((size_t)qkv_.out_features * 4 + (size_t)heads_ * (dk_ + dv_) * 4 + (size_t)hidden_ * 4) + (planes() ? partials : 0) + (1u << 16);
    }
    bool capturable() const override { return true; }
    // keys and values in planes of their own where their sizes are equal, else side by side in one row
    bool planes() const { return dk_ == dv_; }
    CacheNeed cache_need() const override { return planes() ? CacheNeed::paged(kv_heads_, dk_, window_) : CacheNeed::paged_joint(kv_heads_, dk_, dv_, window_); }

    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm*) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        if (cache.group < 0) throw DeviceError("sink attention was handed no paged cache");
        const GroupTables& tables = ctx.groups.at(cache.group);
        const Rows h = in.pending ? in.pending->materialize() : in.rows;
        const Rows proj = qkv_(ctx, h, /*out_f32=*/true);
        HalfRotation rot;
        const bool rotates = position && position->half_rotation(&rot);
        if (position && !rotates) throw DeviceError("sink attention takes a half rotation or no position encoding");
        if (rotates && rot.rotary_dim > dk_) throw DeviceError("sink attention: the rotation covers more than a head");
        const float* table = rotates ? step_rotation_table(ctx, rot) : nullptr;
        Rows q{ctx.take_rows(T, heads_ * dk_, dtype), dtype, T, heads_ * dk_, heads_ * dk_};
        // where a key's row lies: planes of their own, or behind one another in a row of dim + vdim values
        void* values = planes() ? cache.v : (char*)cache.k + (size_t)dk_ * dtype_size(dtype);
        const int row_stride = planes() ? dk_ : dk_ + dv_;
        launch_check(eg_sink_attention_prepare(ctx.stream, (int)dtype, (const float*)proj.p, proj.ld, table, rotates ? rot.rotary_dim : 0, rot.magnitude,
                                               tables.slot_map, cache.writes ? cache.k : nullptr, values, row_stride, cache.head_stride, cache.page_size,
                                               cache.page_stride, (long long)cache.num_pages * cache.page_size, q.p, T, heads_, kv_heads_, dk_, dv_, unit_eps_,
                                               ctx.status), "sink_attention_prepare");
        Rows attn{ctx.take_rows(T, heads_ * dv_, dtype), dtype, T, heads_ * dv_, heads_ * dv_};
        const int window = window_ < 0 ? 0 : (int)window_;
        const long long longest = window_ < 0 ? ctx.max_context_len : std::min<long long>(ctx.max_context_len, window_ + 255);
        if (!has_sink_ || !planes() || !plans::attention_paged_takes(dtype, dk_, cache.page_size)) {
            launch_check(eg_sink_attention(ctx.stream, (int)dtype, q.p, cache.k, values, row_stride, cache.head_stride, tables.block_table, tables.table_width,
                                           ctx.token_seq, ctx.positions, nullptr, attn.p, attn.ld, T, heads_, kv_heads_, dk_, dv_, cache.page_size,
                                           cache.page_stride, cache.num_pages, window, scale_, has_sink_ ? 1 : 0, sink_, ctx.status), "sink_attention");
        } else if (ctx.query_tiles && plans::attention_prefill_takes(dtype, dk_, cache.page_size)) {
            // prompt portions in tiles of query tokens, on tcgen05 when they are long enough to fill its 128-row tiles
            if (ctx.max_query_len >= plans::TCGEN05_ATTENTION_MIN_QUERY && plans::attention_prefill_tcgen05_takes(dtype, dk_, cache.page_size)) {
                int parts, part_tiles;
                plans::attention_prefill_parts(ctx.num_tiles, heads_, dk_, longest, &parts, &part_tiles);
                const size_t slots = (size_t)ctx.num_tiles * heads_;
                while (parts > 1 && slots * parts * 128 * (dk_ + 2) * 4 > plans::PREFILL_PARTS_SCRATCH_BYTES) --parts;
                float *partial_o = nullptr, *partial_ml = nullptr;
                if (parts > 1) {
                    partial_o = ctx.take<float>(slots * parts * 128 * dk_);
                    partial_ml = ctx.take<float>(slots * parts * 128 * 2);
                }
                launch_check(eg_attention_prefill_tcgen05_sink(ctx.stream, q.p, q.ld, T, cache.k, cache.v, tables.block_table, tables.table_width, ctx.positions,
                                                               ctx.query_tiles, ctx.num_tiles, attn.p, attn.ld, heads_, kv_heads_, dk_, cache.page_size,
                                                               cache.page_stride, cache.head_stride, cache.num_pages, window, scale_, ctx.status, parts, part_tiles,
                                                               partial_o, partial_ml, ctx.scratch->prefill_queue.as<int>(), sink_), "attention_prefill_tcgen05_sink");
            } else {
                launch_check(eg_attention_prefill_sink(ctx.stream, q.p, (int)q.ld, cache.k, cache.v, tables.block_table, tables.table_width, ctx.positions,
                                                       ctx.query_tiles, ctx.num_tiles, attn.p, (int)attn.ld, heads_, kv_heads_, dk_, cache.page_size,
                                                       cache.page_stride, cache.head_stride, cache.num_pages, window, scale_, ctx.status, sink_),
                             "attention_prefill_sink");
            }
            if (ctx.small_tokens)      // the decoded tokens beside them: token by token, split over their keys
                paged(ctx, q, cache, tables, attn, ctx.num_small, plans::attention_paged_splits(ctx.num_small, heads_, kv_heads_, longest, dk_), window, nullptr,
                      ctx.small_tokens);
        } else {
            paged(ctx, q, cache, tables, attn, T, plans::attention_paged_splits(T, heads_, kv_heads_, longest, dk_), window, ctx.seq_context, nullptr);
        }
        const Rows o = out_(ctx, attn, /*out_f32=*/true);
        Delta d;
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    void paged(const StepContext& ctx, const Rows& q, const CacheView& cache, const GroupTables& tables, const Rows& attn, int tokens, int splits, int window,
               const int* seq_context, const int* token_list) const {
        float *acc = nullptr, *ml = nullptr;
        int* counters = nullptr;
        if (splits > 1) {
            const size_t T = (size_t)ctx.num_tokens;
            acc = ctx.take<float>(T * heads_ * splits * dv_);
            ml = ctx.take<float>(T * heads_ * splits * 2);
            if ((size_t)tokens * kv_heads_ * ((heads_ / kv_heads_ + 15) / 16) > KernelScratch::ATTENTION_COUNTERS)
                throw DeviceError("a step has more (token, KV head) pairs than the attention's ticket counters");
            counters = ctx.scratch->attention_counters.as<int>();
        }
        launch_check(eg_attention_paged_sink(ctx.stream, q.p, (int)q.ld, cache.k, cache.v, tables.block_table, tables.table_width, ctx.token_seq, ctx.positions,
                                             seq_context, attn.p, (int)attn.ld, acc, ml, tokens, heads_, kv_heads_, dk_, cache.page_size, cache.page_stride,
                                             cache.head_stride, cache.num_pages, window, scale_, splits, ctx.status, counters, plans::use_pdl(), token_list, sink_),
                     "attention_paged_sink");
    }

    int hidden_, heads_, kv_heads_, dk_, dv_;
    float scale_;
    long long window_;
    bool has_sink_;
    float sink_, unit_eps_;
    Linear qkv_, out_;
};

// ---- gated delta rule -----------------------------------------------------------------------------------------------------------
// With h the input, H heads of `vdim` values, G key heads of `dim` values (head i reads key head i / (H / G)), K taps:
//   (q | k | v | z | b | a) = W h as ONE product, float32 out;  q, k, v <- silu(conv_K(.)) per channel, causal, continuing from
//   the request's last K-1 inputs;  q^, k^ unit vectors per key head (unit_eps under the root), q^ times dim^(-1/2);
//   beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)) per head;
//   S <- g S;  u = beta (v - S^T k^);  S <- S + k^ u^T;  o = S^T q^   (S [dim, vdim] per head, float32, in the request's slot)
//   out = W_o (o / rms(o) * w * silu(z)), rms per head over vdim with eps.
// The slot holds the convolution's last K-1 inputs [(K-1), channels] and then S [H, vdim, dim], all float32.
// Parameters: hidden_size, heads, kv_heads, dim, vdim, conv, eps, unit_eps.  Tensors: .q .k .v [out, hidden] with .q.conv
// .k.conv .v.conv [channels, K], .b .a [H, hidden], .A_log .dt_bias [H], .norm [vdim], .g [H vdim, hidden], .o [hidden, H vdim].
class GatedDeltaMixer : public Mixer {
public:
    GatedDeltaMixer(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
        : Mixer(p, prefix, std::move(position)), hidden_((int)p.integer("hidden_size")), heads_((int)p.integer("heads")), kv_heads_((int)p.integer("kv_heads")),
          dk_((int)p.integer("dim")), dv_((int)p.integer("vdim")), taps_((int)p.integer("conv")), eps_((float)p.real("eps")),
          unit_eps_(p.has("unit_eps") ? (float)p.real("unit_eps") : 1e-6f) {
        if (hidden_ <= 0 || heads_ <= 0 || kv_heads_ <= 0 || dk_ <= 0 || dv_ <= 0 || taps_ < 1) throw std::invalid_argument("gated delta: sizes must be positive");
        if (heads_ % kv_heads_) throw std::invalid_argument("gated delta: heads must be a multiple of kv_heads");
        int r = 0, l = 0;
        if (!eg_gated_delta_plan(dk_, dv_, &r, &l))
            throw std::invalid_argument("gated delta: dim " + std::to_string(dk_) + " with vdim " + std::to_string(dv_) +
                                        " is beyond what the kernel takes (dim up to 256, vdim up to 4096)");
    }
    int channels() const { return 2 * kv_heads_ * dk_ + heads_ * dv_; }
    std::vector<TensorRequest> tensor_requests() const override {
        const long long qk = (long long)kv_heads_ * dk_, v = (long long)heads_ * dv_;
        return {TensorRequest::matrix(prefix + ".q", qk, hidden_), TensorRequest::matrix(prefix + ".q.conv", qk, taps_),
                TensorRequest::matrix(prefix + ".k", qk, hidden_), TensorRequest::matrix(prefix + ".k.conv", qk, taps_),
                TensorRequest::matrix(prefix + ".v", v, hidden_), TensorRequest::matrix(prefix + ".v.conv", v, taps_),
                TensorRequest::matrix(prefix + ".b", heads_, hidden_), TensorRequest::matrix(prefix + ".a", heads_, hidden_),
                TensorRequest::vector(prefix + ".A_log", heads_).with_init("log_decay"), TensorRequest::vector(prefix + ".dt_bias", heads_).with_init("step_bias"),
                TensorRequest::vector(prefix + ".norm", dv_).with_init("one"), TensorRequest::matrix(prefix + ".g", v, hidden_),
                TensorRequest::matrix(prefix + ".o", hidden_, v)};
    }
    void load(const HostTensors& file, DType dtype) override {
        std::vector<float> w, cw;
        for (const char* n : {".q", ".k", ".v", ".g", ".b", ".a"}) {
            const std::vector<float> part = host_floats(need_tensor(file, prefix + n));
            w.insert(w.end(), part.begin(), part.end());
        }
        in_ = Linear(w.data(), channels() + heads_ * dv_ + 2 * heads_, hidden_, nullptr, dtype);
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
    size_t weight_bytes() const override { return in_.weight_bytes() + out_.weight_bytes() + (size_t)channels() * taps_ * 4; }
    size_t arena_bytes(long long T) const override {
        return (size_t)T * ((size_t)in_.out_features * 4 + (size_t)channels() * 4 + (size_t)heads_ * dv_ * 8 + (size_t)heads_ * 16 + (size_t)hidden_ * 4) + (1u << 16);
    }
    bool capturable() const override { return true; }
    long long conv_floats() const { return (long long)(taps_ - 1) * channels(); }
    long long slot_floats() const { return conv_floats() + (long long)heads_ * dv_ * dk_; }
    CacheNeed cache_need() const override { return CacheNeed::state({slot_floats()}); }

    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm*) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        if (!cache.state || cache.state_bytes_per_slot != (size_t)slot_floats() * 4) throw DeviceError("a gated delta mixer was handed no state of its shape");
        if (!cache.writes) throw DeviceError("a gated delta mixer cannot read another entry's state without advancing it");
        const Rows h = in.pending ? in.pending->materialize() : in.rows;
        const Rows proj = in_(ctx, h, /*out_f32=*/true);                            // [T, q | k | v | z | b | a] float32
        float* state = (float*)cache.state;
        const long long slot = slot_floats();
        const int C = channels();
        float* u = ctx.take<float>((size_t)T * C);                                  // convolved and activated q | k | v
        launch_check(eg_conv_silu(ctx.stream, (int)DType::F32, proj.p, proj.ld, conv_w_.as<float>(), nullptr, state, slot, ctx.token_seq, ctx.seq_starts,
                                  ctx.seq_slots, u, C, T, C, taps_), "conv_silu");
        launch_check(eg_conv_state(ctx.stream, (int)DType::F32, proj.p, proj.ld, state, slot, ctx.seq_starts, ctx.seq_slots, ctx.num_seqs, C, taps_), "conv_state");
        Rows y{ctx.take_rows(T, heads_ * dv_, dtype), dtype, T, heads_ * dv_, heads_ * dv_};
        const int qk = kv_heads_ * dk_, z_col = C, b_col = C + heads_ * dv_, a_col = b_col + heads_;
        // few (entry, head) pairs: a head's columns are dealt to several blocks (they do not depend on one another), and the
        // norm over a head's outputs becomes a kernel of its own.  The count depends on the step's size alone.
        const int slices = plans::delta_column_slices(ctx.num_seqs, heads_, dv_);
        float* o_raw = ctx.take<float>((size_t)T * heads_ * dv_);                   // raw outputs, where no single block holds a head
        float* aux = ctx.take<float>((size_t)T * heads_ * 4);                       // beta, g, k . q per token and head
        launch_check(eg_gated_delta(ctx.stream, u, C, 0, qk, 2 * qk, (const float*)proj.p, proj.ld, b_col, a_col, z_col, a_log_.as<float>(), dt_bias_.as<float>(),
                                    norm_w_.as<float>(), state, slot, conv_floats(), ctx.seq_starts, ctx.seq_slots, y.p, (int)dtype, y.ld, aux, o_raw, slices, T,
                                    ctx.num_seqs, heads_, kv_heads_, dk_, dv_, unit_eps_, eps_), "gated_delta");
        const Rows o = out_(ctx, y, /*out_f32=*/true);
        Delta d;
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    int hidden_, heads_, kv_heads_, dk_, dv_, taps_;
    float eps_, unit_eps_;
    Linear in_, out_;
    DeviceBuffer conv_w_, a_log_, dt_bias_, norm_w_;
};

// ---- dense feed-forward with xIELU: down(act(up h)), act(z) = softplus(p) z^2 + z / 2 for z > 0 and
// (1/2 + softplus(q)) (e^z - 1 - z) + z / 2 for z <= 0, with the two numbers (p, q) of the tensor .act.
// Parameters: hidden_size, ff.  Tensors: .up [ff, hidden], .down [hidden, ff], .act [2] ------------------------------------------
class XieluFeedForward : public FeedForward {
public:
    XieluFeedForward(const Params& p, const std::string& prefix) : FeedForward(p, prefix), hidden_((int)p.integer("hidden_size")), ff_((int)p.integer("ff")) {
        if (hidden_ <= 0 || ff_ <= 0) throw std::invalid_argument("a dense feed-forward's sizes must be positive");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        return {TensorRequest::matrix(prefix + ".up", ff_, hidden_), TensorRequest::matrix(prefix + ".down", hidden_, ff_), TensorRequest::vector(prefix + ".act", 2)};
    }
    void load(const HostTensors& file, DType dtype) override {
        up_ = Linear(need_tensor(file, prefix + ".up"), nullptr, dtype);
        down_ = Linear(need_tensor(file, prefix + ".down"), nullptr, dtype);
        const std::vector<float> a = host_floats(need_tensor(file, prefix + ".act"));
        auto softplus = [](double v) { return v > 30.0 ? v : std::log1p(std::exp(v)); };
        above_ = (float)softplus(a[0]);
        below_ = (float)(0.5 + softplus(a[1]));
    }
    size_t weight_bytes() const override { return up_.weight_bytes() + down_.weight_bytes(); }
    size_t arena_bytes(long long T) const override { return (size_t)T * ((size_t)ff_ * 8 + (size_t)hidden_ * 4) + (1u << 16); }
    bool capturable() const override { return true; }

    Delta forward(const StepContext& ctx, PartInput in, const FollowingNorm*) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        const Rows h = in.pending ? in.pending->materialize() : in.rows;
        Rows act;
        if (plans::gemm_skinny_takes(dtype, T, hidden_) && Linear::aligned(h)) {
            // steps of few tokens: the decode product with the activation on its finished sums
            act = up_.skinny_xielu(ctx, h, above_, below_);
        } else if (plans::gemm_tcgen05_wide_takes(dtype, T, ff_, hidden_) && Linear::aligned(h)) {
            act = Rows{ctx.take_rows(T, ff_, dtype), dtype, T, ff_, ff_};
            // prompts: the product on the tcgen05 tensor cores (CTA pairs, 256 x 256 tiles) with the activation in its epilogue
            launch_check(eg_gemm_tcgen05_pair_xielu(ctx.stream, h.p, h.ld, up_.weight, hidden_, act.p, ff_, T, ff_, hidden_, 256, ctx.status, above_, below_),
                         "gemm_tcgen05_pair_xielu");
        } else {
            act = Rows{ctx.take_rows(T, ff_, dtype), dtype, T, ff_, ff_};
            const Rows z = up_(ctx, h, /*out_f32=*/true);
            launch_check(eg_xielu(ctx.stream, z.p, (int)z.dtype, z.ld, act.p, (int)dtype, act.ld, T, ff_, above_, below_), "xielu");
        }
        const Rows o = down_(ctx, act, /*out_f32=*/true);
        Delta d;
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    int hidden_, ff_;
    float above_ = 0.f, below_ = 0.f;
    Linear up_, down_;
};

inline void register_delta_parts() {
    PartRegistry& r = PartRegistry::instance();
    if (r.mixers.count("gated_delta")) return;
    r.mixers["sink_attention"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<SinkAttention>(p, prefix, std::move(pos));
    };
    r.mixers["gated_delta"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<GatedDeltaMixer>(p, prefix, std::move(pos));
    };
    r.feed_forwards["xielu"] = [](const Params& p, const std::string& prefix) { return std::make_shared<XieluFeedForward>(p, prefix); };
    r.shifts["token_shift"] = [](const Params& p, const std::string& prefix) { return std::make_shared<TokenShift>(p, prefix); };
}

}  // namespace easygpt::engine
