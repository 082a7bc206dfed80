// Further parts: a gain per channel on a branch's output (a layer scale), a causal convolution over time in front of a
// mixer, attention whose scores are mixed across the heads before the softmax and whose values are the keys as projected,
// a dense feed-forward with a squared ReLU, and a small gated map of a per-token vector that joins the stream through a norm
// of its own.  Each takes its sizes, constants and tensor-name suffixes from its parameters and knows nothing of the model
// around it.
#pragma once
#include "parts_delta.hpp"

namespace easygpt::engine {

// ---- a gain per channel, without normalisation: y = w * x.  As the output "norm" of a branch it rides along with the
// branch's output to the add (Delta::scale), so it costs no kernel.  Parameters: size, weight_name (suffix, default ".weight") ----
class LayerScale : public Norm {
public:
    LayerScale(const Params& p, const std::string& prefix) : Norm(p, prefix), size_((int)p.integer("size")), weight_name_(prefix + p.text("weight_name", ".weight")) {}
    std::vector<TensorRequest> tensor_requests() const override { return {TensorRequest::vector(weight_name_, size_).with_init("one")}; }
    void load(const HostTensors& file, DType) override { gain_ = upload_f32(file, weight_name_); }
    size_t weight_bytes() const override { return (size_t)size_ * 4; }
    bool capturable() const override { return true; }
    const float* plain_gain() const override { return gain_.as<float>(); }
    void forward(const StepContext&, float*, const void*, DType, void*, DType, int, const int*) const override {
        throw DeviceError("a layer scale stands on a branch's output, not in front of a part");
    }
    bool add_normed(const StepContext& ctx, float* residual, const void* y, DType y_dtype, int num_rows) const override {
        launch_check(eg_add_scaled(ctx.stream, residual, y, (int)y_dtype, gain_.as<float>(), num_rows, size_), "add_scaled");
        return true;
    }
    int size() const override { return size_; }

private:
    int size_;
    std::string weight_name_;
    DeviceBuffer gain_;
};

// ---- causal convolution over time, channel by channel, added to the rows themselves:
//   out[t] = h[t] + sum_{j < taps} w[:, j] * h[t - taps + 1 + j]     (rows in front of the request's start are zero)
// The request's slot keeps its last taps - 1 normed rows between steps, in float32, oldest first.
// Parameters: size, taps.  The tensor is the one named by the prefix itself, [size, taps] ---------------------------------------
class ConvShift : public Shift {
public:
    ConvShift(const Params& p, const std::string& prefix) : Shift(p, prefix), size_((int)p.integer("size")), taps_((int)p.integer("taps")) {
        if (size_ <= 0) throw std::invalid_argument("a convolution shift's size must be positive");
        if (taps_ < 1 || taps_ > 8) throw std::invalid_argument("a convolution shift takes 1 to 8 taps");
    }
    std::vector<TensorRequest> tensor_requests() const override { return {TensorRequest::matrix(prefix, size_, taps_)}; }
    void load(const HostTensors& file, DType) override { w_ = upload_f32(file, prefix); }
    size_t weight_bytes() const override { return (size_t)size_ * taps_ * 4; }
    bool capturable() const override { return true; }
    long long state_floats() const override { return (long long)(taps_ - 1) * size_; }
    // a step of single tokens moves the slots on in the same kernel (a token's block is its slot's only reader)
    void forward(const StepContext& ctx, const float* rows, float* state, long long slot_floats, void* out, DType out_dtype) const override {
        launch_check(eg_conv_shift(ctx.stream, rows, w_.as<float>(), state, slot_floats, ctx.token_seq, ctx.seq_starts, ctx.seq_slots, out, (int)out_dtype,
                                   ctx.num_tokens, size_, taps_, ctx.all_decode), "conv_shift");
        if (!ctx.all_decode)
            launch_check(eg_conv_shift_state(ctx.stream, rows, nullptr, 0.f, state, slot_floats, ctx.seq_starts, ctx.seq_slots, ctx.num_seqs, size_, taps_),
                         "conv_shift_state");
    }
    bool forward_rms(const StepContext& ctx, const float* residual, const float* gain, float eps, float* state, long long slot_floats, void* out,
                     void* plain_out, DType out_dtype) const override {
        launch_check(eg_rmsnorm_conv_shift(ctx.stream, residual, gain, eps, w_.as<float>(), state, slot_floats, ctx.token_seq, ctx.seq_starts, ctx.seq_slots,
                                           out, plain_out, (int)out_dtype, ctx.num_tokens, size_, taps_, ctx.all_decode), "rmsnorm_conv_shift");
        if (!ctx.all_decode)
            launch_check(eg_conv_shift_state(ctx.stream, residual, gain, eps, state, slot_floats, ctx.seq_starts, ctx.seq_slots, ctx.num_seqs, size_, taps_),
                         "conv_shift_state");
        return true;
    }

private:
    int size_, taps_;
    DeviceBuffer w_;
};

// ---- attention with mixed heads ------------------------------------------------------------------------------------------------
// H query heads and G key heads of `dim` values (query head h reads key head h / (H / G)):  q | k | gate = W h as ONE product
// (rows stacked), float32 out;  q and k are divided by their root mean square per head (norm_eps under the root) and
// multiplied by a weight [dim] shared by all heads (.q.norm, .k.norm), then turned by the layer's position encoding (a half
// rotation over its first dimensions, with the encoding's factor on cos and sin);  the VALUES are the keys as projected,
// before norm and turn;  score_h = sum_g M[h, g] scale (q_g . k_c(g)) with M the tensor .talk [H, H] (every head's scores are a
// mix of all heads' scores);  causal softmax over all earlier keys;  the heads' outputs side by side, times sigmoid(gate),
// go through W_o.  The mix is folded into the queries (see csrc/attention_mixed.cu): a head's query is a row of G * dim values
// that meets the keys of all key heads of a token.  The cache keeps two planes per token and key head: the normed and
// turned key, and the key as projected.
// Parameters: hidden_size, heads, kv_heads, dim, scale, norm_eps.  Tensors: .q .k .g .o .q.norm .k.norm .talk.
class MixedAttention : public Mixer {
public:
    MixedAttention(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
        : Mixer(p, prefix, std::move(position)), hidden_((int)p.integer("hidden_size")), heads_((int)p.integer("heads")), kv_heads_((int)p.integer("kv_heads")),
          dk_((int)p.integer("dim")), scale_((float)p.real("scale")), norm_eps_((float)p.real("norm_eps")) {
        if (hidden_ <= 0 || heads_ <= 0 || kv_heads_ <= 0 || dk_ <= 0) throw std::invalid_argument("mixed attention: sizes must be positive");
        if (heads_ % kv_heads_) throw std::invalid_argument("mixed attention: heads must be a multiple of kv_heads");
        if (dk_ > 256) throw std::invalid_argument("mixed attention: heads of up to 256 values are what the kernels take");
        if ((size_t)heads_ * dk_ * 4 > 48 * 1024 || (size_t)4 * kv_heads_ * dk_ * 4 > 48 * 1024)
            throw std::invalid_argument("mixed attention: heads * dim up to 12288 and kv_heads * dim up to 3072 are what the kernels take");
        if (norm_eps_ < 0.f) throw std::invalid_argument("mixed attention: norm_eps must not be negative");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        const long long q = (long long)heads_ * dk_, k = (long long)kv_heads_ * dk_;
        return {TensorRequest::matrix(prefix + ".q", q, hidden_), TensorRequest::matrix(prefix + ".k", k, hidden_), TensorRequest::matrix(prefix + ".g", q, hidden_),
                TensorRequest::matrix(prefix + ".o", hidden_, q), TensorRequest::vector(prefix + ".q.norm", dk_).with_init("one"),
                TensorRequest::vector(prefix + ".k.norm", dk_).with_init("one"), TensorRequest::matrix(prefix + ".talk", heads_, heads_).with_init("identity")};
    }
    void load(const HostTensors& file, DType dtype) override {
        std::vector<float> w;
        for (const char* n : {".q", ".k", ".g"}) {
            const std::vector<float> part = host_floats(need_tensor(file, prefix + n));
            w.insert(w.end(), part.begin(), part.end());
        }
        in_ = Linear(w.data(), (2 * heads_ + kv_heads_) * dk_, hidden_, nullptr, dtype);
        out_ = Linear(need_tensor(file, prefix + ".o"), nullptr, dtype);
        q_weight_ = upload_f32(file, prefix + ".q.norm");
        k_weight_ = upload_f32(file, prefix + ".k.norm");
        mix_ = upload_f32(file, prefix + ".talk");
        if (position) position->load(file, dtype);
    }
    size_t weight_bytes() const override { return in_.weight_bytes() + out_.weight_bytes() + (size_t)heads_ * heads_ * 4; }
    size_t arena_bytes(long long T) const override {
        // a step of single tokens keeps per-range sums: fewer than 2 SPLIT_CTAS (token, 16 heads, range) triples
        const size_t ranges = (size_t)2 * SPLIT_CTAS * 16 * (dk_ + 2) * 4;
        return (size_t)T * ((size_t)in_.out_features * 4 + (size_t)heads_ * kv_heads_ * dk_ * 4 + (size_t)heads_ * dk_ * 4 + (size_t)hidden_ * 4) + ranges + (1u << 16);
    }
    bool capturable() const override { return true; }
    CacheNeed cache_need() const override { return CacheNeed::paged(kv_heads_, dk_, -1); }

    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm*) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        if (cache.group < 0) throw DeviceError("mixed attention was handed no paged cache");
        const GroupTables& tables = ctx.groups.at(cache.group);
        const Rows h = in.pending ? in.pending->materialize() : in.rows;
        const Rows proj = in_(ctx, h, /*out_f32=*/true);                     // [T, q | k | gate] float32
        HalfRotation rot;
        const bool rotates = position && position->half_rotation(&rot);
        if (position && !rotates) throw DeviceError("mixed attention takes a half rotation or no position encoding");
        if (rotates && rot.rotary_dim > dk_) throw DeviceError("mixed attention: the rotation covers more than a head");
        const float* table = rotates ? step_rotation_table(ctx, rot) : nullptr;
        const int wide = kv_heads_ * dk_;
        // bfloat16 steps of sizes the tensor-core kernels take: folded queries in bfloat16, prompt portions by tiles, single
        // tokens split over their keys; everything else (and float32) through the generic kernel with float32 queries
        const bool mma = dtype == DType::BF16 && eg_mixed_attention_mma_takes(heads_, kv_heads_, dk_);
        const DType q_dtype = mma ? DType::BF16 : DType::F32;
        void* q = ctx.take_rows(T, (size_t)heads_ * wide, q_dtype);
        launch_check(eg_mixed_attention_prepare(ctx.stream, (int)dtype, (const float*)proj.p, proj.ld, q_weight_.as<float>(), k_weight_.as<float>(), norm_eps_, table,
                                                rotates ? rot.rotary_dim : 0, rot.magnitude, mix_.as<float>(), scale_, tables.slot_map,
                                                cache.writes ? cache.k : nullptr, cache.v, cache.head_stride, cache.page_size, cache.page_stride,
                                                (long long)cache.num_pages * cache.page_size, q, (int)q_dtype, T, heads_, kv_heads_, dk_, ctx.status),
                     "mixed_attention_prepare");
        Rows attn{ctx.take_rows(T, heads_ * dk_, dtype), dtype, T, heads_ * dk_, heads_ * dk_};
        const float* gate = (const float*)proj.p + (size_t)(heads_ + kv_heads_) * dk_;
        if (mma) {
            if (ctx.query_tiles)
                launch_check(eg_mixed_attention_tiles(ctx.stream, q, cache.k, cache.v, cache.head_stride, tables.block_table, tables.table_width, ctx.positions,
                                                      ctx.query_tiles, ctx.num_tiles, gate, proj.ld, attn.p, attn.ld, heads_, kv_heads_, dk_, cache.page_size,
                                                      cache.page_stride, cache.num_pages, ctx.status), "mixed_attention_tiles");
            const int singles = ctx.query_tiles ? ctx.num_small : T;
            if (singles > 0) {
                const int splits = split_plan(singles, heads_, ctx.max_context_len);
                float *acc = nullptr, *ml = nullptr;
                if (splits > 1) {
                    acc = ctx.take<float>((size_t)singles * heads_ * splits * dk_);
                    ml = ctx.take<float>((size_t)singles * heads_ * splits * 2);
                }
                launch_check(eg_mixed_attention_split(ctx.stream, q, cache.k, cache.v, cache.head_stride, tables.block_table, tables.table_width, ctx.token_seq,
                                                      ctx.positions, ctx.query_tiles ? ctx.small_tokens : nullptr, singles, gate, proj.ld, attn.p, attn.ld, acc, ml,
                                                      splits, heads_, kv_heads_, dk_, cache.page_size, cache.page_stride, cache.num_pages, ctx.status),
                             "mixed_attention_split");
            }
        } else {
            launch_check(eg_mixed_attention(ctx.stream, (int)dtype, q, (int)q_dtype, cache.k, cache.v, cache.head_stride, tables.block_table, tables.table_width,
                                            ctx.token_seq, ctx.positions, gate, proj.ld, attn.p, attn.ld, T, heads_, kv_heads_, dk_, cache.page_size,
                                            cache.page_stride, cache.num_pages, ctx.status), "mixed_attention");
        }
        const Rows o = out_(ctx, attn, /*out_f32=*/true);
        Delta d;
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    static constexpr int SPLIT_CTAS = 296;         // two CTAs a multiprocessor are what a step of single tokens is cut for
    static constexpr int MAX_SPLITS = 64;
    // ranges of at least 128 keys, as many as fill the GPU with the step's (token, 16 heads) pairs
    static int split_plan(int tokens, int heads, long long longest) {
        const long long pairs = (long long)tokens * ((heads + 15) / 16);
        const long long wanted = (SPLIT_CTAS + pairs - 1) / pairs, useful = (std::max<long long>(longest, 1) + 127) / 128;
        return (int)std::max<long long>(1, std::min<long long>({wanted, useful, (long long)MAX_SPLITS}));
    }

    int hidden_, heads_, kv_heads_, dk_;
    float scale_, norm_eps_;
    Linear in_, out_;
    DeviceBuffer q_weight_, k_weight_, mix_;
};

// ---- dense feed-forward with a squared ReLU: down(max(up h, 0)^2).  Parameters: hidden_size, ff.  Tensors: .up [ff, hidden],
// .down [hidden, ff] ---------------------------------------------------------------------------------------------------------------
class SquaredReluFeedForward : public FeedForward {
public:
    SquaredReluFeedForward(const Params& p, const std::string& prefix) : FeedForward(p, prefix), hidden_((int)p.integer("hidden_size")), ff_((int)p.integer("ff")) {
        if (hidden_ <= 0 || ff_ <= 0) throw std::invalid_argument("a dense feed-forward's sizes must be positive");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        return {TensorRequest::matrix(prefix + ".up", ff_, hidden_), TensorRequest::matrix(prefix + ".down", hidden_, ff_)};
    }
    void load(const HostTensors& file, DType dtype) override {
        up_ = Linear(need_tensor(file, prefix + ".up"), nullptr, dtype);
        down_ = Linear(need_tensor(file, prefix + ".down"), nullptr, dtype);
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
            // steps of few tokens: the decode product with the square on its finished sums
            act = up_.skinny_relu2(ctx, h);
        } else if (plans::gemm_tcgen05_wide_takes(dtype, T, ff_, hidden_) && Linear::aligned(h)) {
            // prompts: the product on the tcgen05 tensor cores (CTA pairs) with the activation in its epilogue
            act = Rows{ctx.take_rows(T, ff_, dtype), dtype, T, ff_, ff_};
            launch_check(eg_gemm_tcgen05_pair_relu2(ctx.stream, h.p, h.ld, up_.weight, hidden_, act.p, ff_, T, ff_, hidden_, 256, ctx.status), "gemm_tcgen05_pair_relu2");
        } else {
            act = Rows{ctx.take_rows(T, ff_, dtype), dtype, T, ff_, ff_};
            const Rows z = up_(ctx, h, /*out_f32=*/true);
            launch_check(eg_squared_relu(ctx.stream, z.p, (int)z.dtype, z.ld, act.p, (int)dtype, act.ld, T, ff_), "squared_relu");
        }
        const Rows o = down_(ctx, act, /*out_f32=*/true);
        Delta d;
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    int hidden_, ff_;
    Linear up_, down_;
};

// ---- a per-layer token input ------------------------------------------------------------------------------------------------
// Every token brings a vector e of `side` values of its own, the columns [column, column + side) of a table [vocab, columns]
// that all layers share.  It is gated by the stream and mapped to the model's width:
//   y = P (gelu_tanh(G x) * e),     G = .gate [side, hidden], P = .proj [hidden, side]
// and joins the stream through an RMS norm on its output (the sub-layer's output norm).  It reads the stream itself (no norm
// in front).  The two maps are products over all tokens of the step (Linear: the decode product for a few tokens, the library
// product above); forward_joined first takes in the outputs that are still to be added (one kernel: the adds and the rows the
// product reads), and ends with the norm-and-add.
// Parameters: hidden_size, vocab_size, side, column, columns, table (the table's tensor name).
class TokenSide : public FeedForward {
public:
    TokenSide(const Params& p, const std::string& prefix)
        : FeedForward(p, prefix), hidden_((int)p.integer("hidden_size")), vocab_((int)p.integer("vocab_size")), side_((int)p.integer("side")),
          column_((int)p.integer("column", 0)), columns_((int)p.integer("columns", p.integer("side"))), table_name_(p.text("table")) {
        if (hidden_ <= 0 || vocab_ <= 0 || side_ <= 0) throw std::invalid_argument("a token input's sizes must be positive");
        if (column_ < 0 || column_ + side_ > columns_) throw std::invalid_argument("a token input's columns lie outside its table");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        return {TensorRequest::matrix(table_name_, vocab_, columns_), TensorRequest::matrix(prefix + ".gate", side_, hidden_),
                TensorRequest::matrix(prefix + ".proj", hidden_, side_)};
    }
    void load(const HostTensors& file, DType dtype) override {
        // this layer's columns of the shared table, as a table [vocab, side] of its own
        const std::vector<float> all = host_floats(need_tensor(file, table_name_));
        std::vector<float> mine((size_t)vocab_ * side_);
        for (int v = 0; v < vocab_; ++v) std::memcpy(&mine[(size_t)v * side_], &all[(size_t)v * columns_ + column_], (size_t)side_ * 4);
        table_ = upload(mine.data(), mine.size(), dtype);
        gate_ = Linear(need_tensor(file, prefix + ".gate"), nullptr, dtype);
        proj_ = Linear(need_tensor(file, prefix + ".proj"), nullptr, dtype);
    }
    size_t weight_bytes() const override { return gate_.weight_bytes() + proj_.weight_bytes(); }
    size_t arena_bytes(long long T) const override { return joined_arena_bytes(T); }
    size_t joined_arena_bytes(long long T) const override { return (size_t)T * ((size_t)hidden_ * 8 + (size_t)side_ * 8) + (1u << 12); }
    bool capturable() const override { return true; }

    Delta forward(const StepContext& ctx, PartInput in, const FollowingNorm*) override {
        const Rows x = in.pending ? in.pending->materialize() : in.rows;
        const Rows y = map(ctx, x);
        Delta d;
        d.p = y.p;
        d.dtype = y.dtype;
        return d;
    }
    bool forward_joined(const StepContext& ctx, float* residual, const Delta& a, const Delta& b, const float* gain, float eps) override {
        const int T = ctx.num_tokens;
        Rows x{ctx.take_rows(T, hidden_, ctx.dtype), ctx.dtype, T, hidden_, hidden_};
        launch_check(eg_add_scaled_rows(ctx.stream, residual, a.p, (int)a.dtype, a.scale, b.p, (int)b.dtype, b.scale, x.p, (int)x.dtype, T, hidden_), "add_scaled_rows");
        const Rows y = map(ctx, x);
        launch_check(eg_rmsnorm_add(ctx.stream, residual, y.p, (int)y.dtype, y.ld, gain, eps, T, hidden_), "rmsnorm_add");
        return true;
    }

private:
    // y float32 [T, hidden] = P (gelu_tanh(G x) * e)
    Rows map(const StepContext& ctx, const Rows& x) const {
        const int T = ctx.num_tokens;
        const Rows z = gate_(ctx, x, /*out_f32=*/true);
        Rows g{ctx.take_rows(T, side_, ctx.dtype), ctx.dtype, T, side_, side_};
        launch_check(eg_token_side_gate(ctx.stream, (int)ctx.dtype, (const float*)z.p, z.ld, ctx.token_ids, table_.get(), vocab_, g.p, T, side_, ctx.status),
                     "token_side_gate");
        return proj_(ctx, g, /*out_f32=*/true);
    }

    int hidden_, vocab_, side_, column_, columns_;
    std::string table_name_;
    DeviceBuffer table_;
    Linear gate_, proj_;
};

inline void register_mixed_parts() {
    PartRegistry& r = PartRegistry::instance();
    if (r.mixers.count("mixed_attention")) return;
    r.norms["layer_scale"] = [](const Params& p, const std::string& prefix) { return std::make_shared<LayerScale>(p, prefix); };
    r.shifts["conv_shift"] = [](const Params& p, const std::string& prefix) { return std::make_shared<ConvShift>(p, prefix); };
    r.mixers["mixed_attention"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<MixedAttention>(p, prefix, std::move(pos));
    };
    r.feed_forwards["squared_relu"] = [](const Params& p, const std::string& prefix) { return std::make_shared<SquaredReluFeedForward>(p, prefix); };
    r.feed_forwards["token_side"] = [](const Params& p, const std::string& prefix) { return std::make_shared<TokenSide>(p, prefix); };
}

}  // namespace easygpt::engine
