// Further parts: a selective state-space mixer (state per request instead of cached keys), attention whose keys and
// values are expanded from one cached latent row per token, and a routed feed-forward (a router over gated experts and
// pass-through experts, beside an optional gated shared expert).  Each takes its sizes, constants and tensor-name
// suffixes from its parameters and knows nothing of the model around it.
#pragma once
#include "parts.hpp"

namespace easygpt::engine {

// ---- selective state-space mixer ---------------------------------------------------------------------------------------
// With h the input, I channels, N states per channel, R the rank of the step-size projection, K taps:
//   (x | z) = W_in h;  u = silu(conv_K(x) + b_conv) per channel, causal, continuing from the request's last K-1 inputs
//   (low_dt | B | C) = W_x u;  dt = softplus(W_dt low_dt + b_dt);  A = -exp(A_log)
//   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n;  y_c = sum_n S[c, n] C_n + D_c u_c;  out = W_o (y * silu(z))
// The request's state slot holds the K-1 last inputs of the convolution and S, in float32; step sizes, decays,
// exponentials and S are float32 in both precisions.
// Parameters: hidden_size, inner, state, dt_rank, conv.  Tensors under the prefix: .in [2I, hidden], .conv [I, K],
// .conv.b [I], .x [R + 2N, I], .dt [I, R], .dt.b [I], .A_log [I, N], .D [I], .o [hidden, I].
class SelectiveScanMixer : public Mixer {
public:
    SelectiveScanMixer(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
        : Mixer(p, prefix, std::move(position)), hidden_((int)p.integer("hidden_size")), inner_((int)p.integer("inner")), states_((int)p.integer("state")),
          rank_((int)p.integer("dt_rank")), taps_((int)p.integer("conv")) {
        if (hidden_ <= 0 || inner_ <= 0 || rank_ <= 0 || taps_ < 1) throw std::invalid_argument("a selective-scan mixer's sizes must be positive");
        if (states_ <= 0 || states_ > 512) throw std::invalid_argument("a selective-scan mixer takes 1 to 512 states per channel");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        return {TensorRequest::matrix(prefix + ".in", 2LL * inner_, hidden_), TensorRequest::matrix(prefix + ".conv", inner_, taps_),
                TensorRequest::vector(prefix + ".conv.b", inner_), TensorRequest::matrix(prefix + ".x", rank_ + 2LL * states_, inner_),
                TensorRequest::matrix(prefix + ".dt", inner_, rank_), TensorRequest::vector(prefix + ".dt.b", inner_).with_init("step_bias"),
                TensorRequest::matrix(prefix + ".A_log", inner_, states_).with_init("log_decay"), TensorRequest::vector(prefix + ".D", inner_).with_init("one"),
                TensorRequest::matrix(prefix + ".o", hidden_, inner_)};
    }
    void load(const HostTensors& file, DType dtype) override {
        in_ = Linear(need_tensor(file, prefix + ".in"), nullptr, dtype);
        x_ = Linear(need_tensor(file, prefix + ".x"), nullptr, dtype);
        out_ = Linear(need_tensor(file, prefix + ".o"), nullptr, dtype);
        // bfloat16 with a rank the products take: the step sizes' projection is a product of its own on the tensor cores
        // (then the rows of W_x for it and those for B and C are two products, one with bfloat16 output to feed it)
        split_ = dtype == DType::BF16 && rank_ % 8 == 0;
        if (split_) {
            const std::vector<float> wx = host_floats(need_tensor(file, prefix + ".x"));
            x_dt_ = Linear(wx.data(), rank_, inner_, nullptr, dtype);
            x_bc_ = Linear(wx.data() + (size_t)rank_ * inner_, 2 * states_, inner_, nullptr, dtype);
            dt_ = Linear(need_tensor(file, prefix + ".dt"), nullptr, dtype);
        }
        auto f32 = [&](const std::string& name) {
            const std::vector<float> v = host_floats(need_tensor(file, prefix + name));
            return upload(v.data(), v.size(), DType::F32);
        };
        conv_w_ = f32(".conv");
        conv_b_ = f32(".conv.b");
        dt_w_ = f32(".dt");
        dt_b_ = f32(".dt.b");
        skip_ = f32(".D");
        std::vector<float> a = host_floats(need_tensor(file, prefix + ".A_log"));
        for (float& v : a) v = -std::exp(v);                 // float32, as the recurrence uses it
        decay_ = upload(a.data(), a.size(), DType::F32);
    }
    size_t weight_bytes() const override {
        return in_.weight_bytes() + x_.weight_bytes() + out_.weight_bytes() + (size_t)inner_ * (taps_ + rank_ + states_ + 3) * 4;
    }
    size_t arena_bytes(long long T) const override { return (size_t)T * ((size_t)4 * inner_ * 4 + (size_t)(rank_ + 2 * states_) * 8 + (size_t)hidden_ * 4) + (1u << 16); }
    bool capturable() const override { return true; }
    CacheNeed cache_need() const override { return CacheNeed::state({slot_floats()}); }
    long long slot_floats() const { return (long long)(taps_ - 1) * inner_ + (long long)inner_ * states_; }

    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm*) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        if (!cache.state || cache.state_bytes_per_slot != (size_t)slot_floats() * 4) throw DeviceError("a selective-scan mixer was handed no state of its shape");
        if (!cache.writes) throw DeviceError("a selective-scan mixer cannot read another entry's state without advancing it");
        const Rows h = in.pending ? in.pending->materialize() : in.rows;
        const Rows xz = in_(ctx, h);                                                 // [T, 2I]: x | z
        float* state = (float*)cache.state;
        const long long slot = slot_floats(), es = (long long)dtype_size(dtype);
        Rows u{ctx.take_rows(T, inner_, dtype), dtype, T, inner_, inner_};
        launch_check(eg_conv_silu(ctx.stream, (int)dtype, xz.p, xz.ld, conv_w_.as<float>(), conv_b_.as<float>(), state, slot, ctx.token_seq, ctx.seq_starts,
                                  ctx.seq_slots, u.p, u.ld, T, inner_, taps_), "conv_silu");
        launch_check(eg_conv_state(ctx.stream, (int)dtype, xz.p, xz.ld, state, slot, ctx.seq_starts, ctx.seq_slots, ctx.num_seqs, inner_, taps_), "conv_state");
        Rows low;
        const float *dt = nullptr, *dt_bias = nullptr;
        int b_col = rank_;
        if (split_) {
            const Rows low_dt = x_dt_(ctx, u);                                       // [T, R] bfloat16
            low = x_bc_(ctx, u, /*out_f32=*/true);                                   // [T, 2N] float32: B | C
            dt = (const float*)dt_(ctx, low_dt, /*out_f32=*/true).p;                 // [T, I] float32, before bias and softplus
            dt_bias = dt_b_.as<float>();
            b_col = 0;
        } else {
            low = x_(ctx, u, /*out_f32=*/true);                                      // [T, R + 2N] float32: low_dt | B | C
            float* sizes = ctx.take<float>((size_t)T * inner_);
            launch_check(eg_step_sizes(ctx.stream, (const float*)low.p, low.ld, dt_w_.as<float>(), dt_b_.as<float>(), sizes, T, inner_, rank_), "step_sizes");
            dt = sizes;
        }
        Rows y{ctx.take_rows(T, inner_, dtype), dtype, T, inner_, inner_};
        launch_check(eg_selective_scan(ctx.stream, (int)dtype, u.p, u.ld, dt, dt_bias, (const float*)low.p, low.ld, b_col, b_col + states_, decay_.as<float>(),
                                       skip_.as<float>(), (const char*)xz.p + (size_t)inner_ * es, xz.ld, state, slot, (long long)(taps_ - 1) * inner_,
                                       ctx.seq_starts, ctx.seq_slots, y.p, y.ld, ctx.num_seqs, inner_, states_,
                                       plans::scan_states_per_lane(inner_, states_)), "selective_scan");
        const Rows o = out_(ctx, y, /*out_f32=*/true);
        Delta d;
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    int hidden_, inner_, states_, rank_, taps_;
    Linear in_, x_, out_, x_dt_, x_bc_, dt_;
    bool split_ = false;
    DeviceBuffer conv_w_, conv_b_, dt_w_, dt_b_, decay_, skip_;
};

// ---- attention through a latent ------------------------------------------------------------------------------------------
// With h the input, H heads, per head `dim` plain and `rot_dim` rotated query/key values, value size `vdim`:
//   c_q = unit_rms(W_dq h) * g_q;  q = W_uq c_q, head by head (dim plain | rot_dim rotated)
//   (c' | k_r') = W_dkv h;  c = unit_rms(c') * g_kv [kv_rank];  k_r = rotate(k_r') [rot_dim], one for all heads
//   key_h = (W_uk,h c | k_r), value_h = W_uv,h c;  score = (q_plain . key_plain + rotate(q_rot) . k_r) * scale
//   causal softmax whose denominator also holds exp(sink_h) if the model has sinks;  out = W_o (heads' values side by side)
// Only (c | k_r) is cached: one row per token for all heads (CacheNeed::paged_rows).  The rotation turns neighbouring
// pairs (2i, 2i+1) of the first rot_dims values by position * base^(-2i / rot_dims).
// Parameters: hidden_size, heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot_base, rot_dims, eps, sink.
// Tensors: .dq [q_rank, hidden], .dq.norm, .uq [H (dim + rot_dim), q_rank], .dkv [kv_rank + rot_dim, hidden], .dkv.norm,
// .uk [H dim, kv_rank], .uv [H vdim, kv_rank], .sink [H], .o [hidden, H vdim].
class LatentAttention : public Mixer {
public:
    LatentAttention(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
        : Mixer(p, prefix, std::move(position)), hidden_((int)p.integer("hidden_size")), heads_((int)p.integer("heads")), dim_((int)p.integer("dim")),
          rot_((int)p.integer("rot_dim")), vdim_((int)p.integer("vdim")), rank_((int)p.integer("kv_rank")), q_rank_((int)p.integer("q_rank")),
          rot_dims_((int)p.integer("rot_dims", p.integer("rot_dim"))), scale_((float)p.real("scale")), base_(p.real("rot_base")), eps_((float)p.real("eps")),
          sink_(p.flag("sink", false)) {
        if (heads_ <= 0 || dim_ < 0 || rot_ < 0 || dim_ + rot_ <= 0 || vdim_ <= 0 || rank_ <= 0 || q_rank_ <= 0)
            throw std::invalid_argument("latent attention: sizes must be positive");
        if (rot_dims_ % 2 || rot_dims_ < 0 || rot_dims_ > rot_) throw std::invalid_argument("latent attention: rot_dims must be even and within rot_dim");
        if (rot_dims_ > 0 && base_ <= 0) throw std::invalid_argument("latent attention: the rotation's base must be > 0");
        if (rank_ + rot_ > 1024) throw std::invalid_argument("latent attention: kv_rank + rot_dim is beyond what the kernel takes (1024)");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        std::vector<TensorRequest> r = {TensorRequest::matrix(prefix + ".dq", q_rank_, hidden_), TensorRequest::vector(prefix + ".dq.norm", q_rank_).with_init("one"),
                                        TensorRequest::matrix(prefix + ".uq", (long long)heads_ * (dim_ + rot_), q_rank_),
                                        TensorRequest::matrix(prefix + ".dkv", rank_ + rot_, hidden_), TensorRequest::vector(prefix + ".dkv.norm", rank_).with_init("one"),
                                        TensorRequest::matrix(prefix + ".uk", (long long)heads_ * dim_, rank_),
                                        TensorRequest::matrix(prefix + ".uv", (long long)heads_ * vdim_, rank_), TensorRequest::matrix(prefix + ".o", hidden_, (long long)heads_ * vdim_)};
        if (sink_) r.push_back(TensorRequest::vector(prefix + ".sink", heads_).with_init("zero"));
        return r;
    }
    void load(const HostTensors& file, DType dtype) override {
        // one product for both down-projections: rows (query latent | latent | rotated key part)
        std::vector<float> w = host_floats(need_tensor(file, prefix + ".dq"));
        const std::vector<float> dkv = host_floats(need_tensor(file, prefix + ".dkv"));
        w.insert(w.end(), dkv.begin(), dkv.end());
        down_ = Linear(w.data(), q_rank_ + rank_ + rot_, hidden_, nullptr, dtype);
        up_q_ = Linear(need_tensor(file, prefix + ".uq"), nullptr, dtype);
        out_ = Linear(need_tensor(file, prefix + ".o"), nullptr, dtype);
        up_k_ = upload(need_tensor(file, prefix + ".uk"), dtype);
        up_v_ = upload(need_tensor(file, prefix + ".uv"), dtype);
        auto f32 = [&](const std::string& name) {
            const std::vector<float> v = host_floats(need_tensor(file, prefix + name));
            return upload(v.data(), v.size(), DType::F32);
        };
        gain_q_ = f32(".dq.norm");
        gain_c_ = f32(".dkv.norm");
        if (sink_) sinks_ = f32(".sink");
        std::vector<float> inv(std::max(1, rot_dims_ / 2));
        for (int i = 0; i < rot_dims_ / 2; ++i) inv[i] = (float)std::pow(base_, -2.0 * i / rot_dims_);
        inv_freq_ = upload(inv.data(), inv.size(), DType::F32);
    }
    size_t weight_bytes() const override {
        return down_.weight_bytes() + up_q_.weight_bytes() + out_.weight_bytes() + (size_t)heads_ * (dim_ + vdim_) * rank_ * dtype_size(down_.dtype);
    }
    size_t arena_bytes(long long T) const override {
        const size_t per_token = (size_t)(q_rank_ + rank_ + rot_) * 4 + (size_t)q_rank_ * 4 + (size_t)heads_ * (dim_ + rot_) * 4 + (size_t)heads_ * (rank_ + rot_) * 4 +
                                 (size_t)heads_ * rank_ * 4 + (size_t)heads_ * vdim_ * 4 + (size_t)hidden_ * 4;
        // the parts of an attention whose keys are cut: at most two CTAs an SM's worth of them beyond one per token
        const size_t parts = (size_t)(4 * plans::sm_count() + 64) * 16 * (size_t)(rank_ + 2) * 4;
        return (size_t)T * per_token + parts + (1u << 16);
    }
    bool capturable() const override { return true; }
    CacheNeed cache_need() const override { return CacheNeed::paged_rows(rank_ + rot_, -1); }

    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm*) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        if (cache.group < 0) throw DeviceError("latent attention was handed no paged cache");
        const GroupTables& tables = ctx.groups.at(cache.group);
        const Rows h = in.pending ? in.pending->materialize() : in.rows;
        const Rows down = down_(ctx, h, /*out_f32=*/true);
        Rows cq{ctx.take_rows(T, q_rank_, dtype), dtype, T, q_rank_, q_rank_};
        launch_check(eg_latent_prepare(ctx.stream, (const float*)down.p, down.ld, q_rank_, rank_, rot_, rot_dims_, gain_q_.as<float>(), gain_c_.as<float>(), eps_,
                                       inv_freq_.as<float>(), ctx.positions, tables.slot_map, cache.writes ? cache.k : nullptr, (int)dtype, cache.page_size,
                                       cache.page_stride, (long long)cache.num_pages * cache.page_size, cq.p, (int)dtype, T, ctx.status), "latent_prepare");
        const int D = rank_ + rot_;
        if (dtype == DType::BF16 && eg_attention_latent_mma_takes(rank_, rot_) && (dim_ + rot_) % 8 == 0 && dim_ % 8 == 0 && vdim_ % 8 == 0 && dim_ > 0) {
            // bfloat16 on the tensor cores: the per-head maps are strided batches of the library's product (a head is a
            // stride in the row, not a copy), the attention takes the heads of a token as the rows of its products
            const Rows q = up_q_(ctx, cq);
            void* qa = ctx.take_rows((size_t)T * heads_, D, dtype);
            ctx.blas->gemm_bf16_batched(ctx.stream, false, rank_, T, dim_, scale_, up_k_.get(), rank_, (long long)dim_ * rank_, q.p, q.ld, dim_ + rot_, qa,
                                        (long long)heads_ * D, D, false, heads_);
            launch_check(eg_latent_rotate_query(ctx.stream, q.p, q.ld, ctx.positions, inv_freq_.as<float>(), rot_dims_, scale_, qa, T, heads_, dim_, rot_, rank_),
                         "latent_rotate_query");
            const int splits = plans::latent_attention_splits(T, heads_, ctx.max_context_len);
            float *part_o = nullptr, *part_ml = nullptr;
            if (splits > 1) {
                part_o = ctx.take<float>((size_t)T * heads_ * splits * rank_);
                part_ml = ctx.take<float>((size_t)T * heads_ * splits * 2);
            }
            void* o = ctx.take_rows((size_t)T * heads_, rank_, dtype);
            launch_check(eg_attention_latent_mma(ctx.stream, qa, cache.k, tables.block_table, tables.table_width, ctx.token_seq, ctx.positions,
                                                 sink_ ? sinks_.as<float>() : nullptr, o, part_o, part_ml, T, heads_, rank_, rot_, cache.page_size, cache.page_stride,
                                                 cache.num_pages, splits, ctx.status), "attention_latent_mma");
            Rows values{ctx.take_rows(T, heads_ * vdim_, dtype), dtype, T, heads_ * vdim_, heads_ * vdim_};
            ctx.blas->gemm_bf16_batched(ctx.stream, true, vdim_, T, rank_, 1.0f, up_v_.get(), rank_, (long long)vdim_ * rank_, o, (long long)heads_ * rank_, rank_,
                                        values.p, values.ld, vdim_, false, heads_);
            const Rows res = out_(ctx, values, /*out_f32=*/true);
            Delta d;
            d.p = res.p;
            d.dtype = res.dtype;
            return d;
        }
        const Rows q = up_q_(ctx, cq, /*out_f32=*/true);
        float* qa = ctx.take<float>((size_t)T * heads_ * (rank_ + rot_));
        launch_check(eg_latent_absorb(ctx.stream, (int)dtype, (const float*)q.p, q.ld, up_k_.get(), ctx.positions, inv_freq_.as<float>(), rot_dims_, scale_, qa, T,
                                      heads_, dim_, rot_, rank_), "latent_absorb");
        float* o = ctx.take<float>((size_t)T * heads_ * rank_);
        launch_check(eg_attention_latent(ctx.stream, (int)dtype, qa, cache.k, tables.block_table, tables.table_width, ctx.token_seq, ctx.positions,
                                         sink_ ? sinks_.as<float>() : nullptr, o, T, heads_, rank_, rot_, cache.page_size, cache.page_stride, cache.num_pages,
                                         ctx.status), "attention_latent");
        Rows values{ctx.take_rows(T, heads_ * vdim_, dtype), dtype, T, heads_ * vdim_, heads_ * vdim_};
        launch_check(eg_latent_expand(ctx.stream, (int)dtype, o, up_v_.get(), values.p, (int)dtype, values.ld, T, heads_, vdim_, rank_), "latent_expand");
        const Rows res = out_(ctx, values, /*out_f32=*/true);
        Delta d;
        d.p = res.p;
        d.dtype = res.dtype;
        return d;
    }

private:
    int hidden_, heads_, dim_, rot_, vdim_, rank_, q_rank_, rot_dims_;
    float scale_;
    double base_;
    float eps_;
    bool sink_;
    Linear down_, up_q_, out_;
    DeviceBuffer up_k_, up_v_, gain_q_, gain_c_, sinks_, inv_freq_;
};

// ---- routed feed-forward -------------------------------------------------------------------------------------------------
// The router has experts + identity outputs: logits = R h and s = softmax(logits) in float32.  The `top` outputs with the
// largest s + correction are chosen; their weights are s (no correction, no renormalisation).  A chosen output below
// `experts` is a gated expert, down(silu(gate h) * (up h)); the last `identity` outputs stand for the input itself.
// out = sum of weight * (expert(h) or h).  A shared expert of the same form (shared_ff > 0) runs for every token and is
// added times sigmoid(w_g . h).
// Parameters: hidden_size, experts, identity, top, ff, shared_ff.  Tensors: .router [experts + identity, hidden],
// .correction [experts + identity], .e<i>.gate / .up [ff, hidden], .e<i>.down [hidden, ff], .shared.gate / .up / .down,
// .shared.sg [1, hidden].
// Further parameters, each with the default that leaves the above as it is: scoring "sigmoid" (s = sigmoid(logits) instead of
// the softmax); correction 0 (no .correction tensor); activation "clamped" with limit (an expert is
// down(g sigmoid(1.702 g) (u + 1)), g = min(gate x, limit), u = clamp(up x, -limit, limit)); weight_input 1 (the weight
// multiplies the expert's input, out = sum of expert(weight * h), not its output); shared_gated 0 (the shared expert is added
// as it is, no .shared.sg), shared_activation / shared_limit (the shared expert's own form).
class RoutedExperts : public FeedForward {
public:
    RoutedExperts(const Params& p, const std::string& prefix)
        : FeedForward(p, prefix), hidden_((int)p.integer("hidden_size")), experts_((int)p.integer("experts")), identity_((int)p.integer("identity", 0)),
          top_((int)p.integer("top")), ff_((int)p.integer("ff", 0)), shared_ff_((int)p.integer("shared_ff", 0)),
          sigmoid_(p.text("scoring", "softmax") == "sigmoid"), corrected_(p.integer("correction", 1) != 0), clamped_(p.text("activation", "swiglu") == "clamped"),
          weight_input_(p.integer("weight_input", 0) != 0), shared_gated_(p.integer("shared_gated", 1) != 0), limit_((float)p.real("limit", 0.0)) {
        if (p.text("scoring", "softmax") != "softmax" && !sigmoid_) throw std::invalid_argument("a routed feed-forward's scoring is 'softmax' or 'sigmoid'");
        if (p.text("activation", "swiglu") != "swiglu" && !clamped_) throw std::invalid_argument("a routed feed-forward's activation is 'swiglu' or 'clamped'");
        if (clamped_ && !(limit_ > 0.f)) throw std::invalid_argument("a clamped gate needs a positive limit");
        if (weight_input_ && identity_ > 0) throw std::invalid_argument("identity outputs take their weight on the output");
        if (experts_ < 0 || identity_ < 0 || experts_ + identity_ <= 0) throw std::invalid_argument("a routed feed-forward needs at least one router output");
        if (top_ < 1 || top_ > experts_ + identity_) throw std::invalid_argument("a routed feed-forward chooses between 1 and all of its router outputs");
        if (experts_ > 0 && ff_ <= 0) throw std::invalid_argument("a routed feed-forward's experts need a positive ff");
        if (experts_ + identity_ > 2048) throw std::invalid_argument("a routed feed-forward takes at most 2048 router outputs");
        if (shared_ff_ > 0) {
            Params sp{{"hidden_size", hidden_}, {"intermediate_size", shared_ff_}, {"gate_name", ".gate"}, {"up_name", ".up"}, {"down_name", ".down"}};
            if (p.has("shared_activation")) sp.set("activation", p.text("shared_activation"));
            if (p.has("shared_limit")) sp.set("limit", p.real("shared_limit"));
            shared_ = std::make_shared<SwiGLU>(sp, prefix + ".shared");
        }
    }
    std::vector<TensorRequest> tensor_requests() const override {
        std::vector<TensorRequest> r = {TensorRequest::matrix(prefix + ".router", experts_ + identity_, hidden_)};
        if (corrected_) r.push_back(TensorRequest::vector(prefix + ".correction", experts_ + identity_).with_init("zero"));
        for (int e = 0; e < experts_; ++e) {
            const std::string ep = prefix + ".e" + std::to_string(e);
            r.push_back(TensorRequest::matrix(ep + ".gate", ff_, hidden_));
            r.push_back(TensorRequest::matrix(ep + ".up", ff_, hidden_));
            r.push_back(TensorRequest::matrix(ep + ".down", hidden_, ff_));
        }
        if (shared_) {
            for (auto& t : shared_->tensor_requests()) r.push_back(t);
            if (shared_gated_) r.push_back(TensorRequest{prefix + ".shared.sg", {{1, hidden_}, {hidden_}}, false, ""});
        }
        return r;
    }
    void load(const HostTensors& file, DType dtype) override {
        auto f32 = [&](const std::string& name) {
            const std::vector<float> v = host_floats(need_tensor(file, prefix + name));
            return upload(v.data(), v.size(), DType::F32);
        };
        router_ = f32(".router");
        if (corrected_) correction_ = f32(".correction");
        // all experts in one block each: gate and up rows interleaved per hidden unit (gate_f, up_f), and the down maps
        std::vector<float> gu((size_t)experts_ * 2 * ff_ * hidden_), dn((size_t)experts_ * hidden_ * ff_);
        for (int e = 0; e < experts_; ++e) {
            const std::string ep = prefix + ".e" + std::to_string(e);
            const std::vector<float> g = host_floats(need_tensor(file, ep + ".gate")), u = host_floats(need_tensor(file, ep + ".up")),
                                     d = host_floats(need_tensor(file, ep + ".down"));
            float* base = gu.data() + (size_t)e * 2 * ff_ * hidden_;
            for (int f = 0; f < ff_; ++f) {
                std::memcpy(base + (size_t)(2 * f) * hidden_, &g[(size_t)f * hidden_], (size_t)hidden_ * 4);
                std::memcpy(base + (size_t)(2 * f + 1) * hidden_, &u[(size_t)f * hidden_], (size_t)hidden_ * 4);
            }
            std::memcpy(dn.data() + (size_t)e * hidden_ * ff_, d.data(), d.size() * 4);
        }
        gate_up_ = upload(gu.data(), gu.size(), dtype);
        down_ = upload(dn.data(), dn.size(), dtype);
        dtype_ = dtype;
        if (shared_) {
            shared_->load(file, dtype);
            if (shared_gated_) shared_gate_ = f32(".shared.sg");
        }
    }
    // a step reads the router, and per token `top` experts at most (all of them once there are many tokens)
    size_t weight_bytes() const override {
        return (size_t)(experts_ + identity_) * hidden_ * 4 + (size_t)std::min(top_, experts_) * 3 * ff_ * hidden_ * dtype_size(dtype_) +
               (shared_ ? shared_->weight_bytes() + (size_t)hidden_ * 4 : 0);
    }
    size_t arena_bytes(long long T) const override {
        const size_t sorted = (size_t)grouped_rows(T) * ((size_t)hidden_ + ff_) * 2 + (size_t)grouped_rows(T) / 32 + (size_t)experts_ * 16;
        return (size_t)T * ((size_t)top_ * (12 + (size_t)ff_ * 4) + 4 + (size_t)(experts_ + identity_) * 4 + (size_t)hidden_ * 8 + (size_t)shared_ff_ * 3 * 4) + sorted + (1u << 16);
    }
    // rows of the sorted copy of a step of T tokens: every expert's run starts at a multiple of 128
    int grouped_rows(long long T) const { return (int)((T * top_ + 127) / 128 * 128 + 128LL * experts_); }
    bool capturable() const override { return true; }

    Delta forward(const StepContext& ctx, PartInput in, const FollowingNorm*) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        const Rows h = in.pending ? in.pending->materialize() : in.rows;
        int* ids = ctx.take<int>((size_t)T * top_);
        float* weights = ctx.take<float>((size_t)T * top_);
        const bool gated = shared_ && shared_gated_;
        float* gate = gated ? ctx.take<float>((size_t)T) : nullptr;
        float* scores = ctx.take<float>((size_t)T * (experts_ + identity_));
        launch_check(eg_moe_route(ctx.stream, (int)dtype, h.p, h.ld, router_.as<float>(), corrected_ ? correction_.as<float>() : nullptr,
                                  gated ? shared_gate_.as<float>() : nullptr, scores, ids, weights, gate, T, hidden_, experts_ + identity_, top_, sigmoid_ ? 1 : 0),
                     "moe_route");
        // where the weight multiplies an expert's input, the sums over the chosen experts count every term once
        const float* in_w = weight_input_ ? weights : nullptr;
        const float* out_w = weight_input_ ? nullptr : weights;
        Delta shared;
        if (shared_) {
            PartInput rows;
            rows.rows = h;
            shared = shared_->forward(ctx, rows, nullptr);
        }
        float* out = ctx.take<float>((size_t)T * hidden_);
        if (plans::moe_grouped_takes(dtype, T, hidden_, ff_, experts_)) {
            // many tokens: rows sorted by expert, one grouped product on the tensor cores per projection
            const int max_rows = grouped_rows(T);
            int* scratch = ctx.take<int>((size_t)3 * experts_ + 1 + max_rows / 128 + (size_t)T * top_);
            int *counts = scratch, *starts = counts + experts_, *cursors = starts + experts_ + 1, *tile_group = cursors + experts_,
                *row_of = tile_group + max_rows / 128;
            void* rows = ctx.take_rows(max_rows, hidden_, dtype);
            launch_check(eg_moe_dispatch(ctx.stream, h.p, h.ld, ids, in_w, counts, starts, cursors, tile_group, row_of, rows, T, hidden_, top_, experts_, max_rows),
                         "moe_dispatch");
            void* hidden = ctx.take_rows(max_rows, ff_, dtype);
            if (clamped_)
                launch_check(eg_gemm_tcgen05_grouped_glu(ctx.stream, rows, hidden_, gate_up_.get(), hidden_, hidden, ff_, max_rows, 2 * ff_, hidden_, experts_,
                                                         tile_group, ctx.status, limit_), "gemm_tcgen05_grouped_glu");
            else
                launch_check(eg_gemm_tcgen05_grouped(ctx.stream, plans::EPI_SWIGLU, rows, hidden_, gate_up_.get(), hidden_, hidden, ff_, max_rows, 2 * ff_, hidden_,
                                                     experts_, tile_group, ctx.status), "gemm_tcgen05_grouped");
            launch_check(eg_gemm_tcgen05_grouped(ctx.stream, plans::EPI_STORE, hidden, ff_, down_.get(), ff_, rows, hidden_, max_rows, hidden_, ff_, experts_,
                                                 tile_group, ctx.status), "gemm_tcgen05_grouped");
            launch_check(eg_moe_gather(ctx.stream, rows, row_of, ids, out_w, h.p, h.ld, shared.p, (int)shared.dtype, gate, out, T, hidden_, top_, experts_),
                         "moe_gather");
            Delta d;
            d.p = out;
            d.dtype = DType::F32;
            return d;
        }
        void* act = ctx.take_rows((size_t)T * top_, std::max(ff_, 1), dtype);
        launch_check(eg_moe_hidden(ctx.stream, (int)dtype, h.p, h.ld, gate_up_.get(), ids, in_w, act, T, hidden_, ff_, top_, experts_, clamped_ ? 1 : 0, limit_),
                     "moe_hidden");
        launch_check(eg_moe_combine(ctx.stream, (int)dtype, h.p, h.ld, act, down_.get(), ids, out_w, shared.p, (int)shared.dtype, gate, out, T, hidden_, ff_,
                                    top_, experts_), "moe_combine");
        Delta d;
        d.p = out;
        d.dtype = DType::F32;
        return d;
    }

private:
    int hidden_, experts_, identity_, top_, ff_, shared_ff_;
    bool sigmoid_, corrected_, clamped_, weight_input_, shared_gated_;
    float limit_;
    DType dtype_ = DType::BF16;
    std::shared_ptr<SwiGLU> shared_;
    DeviceBuffer router_, correction_, gate_up_, down_, shared_gate_;
};

inline void register_sequence_parts() {
    PartRegistry& r = PartRegistry::instance();
    if (r.mixers.count("selective_scan")) return;
    r.mixers["selective_scan"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<SelectiveScanMixer>(p, prefix, std::move(pos));
    };
    r.mixers["latent_attention"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<LatentAttention>(p, prefix, std::move(pos));
    };
    r.feed_forwards["routed_experts"] = [](const Params& p, const std::string& prefix) { return std::make_shared<RoutedExperts>(p, prefix); };
}

}  // namespace easygpt::engine
