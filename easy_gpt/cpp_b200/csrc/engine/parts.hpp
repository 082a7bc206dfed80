// The parts the engine ships: grouped-query attention over the paged cache, the SwiGLU feed-forward, RMSNorm,
// the rotary position encoding, the token embedding and the output head, and the linear product they share.
// Formulas and their order are the reference's (cited at each part); sizes and constants are parameters.
#pragma once
#include <cmath>
#include <cstring>

#include "parts_base.hpp"

namespace easygpt::engine {

// ---- host-side assembly of weights ---------------------------------------------------------------------------
inline std::vector<float> host_floats(const StoredTensor& t) {
    std::vector<float> out((size_t)t.numel());
    t.to_float(out.data());
    return out;
}
inline const StoredTensor& need_tensor(const HostTensors& file, const std::string& name) {
    const StoredTensor* t = file.find(name);
    if (!t) throw WeightError("Missing required model weights: " + name);
    return *t;
}
// float32 values -> device memory in `dtype` (bfloat16: round to nearest even)
inline DeviceBuffer upload(const float* values, size_t n, DType dtype) {
    DeviceBuffer buf(n * dtype_size(dtype));
    if (dtype == DType::F32) {
        EG_CUDA(cudaMemcpy(buf.get(), values, n * 4, cudaMemcpyHostToDevice));
    } else {
        std::vector<uint16_t> low(n);
        for (size_t i = 0; i < n; ++i) low[i] = float_to_bf16(values[i]);
        EG_CUDA(cudaMemcpy(buf.get(), low.data(), n * 2, cudaMemcpyHostToDevice));
    }
    return buf;
}
// a stored tensor as it is, where its stored precision is the wanted one (no round trip through float32)
inline DeviceBuffer upload(const StoredTensor& t, DType dtype) {
    if ((t.dtype == Stored::BF16 && dtype == DType::BF16) || (t.dtype == Stored::F32 && dtype == DType::F32)) {
        DeviceBuffer buf(t.bytes);
        EG_CUDA(cudaMemcpy(buf.get(), t.data, t.bytes, cudaMemcpyHostToDevice));
        return buf;
    }
    const std::vector<float> f = host_floats(t);
    return upload(f.data(), f.size(), dtype);
}

// ---- y = x W^T + b with W stored [out, in] (src/models/linear.cpp:42-44) ------------------------------------------
// In bfloat16, steps of up to 16 tokens go to the engine's own weight-streaming kernel (gemm_skinny.cu); larger ones
// to the library product (cuBLAS), where the reference's engine calls cublasGemmEx too (src/cuda/ops/matmul.cu:194-204).
// In float32 it is always the engine's own FFMA kernel: true 32-bit arithmetic whose sums do not depend on the batch.
struct SkinnyRope {
    int num_heads, num_kv_heads, head_dim;
    const int *positions, *slot_map;
    void *k_cache, *v_cache;
    const float* inv_freq;
    int page_size;
    long long page_stride, head_stride, pool_slots;
};

class Linear {
public:
    Linear() = default;
    Linear(const float* w, int out_features, int in_features, const float* bias, DType dtype)
        : out_features(out_features), in_features(in_features), dtype(dtype) {
        store_ = upload(w, (size_t)out_features * in_features, dtype);
        weight = store_.get();
        set_bias(bias);
    }
    Linear(const StoredTensor& w, const float* bias, DType dtype)
        : out_features((int)w.shape[0]), in_features((int)w.shape[1]), dtype(dtype) {
        store_ = upload(w, dtype);
        weight = store_.get();
        set_bias(bias);
    }
    // a bias-free product with a weight that another part owns (a tied head multiplies by the embedding table itself)
    static Linear sharing(const void* weight, int out_features, int in_features, DType dtype) {
        Linear l;
        l.weight = weight;
        l.out_features = out_features;
        l.in_features = in_features;
        l.dtype = dtype;
        return l;
    }
    size_t weight_bytes() const { return (size_t)out_features * in_features * dtype_size(dtype); }

    static bool aligned(const Rows& x) { return x.ld % 8 == 0 && (uintptr_t)x.p % 16 == 0; }

    // the decode product with every prologue and epilogue it has; see csrc/gemm_skinny.cu
    void skinny(const StepContext& ctx, int epilogue, int M, const Rows* x, const NormInFront* norm, void* out, long long ldo,
                const SkinnyRope* rope, float* follow_residual, const float* follow_gain, void* xn_out, float* ss_out,
                const plans::SkinnyPlan* plan_override = nullptr) const {
        const int N = out_features, K = in_features;
        const plans::SkinnyPlan plan = plan_override ? *plan_override : plans::skinny_plan(N, K, rope ? rope->head_dim : 0);
        int norm_mode = 0;
        const void* delta = nullptr;
        const float *resid_in = nullptr, *gain = nullptr, *ss_in = nullptr;
        float* resid_out = nullptr;
        float eps = 0.f;
        int ss_parts = 0;
        if (norm) {
            eps = norm->eps;
            if (norm->prepared_rows) {
                norm_mode = 2;
                delta = norm->prepared_rows;
                ss_in = norm->prepared_sums;
                ss_parts = norm->prepared_parts;
            } else {
                norm_mode = 1;
                resid_in = norm->residual;
                resid_out = norm->residual_out;
                delta = norm->delta;
                gain = norm->gain;
            }
        }
        float* partials = nullptr;
        int* counters = nullptr;
        if (plan.k_split > 1) {
            const size_t groups = (size_t)(N + plan.row_blocks * 16 - 1) / (plan.row_blocks * 16);
            const size_t floats = (size_t)plan.k_split * groups * plan.row_blocks * 16 * plans::skinny_padded_tokens(M);
            if (floats > KernelScratch::SKINNY_FLOATS || groups > KernelScratch::SKINNY_COUNTERS)
                throw DeviceError("a decode product's split needs more scratch memory than the engine holds");
            partials = ctx.scratch->skinny_partials.as<float>();
            counters = ctx.scratch->skinny_counters.as<int>();
        }
        SkinnyRope none{};
        const SkinnyRope& r = rope ? *rope : none;
        launch_check(eg_gemm_skinny(ctx.stream, epilogue, norm_mode, plans::use_pdl(), weight, in_features, bias_f32(), M, N, K,
                                    x ? x->p : nullptr, x ? x->ld : 0, resid_in, resid_out, delta, gain, eps, out, ldo, plan.row_blocks,
                                    plan.k_slices, plan.k_split, partials, counters, r.num_heads, r.num_kv_heads, r.head_dim, r.positions,
                                    r.slot_map, r.k_cache, r.v_cache, r.inv_freq, r.page_size, r.page_stride, r.head_stride, r.pool_slots,
                                    ctx.status, nullptr, 0, nullptr, ss_in, ss_parts, follow_residual, follow_gain, xn_out, ss_out),
                     "gemm_skinny");
    }

    // out [M, out_features] (compute dtype, from the arena) = xielu(x W^T) by the decode product, the activation on its
    // finished sums; the caller has checked that the decode product takes the input
    Rows skinny_xielu(const StepContext& ctx, const Rows& x, float act_a, float act_b) const {
        const int M = x.rows, N = out_features;
        const plans::SkinnyPlan plan = plans::skinny_plan(N, in_features, 0);
        float* partials = nullptr;
        int* counters = nullptr;
        if (plan.k_split > 1) {
            const size_t groups = (size_t)(N + plan.row_blocks * 16 - 1) / (plan.row_blocks * 16);
            const size_t floats = (size_t)plan.k_split * groups * plan.row_blocks * 16 * plans::skinny_padded_tokens(M);
            if (floats > KernelScratch::SKINNY_FLOATS || groups > KernelScratch::SKINNY_COUNTERS)
                throw DeviceError("a decode product's split needs more scratch memory than the engine holds");
            partials = ctx.scratch->skinny_partials.as<float>();
            counters = ctx.scratch->skinny_counters.as<int>();
        }
        Rows out{ctx.take_rows(M, N, DType::BF16), DType::BF16, M, N, N};
        launch_check(eg_gemm_skinny_xielu(ctx.stream, plans::use_pdl(), weight, in_features, M, N, in_features, x.p, x.ld, out.p, N, plan.row_blocks,
                                          plan.k_slices, plan.k_split, partials, counters, ctx.status, act_a, act_b), "gemm_skinny_xielu");
        return out;
    }

    // the same with act(z) = max(z, 0)^2 (limit 0), or, over interleaved gate and up rows, the clamped gate (limit > 0):
    // out [M, out_features / 2]
    Rows skinny_relu2(const StepContext& ctx, const Rows& x) const { return skinny_act(ctx, x, 0.f); }
    Rows skinny_clamped_glu(const StepContext& ctx, const Rows& x, float limit) const { return skinny_act(ctx, x, limit); }
    Rows skinny_act(const StepContext& ctx, const Rows& x, float limit) const {
        const int M = x.rows, N = out_features;
        const plans::SkinnyPlan plan = plans::skinny_plan(N, in_features, 0);
        float* partials = nullptr;
        int* counters = nullptr;
        if (plan.k_split > 1) {
            const size_t groups = (size_t)(N + plan.row_blocks * 16 - 1) / (plan.row_blocks * 16);
            const size_t floats = (size_t)plan.k_split * groups * plan.row_blocks * 16 * plans::skinny_padded_tokens(M);
            if (floats > KernelScratch::SKINNY_FLOATS || groups > KernelScratch::SKINNY_COUNTERS)
                throw DeviceError("a decode product's split needs more scratch memory than the engine holds");
            partials = ctx.scratch->skinny_partials.as<float>();
            counters = ctx.scratch->skinny_counters.as<int>();
        }
        const int cols = limit > 0.f ? N / 2 : N;
        Rows out{ctx.take_rows(M, cols, DType::BF16), DType::BF16, M, cols, cols};
        if (limit > 0.f)
            launch_check(eg_gemm_skinny_clamped_glu_bias(ctx.stream, plans::use_pdl(), weight, in_features, bias_f32(), M, N, in_features, x.p, x.ld, out.p, cols,
                                                         plan.row_blocks, plan.k_slices, plan.k_split, partials, counters, ctx.status, limit), "gemm_skinny_clamped_glu");
        else
            launch_check(eg_gemm_skinny_relu2(ctx.stream, plans::use_pdl(), weight, in_features, M, N, in_features, x.p, x.ld, out.p, N, plan.row_blocks,
                                              plan.k_slices, plan.k_split, partials, counters, ctx.status), "gemm_skinny_relu2");
        return out;
    }

    // whether with_following_norm can run for this input (the decode kernel takes it)
    bool takes_following_norm(const Rows& x) const {
        return dtype == DType::BF16 && plans::gemm_skinny_takes(dtype, x.rows, in_features) && x.rows <= plans::FUSED_NORM_MAX_TOKENS && aligned(x);
    }
    // The product, the add to the residual and the preparation of the norm that follows, in one kernel:
    // follow.residual() += x W^T + b (in place); returns a PreNormed for follow.norm.
    PreNormed with_following_norm(const StepContext& ctx, const Rows& x, const FollowingNorm& follow) const {
        const plans::SkinnyPlan plan = plans::skinny_plan(out_features, in_features);
        const int parts = (out_features + plan.row_blocks * 16 - 1) / (plan.row_blocks * 16);
        void* xn = ctx.take_rows(x.rows, out_features, DType::BF16);
        float* ss = ctx.take<float>((size_t)parts * plans::skinny_padded_tokens(x.rows));
        skinny(ctx, plans::EPI_RESID_NORM, x.rows, &x, nullptr, nullptr, 0, nullptr, follow.residual(), follow.gain, xn, ss, &plan);
        return PreNormed{follow.norm, xn, ss, parts};
    }

    // out [M, out_features] from the arena, in the compute dtype or (out_f32) in float32
    Rows operator()(const StepContext& ctx, const Rows& x, bool out_f32 = false) const {
        const int M = x.rows;
        Rows out{nullptr, (out_f32 || dtype == DType::F32) ? DType::F32 : DType::BF16, M, out_features, out_features};
        out.p = ctx.take_rows(M, out_features, out.dtype);
        if (dtype == DType::F32) {
            launch_check(eg_gemm_f32_nt(ctx.stream, (const float*)x.p, (int)x.ld, (const float*)weight, in_features, bias_f32(), (float*)out.p,
                                        out_features, M, out_features, in_features), "gemm_f32_nt");
            return out;
        }
        if (plans::gemm_skinny_takes(dtype, M, in_features) && aligned(x)) {
            skinny(ctx, out_f32 ? plans::EPI_F32 : plans::EPI_STORE, M, &x, nullptr, out.p, out_features, nullptr, nullptr, nullptr, nullptr, nullptr);
            return out;
        }
        // the library's product into float32 takes no bias: it is added by a kernel behind it, in float32
        ctx.blas->gemm_bf16(ctx.stream, x.p, x.ld, weight, in_features, has_bias() && !out_f32 ? bias_lp_.get() : nullptr, out.p, out_features, M, out_features,
                            in_features, out_f32);
        if (out_f32 && has_bias()) launch_check(eg_add_bias_rows(ctx.stream, (float*)out.p, out_features, bias_f32(), M, out_features), "add_bias_rows");
        return out;
    }

    // The product into float32 whose bias may be left to the consumer: where the library runs it (which writes float32 without a
    // bias) *pending_bias is set to the bias and nothing is added here; our own kernels add it themselves (*pending_bias null).
    Rows f32_bias_pending(const StepContext& ctx, const Rows& x, const float** pending_bias) const {
        *pending_bias = nullptr;
        if (dtype == DType::F32 || !has_bias() || (plans::gemm_skinny_takes(dtype, x.rows, in_features) && aligned(x))) return (*this)(ctx, x, true);
        *pending_bias = bias_f32();
        return without_bias_f32(ctx, x);
    }
    // the bare product into float32, for a consumer whose own kernel adds the bias
    Rows without_bias_f32(const StepContext& ctx, const Rows& x) const {
        const int M = x.rows;
        Rows out{ctx.take_rows(M, out_features, DType::F32), DType::F32, M, out_features, out_features};
        if (dtype == DType::F32)
            launch_check(eg_gemm_f32_nt(ctx.stream, (const float*)x.p, (int)x.ld, (const float*)weight, in_features, nullptr, (float*)out.p, out_features, M,
                                        out_features, in_features), "gemm_f32_nt");
        else
            ctx.blas->gemm_bf16(ctx.stream, x.p, x.ld, weight, in_features, nullptr, out.p, out_features, M, out_features, in_features, true);
        return out;
    }
    const float* bias_f32() const { return bias_f32_.get() ? bias_f32_.as<float>() : nullptr; }
    bool has_bias() const { return bias_f32_.get() != nullptr; }

    const void* weight = nullptr;
    int out_features = 0, in_features = 0;
    DType dtype = DType::BF16;

private:
    void set_bias(const float* bias) {
        if (!bias) return;
        // the bias is added in float32 by our kernels; the library product wants it in its own dtype
        bias_f32_ = upload(bias, (size_t)out_features, DType::F32);
        if (dtype == DType::BF16) bias_lp_ = upload(bias, (size_t)out_features, DType::BF16);
    }
    DeviceBuffer store_, bias_f32_, bias_lp_;
};

// ---- RMSNorm: y = w * (x / sqrt(mean(x^2) + eps)) (src/models/norm.cpp:46-60), eps a parameter (the reference fixes
// 1e-6, src/models/norm.cpp:41), fused with the float32 residual add; with single_gain the stored gain is one number ---------------------------------------------------
class RMSNorm : public Norm {
public:
    RMSNorm(const Params& p, const std::string& prefix)
        : Norm(p, prefix), size_((int)p.integer("size")), eps_((float)p.real("eps")), weight_name_(prefix + p.text("weight_name", ".weight")),
          single_(p.integer("single_gain", 0) != 0), offset_((float)p.real("offset", 0.0)) {}
    std::vector<TensorRequest> tensor_requests() const override {
        return {(single_ ? TensorRequest::scalar(weight_name_) : TensorRequest::vector(weight_name_, size_)).with_init(offset_ != 0.f ? "zero" : "one")};
    }
    void load(const HostTensors& file, DType) override {
        std::vector<float> g = host_floats(need_tensor(file, weight_name_));       // gains are used in float32 whatever they were stored in
        if (single_) g.assign((size_t)size_, g.at(0));                               // one number for all coordinates: the kernels read a gain per channel
        if (offset_ != 0.f)                                                          // the tensor holds the gain's distance from the offset: the kernels read offset + w
            for (float& v : g) v += offset_;
        gain_ = upload(g.data(), g.size(), DType::F32);
    }
    size_t weight_bytes() const override { return (size_t)size_ * 4; }
    bool capturable() const override { return true; }
    bool rms_parameters(const float** gain, float* eps) const override {
        *gain = gain_.as<float>();
        *eps = eps_;
        return true;
    }
    void forward(const StepContext& ctx, float* residual, const void* delta, DType delta_dtype, void* out, DType out_dtype, int num_rows,
                 const int* rows) const override {
        launch_check(eg_add_rmsnorm(ctx.stream, (int)(delta ? delta_dtype : out_dtype), (int)out_dtype, residual, delta, rows, gain_.as<float>(), out,
                                    num_rows, size_, eps_), "add_rmsnorm");
    }
    bool add_normed(const StepContext& ctx, float* residual, const void* y, DType y_dtype, int num_rows) const override {
        launch_check(eg_rmsnorm_add(ctx.stream, residual, y, (int)y_dtype, size_, gain_.as<float>(), eps_, num_rows, size_), "rmsnorm_add");
        return true;
    }
    bool add_normed_rows(const StepContext& ctx, float* residual, const void* y, DType y_dtype, const float* bias, int num_rows, void* out,
                         DType out_dtype) const override {
        const int rc = eg_rmsnorm_add_rows(ctx.stream, residual, y, (int)y_dtype, size_, bias, gain_.as<float>(), eps_, out, (int)out_dtype, num_rows, size_);
        if (rc == (int)cudaErrorInvalidValue) return false;      // a size the fused kernel does not take
        launch_check(rc, "rmsnorm_add_rows");
        return true;
    }
    bool add_normed_then(const StepContext& ctx, float* residual, const void* y, DType y_dtype, int num_rows, const Norm* next, void* out,
                         DType out_dtype) const override {
        const float* gain2 = nullptr;
        float eps2 = 0.f;
        if (!next || next->size() != size_ || !next->rms_parameters(&gain2, &eps2)) return false;
        const int rc = eg_rmsnorm_add_norm(ctx.stream, residual, y, (int)y_dtype, size_, gain_.as<float>(), eps_, gain2, eps2, out, (int)out_dtype, num_rows, size_);
        if (rc == (int)cudaErrorInvalidValue) return false;      // a size the fused kernel does not take
        launch_check(rc, "rmsnorm_add_norm");
        return true;
    }
    int size() const override { return size_; }

private:
    int size_;
    float eps_;
    std::string weight_name_;      // parameter weight_name: the gain's tensor name as a suffix of the prefix (default ".weight")
    bool single_;                  // parameter single_gain: the tensor is ONE number, the gain of every coordinate
    float offset_;                 // parameter offset: the gain is offset + the stored tensor (1 where the file holds the gain minus one)
    DeviceBuffer gain_;
};

// ---- layer norm with gain and bias: y = (x - mean(x)) / sqrt(var(x) + eps) * w + b, var the mean of the squared
// deviations, fused with the float32 residual add.  Two layer norms of the same width and eps that read the same stream
// (a layer whose mixer and feed-forward run side by side) leave one kernel together.  Parameters: size, eps,
// weight_name / bias_name (tensor names under the prefix; defaults ".weight" / ".bias") ---------------------------------
class LayerNorm : public Norm {
public:
    LayerNorm(const Params& p, const std::string& prefix)
        : Norm(p, prefix), size_((int)p.integer("size")), eps_((float)p.real("eps")), weight_name_(prefix + p.text("weight_name", ".weight")),
          bias_name_(prefix + p.text("bias_name", ".bias")) {}
    std::vector<TensorRequest> tensor_requests() const override {
        return {TensorRequest::vector(weight_name_, size_).with_init("one"), TensorRequest::vector(bias_name_, size_).with_init("zero")};
    }
    void load(const HostTensors& file, DType) override {
        const std::vector<float> g = host_floats(need_tensor(file, weight_name_)), b = host_floats(need_tensor(file, bias_name_));
        gain_ = upload(g.data(), g.size(), DType::F32);
        bias_ = upload(b.data(), b.size(), DType::F32);
    }
    size_t weight_bytes() const override { return (size_t)size_ * 8; }
    bool capturable() const override { return true; }
    void forward(const StepContext& ctx, float* residual, const void* delta, DType delta_dtype, void* out, DType out_dtype, int num_rows,
                 const int* rows) const override {
        launch_check(eg_add_layernorm(ctx.stream, residual, delta, (int)delta_dtype, nullptr, 0, rows, gain_.as<float>(), bias_.as<float>(), out, nullptr,
                                      nullptr, nullptr, (int)out_dtype, num_rows, size_, eps_), "add_layernorm");
    }
    bool forward_pair(const StepContext& ctx, float* residual, const void* delta_a, DType dtype_a, const void* delta_b, DType dtype_b, const Norm* second,
                      void* out, void* out2, DType out_dtype, int num_rows) const override {
        const LayerNorm* other = dynamic_cast<const LayerNorm*>(second);
        if (!other || other->size_ != size_ || other->eps_ != eps_) return false;
        launch_check(eg_add_layernorm(ctx.stream, residual, delta_a, (int)dtype_a, delta_b, (int)dtype_b, nullptr, gain_.as<float>(), bias_.as<float>(), out,
                                      other->gain_.as<float>(), other->bias_.as<float>(), out2, (int)out_dtype, num_rows, size_, eps_), "add_layernorm");
        return true;
    }
    int size() const override { return size_; }

private:
    int size_;
    float eps_;
    std::string weight_name_, bias_name_;
    DeviceBuffer gain_, bias_;
};

// ---- learned vectors added to the stream before a pass of a repeated run of layers: x += (first) + table[row].
// Parameters: rows, hidden_size; the table is the tensor named by the prefix itself -----------------------------------------
class PassOffsets : public StreamAdd {
public:
    PassOffsets(const Params& p, const std::string& prefix) : StreamAdd(p, prefix), rows_((int)p.integer("rows")), hidden_((int)p.integer("hidden_size")) {}
    std::vector<TensorRequest> tensor_requests() const override { return {TensorRequest::matrix(prefix, rows_, hidden_)}; }
    void load(const HostTensors& file, DType) override {
        const std::vector<float> t = host_floats(need_tensor(file, prefix));
        table_ = upload(t.data(), t.size(), DType::F32);
    }
    bool capturable() const override { return true; }
    void forward(const StepContext& ctx, float* residual, const float* first, int row) const override {
        if (row < 0 || row >= rows_) throw DeviceError("a pass names row " + std::to_string(row) + " of a table of " + std::to_string(rows_));
        launch_check(eg_stream_add(ctx.stream, residual, first, table_.as<float>() + (size_t)row * hidden_, ctx.num_tokens, hidden_), "stream_add");
    }

private:
    int rows_, hidden_;
    DeviceBuffer table_;
};

// ---- rotary position encoding, half rotation over rotary_dim dimensions of each head (src/ops.cpp:404-421).  The table
// inv_freq[k] = theta^(-2k/rotary_dim) (src/ops.cpp:172-177) is built once on the host, in double, rounded to float32.
// With scaling_factor s > 1 (and scaling_original L, scaling_fast b_f, scaling_slow b_s) the frequencies are stretched
// for long contexts: with turn(b) = rotary_dim ln(L / (2 pi b)) / (2 ln theta), the index of the pair that makes b turns
// over L positions, lo = max(floor(turn(b_f)), 0), hi = min(ceil(turn(b_s)), rotary_dim - 1),
// r_k = clamp((k - lo) / max(hi - lo, 0.001), 0, 1), inv_freq[k] <- inv_freq[k] (r_k / s + 1 - r_k), and cos and sin
// are multiplied by 0.1 ln s + 1 (HalfRotation::magnitude) -----
class RotaryEncoding : public PositionEncoding {
public:
    RotaryEncoding(const Params& p, const std::string& prefix)
        : PositionEncoding(p, prefix), head_dim_((int)p.integer("head_dim")), rotary_dim_((int)p.integer("rotary_dim", p.integer("head_dim"))),
          theta_(p.real("theta")), factor_(p.has("scaling_factor") ? p.real("scaling_factor") : 0.0) {
        if (rotary_dim_ % 2 || rotary_dim_ <= 0 || rotary_dim_ > head_dim_)
            throw std::invalid_argument("rotary_dim " + std::to_string(rotary_dim_) + " must be even and within head_dim " + std::to_string(head_dim_));
        if (theta_ <= 0) throw std::invalid_argument("rope theta must be > 0");
        if (factor_ != 0.0) {
            original_ = p.real("scaling_original");
            fast_ = p.real("scaling_fast");
            slow_ = p.real("scaling_slow");
            if (factor_ <= 0.0 || original_ <= 0.0 || fast_ <= 0.0 || slow_ <= 0.0 || theta_ == 1.0)
                throw std::invalid_argument("a rotation's scaling needs positive factor, original, fast and slow, and a base other than 1");
            magnitude_ = (float)(0.1 * std::log(factor_) + 1.0);
        }
    }
    void load(const HostTensors&, DType) override {
        std::vector<float> inv(rotary_dim_ / 2);
        for (int k = 0; k < rotary_dim_ / 2; ++k) {
            double f = 1.0 / std::pow(theta_, 2.0 * k / rotary_dim_);
            if (factor_ != 0.0) {
                auto turn = [&](double b) { return rotary_dim_ * std::log(original_ / (2.0 * M_PI * b)) / (2.0 * std::log(theta_)); };
                const double lo = std::max(std::floor(turn(fast_)), 0.0), hi = std::min(std::ceil(turn(slow_)), (double)rotary_dim_ - 1.0);
                const double ramp = std::min(1.0, std::max(0.0, (k - lo) / std::max(hi - lo, 0.001)));
                f = f / factor_ * ramp + f * (1.0 - ramp);
            }
            inv[k] = (float)f;
        }
        inv_freq_ = upload(inv.data(), inv.size(), DType::F32);
    }
    bool capturable() const override { return true; }
    bool half_rotation(HalfRotation* out) const override {
        out->inv_freq = inv_freq_.as<float>();
        out->rotary_dim = rotary_dim_;
        out->magnitude = magnitude_;
        out->key = "rope:" + std::to_string(theta_) + ":" + std::to_string(rotary_dim_);
        if (factor_ != 0.0) out->key += ":" + std::to_string(factor_) + ":" + std::to_string(original_) + ":" + std::to_string(fast_) + ":" + std::to_string(slow_);
        return true;
    }

private:
    int head_dim_, rotary_dim_;
    double theta_, factor_, original_ = 0.0, fast_ = 0.0, slow_ = 0.0;
    float magnitude_ = 1.0f;
    DeviceBuffer inv_freq_;
};

// cos/sin [T, rotary_dim/2, 2] of this step's positions: computed by the first layer that asks and shared by every layer
// whose rotation has the same key
inline const float* step_rotation_table(const StepContext& ctx, const HalfRotation& rot) {
    auto& shared = const_cast<StepContext&>(ctx).shared;
    const std::string key = "rotation table " + rot.key;
    auto it = shared.find(key);
    if (it != shared.end()) return (const float*)it->second;
    float* table = ctx.take_for_step<float>((size_t)ctx.num_tokens * rot.rotary_dim);
    launch_check(eg_rope_table(ctx.stream, ctx.positions, rot.inv_freq, table, ctx.num_tokens, rot.rotary_dim / 2), "rope_table");
    shared[key] = table;
    return table;
}

// ---- grouped-query attention over the paged cache -----------------------------------------------------------------
// Per token: q, k, v = x Wq^T + bq, ... (src/models/self_attn.cpp:225-227) as ONE product with the three weights
// stacked; q and k are changed by the layer's position encoding (a half rotation is applied by the kernel that also
// stores k, v in the cache; another encoding changes q and k itself; none is fine too); every query head h attends
// the keys of KV head h / (NH/NKV) of its own request up to its own position (optionally only the last `window` of
// them); the heads are concatenated head-major and projected by Wo (src/models/self_attn.cpp:255-258).  Scale
// 1/sqrt(head_dim) (:253).  Parameters: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, out_bias, window.
class Attention : public Mixer {
public:
    Attention(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
        : Mixer(p, prefix, std::move(position)), hidden_((int)p.integer("hidden_size")), heads_((int)p.integer("num_heads")),
          kv_heads_((int)p.integer("num_kv_heads")), head_dim_((int)p.integer("head_dim")), qkv_bias_(p.flag("qkv_bias", false)),
          out_bias_(p.flag("out_bias", false)), window_(p.has("window") ? p.integer("window") : -1) {
        if (heads_ % kv_heads_) throw std::invalid_argument("num_heads must be a multiple of num_kv_heads");
        if (p.has("window") && window_ <= 0) throw std::invalid_argument("window must be positive");
        if (head_dim_ <= 0 || head_dim_ > plans::MAX_HEAD_DIM)
            throw std::invalid_argument("head_dim " + std::to_string(head_dim_) + " is outside what the attention kernels take (1.." +
                                        std::to_string(plans::MAX_HEAD_DIM) + ")");
        scale_ = (float)(1.0 / std::sqrt((double)head_dim_));
    }
    std::vector<TensorRequest> tensor_requests() const override {
        const long long q_out = (long long)heads_ * head_dim_, kv_out = (long long)kv_heads_ * head_dim_;
        std::vector<TensorRequest> r = {TensorRequest::matrix(prefix + ".q_proj.weight", q_out, hidden_), TensorRequest::matrix(prefix + ".k_proj.weight", kv_out, hidden_),
                                        TensorRequest::matrix(prefix + ".v_proj.weight", kv_out, hidden_), TensorRequest::matrix(prefix + ".o_proj.weight", hidden_, q_out)};
        if (qkv_bias_) {
            r.push_back(TensorRequest::vector(prefix + ".q_proj.bias", q_out));
            r.push_back(TensorRequest::vector(prefix + ".k_proj.bias", kv_out));
            r.push_back(TensorRequest::vector(prefix + ".v_proj.bias", kv_out));
        }
        if (out_bias_) r.push_back(TensorRequest::vector(prefix + ".o_proj.bias", hidden_));
        return r;
    }
    void load(const HostTensors& file, DType dtype) override {
        std::vector<float> w, b;
        for (const char* n : {"q", "k", "v"}) {
            const std::vector<float> part = host_floats(need_tensor(file, prefix + "." + n + "_proj.weight"));
            w.insert(w.end(), part.begin(), part.end());
            if (qkv_bias_) {
                const std::vector<float> bias = host_floats(need_tensor(file, prefix + "." + n + "_proj.bias"));
                b.insert(b.end(), bias.begin(), bias.end());
            }
        }
        const int rows = (heads_ + 2 * kv_heads_) * head_dim_;
        qkv_ = Linear(w.data(), rows, hidden_, qkv_bias_ ? b.data() : nullptr, dtype);
        std::vector<float> ob;
        if (out_bias_) ob = host_floats(need_tensor(file, prefix + ".o_proj.bias"));
        out_ = Linear(need_tensor(file, prefix + ".o_proj.weight"), out_bias_ ? ob.data() : nullptr, dtype);
        if (position) position->load(file, dtype);
    }
    size_t weight_bytes() const override { return qkv_.weight_bytes() + out_.weight_bytes(); }
    bool capturable() const override { return true; }
    CacheNeed cache_need() const override { return CacheNeed::paged(kv_heads_, head_dim_, window_); }
    bool accepts_pending_norm() const override { return true; }
    bool fuses_following_norm() const override { return true; }

    // norm + QKV (+ bias, rotation, cache write); attention over the cache; output projection into the residual
    bool emit_fused(FusedBuilder& b, const float* gain, float eps, const CacheView& cache) const override {
        const StepContext& ctx = *b.ctx;
        HalfRotation rot;
        const bool rotates = position && position->half_rotation(&rot);
        const int G = heads_ / kv_heads_;
        if (ctx.dtype != DType::BF16 || head_dim_ != 64 || G > 16 || cache.group < 0 || !cache.writes || cache.page_size % 16 || hidden_ != b.hidden) return false;
        if (position && (!rotates || rot.rotary_dim != head_dim_)) return false;
        const GroupTables& tables = ctx.groups.at(cache.group);
        const int q_width = heads_ * head_dim_, T = b.tokens;
        void* q = b.arena->take((size_t)T * q_width * 2);
        void* attn = b.arena->take((size_t)T * q_width * 2);
        EgFusedTemplate t = FusedBuilder::blank();
        t.input = EGF_IN_NORM;
        t.output = EGF_OUT_QKV_ROPE;
        t.N = (heads_ + 2 * kv_heads_) * head_dim_;
        t.K = hidden_;
        t.tiles_per_unit = 2;
        t.group_rows = head_dim_;
        t.units_per_group = head_dim_ / 16;
        t.pair_offset = head_dim_ / 2;
        t.eps = eps;
        t.out = q;
        t.ldo = q_width;
        t.num_heads = heads_;
        t.num_kv_heads = kv_heads_;
        t.head_dim = head_dim_;
        t.page_size = cache.page_size;
        t.num_pages = cache.num_pages;
        t.positions = ctx.positions;
        t.slot_map = tables.slot_map;
        t.inv_freq = rotates ? rot.inv_freq : nullptr;
        t.page_stride = cache.page_stride;
        t.head_stride = cache.head_stride;
        t.pool_slots = (long long)cache.num_pages * cache.page_size;
        if (!b.linear(t, qkv_.weight, hidden_, qkv_.bias_f32(), gain, cache.k, cache.v)) return false;

        // as many CTAs per (token, KV head) as the grid has for them, a key tile each at least
        const long long longest = window_ < 0 ? ctx.max_context_len : std::min<long long>(ctx.max_context_len, window_ + 255);
        const int tiles = (int)std::max<long long>(1, (longest + 63) / 64);
        // (at most 16, and four tiles each where there are that many: the merge of the splits is one CTA's work)
        const int splits = std::max(1, std::min({std::max(1, tiles / 4), 16, b.grid / std::max(1, T * kv_heads_)}));
        EgFusedTemplate a = FusedBuilder::blank();
        a.num_heads = heads_;
        a.num_kv_heads = kv_heads_;
        a.head_dim = head_dim_;
        a.page_size = cache.page_size;
        a.num_pages = cache.num_pages;
        a.window = window_ < 0 ? 0 : (int)window_;
        a.positions = ctx.positions;
        a.page_stride = cache.page_stride;
        a.head_stride = cache.head_stride;
        a.q = q;
        a.ldq = q_width;
        a.block_table = tables.block_table;
        a.table_stride = tables.table_width;
        a.seq_context = ctx.seq_context;
        a.scale = scale_;
        a.splits = splits;
        if (splits > 1) {
            if ((size_t)T * kv_heads_ > KernelScratch::ATTENTION_COUNTERS) return false;
            a.partial_acc = b.arena->take_n<float>((size_t)T * heads_ * splits * head_dim_);
            a.partial_ml = b.arena->take_n<float>((size_t)T * heads_ * splits * 2);
            a.tickets = ctx.scratch->attention_counters.as<int>();
        }
        a.attn_out = attn;
        a.ld_attn = q_width;
        b.attention(a, cache.k, cache.v);

        EgFusedTemplate o = FusedBuilder::blank();
        o.input = EGF_IN_ROWS;
        o.output = EGF_OUT_RESIDUAL;
        o.N = hidden_;
        o.K = q_width;
        o.tiles_per_unit = 1;
        o.group_rows = 8;
        o.units_per_group = 1;
        o.x = attn;
        o.ldx = q_width;
        return b.linear(o, out_.weight, q_width, out_.bias_f32(), nullptr);
    }

    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm* follow) override {
        const int T = ctx.num_tokens;
        const GroupTables& tables = ctx.groups.at(cache.group);
        const DType dtype = ctx.dtype;
        const int q_width = heads_ * head_dim_, kv_width = kv_heads_ * head_dim_;
        const long long pool_slots = (long long)cache.num_pages * cache.page_size;
        HalfRotation rot;
        const bool rotates = position && position->half_rotation(&rot);
        if (rotates && rot.magnitude != 1.0f) throw DeviceError("this attention's kernels take no rotation with a factor on cos and sin");
        Rows qkv;
        if (in.pending && in.pending->fusable && cache.writes && rotates && rot.rotary_dim == head_dim_ &&
            (head_dim_ == 16 || head_dim_ == 32 || head_dim_ == 64 || head_dim_ == 128)) {
            // decode: add + norm + QKV product + bias + rotation + cache write in one kernel
            qkv = Rows{ctx.take_rows(T, q_width, dtype), dtype, T, q_width, q_width};
            const NormInFront norm = in.pending->fused();
            const SkinnyRope rope{heads_, kv_heads_, head_dim_, ctx.positions, tables.slot_map, cache.k, cache.v, rot.inv_freq, cache.page_size,
                                  cache.page_stride, cache.head_stride, pool_slots};
            qkv_.skinny(ctx, plans::EPI_QKV_ROPE, T, nullptr, &norm, qkv.p, q_width, &rope, nullptr, nullptr, nullptr, nullptr);
        } else {
            const Rows x = in.pending ? in.pending->materialize() : in.rows;
            qkv = qkv_(ctx, x);
            const int* slot_map = cache.writes ? tables.slot_map : nullptr;
            void* kc = cache.writes ? cache.k : nullptr;
            void* vc = cache.writes ? cache.v : nullptr;
            if (rotates && rot.rotary_dim == head_dim_ && head_dim_ % (dtype == DType::BF16 ? 16 : 8) == 0) {      // halves of a head in 16-byte pieces
                launch_check(eg_rope_cache_vec(ctx.stream, (int)dtype, qkv.p, (int)qkv.ld, rotation_table(ctx, rot), slot_map, kc, vc, T, heads_, kv_heads_,
                                               head_dim_, cache.page_size, cache.page_stride, cache.head_stride, slot_map ? pool_slots : 0, ctx.status),
                             "rope_cache_table");
            } else {
                if (!rotates && position) {
                    char* base = (char*)qkv.p;
                    position->apply_to_query_key(base, base + (size_t)q_width * dtype_size(dtype), qkv.ld, heads_, kv_heads_, head_dim_, ctx);
                }
                launch_check(eg_rope_cache(ctx.stream, (int)dtype, qkv.p, (int)qkv.ld, nullptr, ctx.positions, slot_map, kc, vc,
                                           rotates ? rot.inv_freq : nullptr, T, heads_, kv_heads_, head_dim_, rotates ? rot.rotary_dim : 0,
                                           cache.page_size, cache.page_stride, cache.head_stride, slot_map ? pool_slots : 0, ctx.status),
                             "rope_cache");
            }
        }
        (void)kv_width;
        Rows attn{ctx.take_rows(T, q_width, dtype), dtype, T, q_width, q_width};
        const long long longest = window_ < 0 ? ctx.max_context_len : std::min<long long>(ctx.max_context_len, window_ + 255);
        const int window = window_ < 0 ? 0 : (int)window_;
        if (ctx.query_tiles && plans::attention_prefill_takes(dtype, head_dim_, cache.page_size)) {
            // prompt portions: tiles of query tokens against the cache, on the tcgen05 tensor cores when the portions are
            // long enough to fill their 128-row tiles
            if (ctx.max_query_len >= plans::TCGEN05_ATTENTION_MIN_QUERY && plans::attention_prefill_tcgen05_takes(dtype, head_dim_, cache.page_size)) {
                int parts, part_tiles;
                plans::attention_prefill_parts(ctx.num_tiles, heads_, head_dim_, longest, &parts, &part_tiles);
                const size_t slots = (size_t)ctx.num_tiles * heads_;
                while (parts > 1 && slots * parts * 128 * (head_dim_ + 2) * 4 > plans::PREFILL_PARTS_SCRATCH_BYTES) --parts;
                float *partial_o = nullptr, *partial_ml = nullptr;
                if (parts > 1) {
                    partial_o = ctx.take<float>(slots * parts * 128 * head_dim_);
                    partial_ml = ctx.take<float>(slots * parts * 128 * 2);
                }
                launch_check(eg_attention_prefill_tcgen05(ctx.stream, qkv.p, qkv.ld, T, cache.k, cache.v, tables.block_table, tables.table_width,
                                                          ctx.positions, ctx.query_tiles, ctx.num_tiles, attn.p, attn.ld, heads_, kv_heads_, head_dim_,
                                                          cache.page_size, cache.page_stride, cache.head_stride, cache.num_pages, window, scale_,
                                                          ctx.status, nullptr, parts, part_tiles, partial_o, partial_ml,
                                                          ctx.scratch->prefill_queue.as<int>()), "attention_prefill_tcgen05");
            } else {
                launch_check(eg_attention_prefill(ctx.stream, qkv.p, (int)qkv.ld, cache.k, cache.v, tables.block_table, tables.table_width, ctx.positions,
                                                  ctx.query_tiles, ctx.num_tiles, attn.p, (int)attn.ld, heads_, kv_heads_, head_dim_, cache.page_size,
                                                  cache.page_stride, cache.head_stride, cache.num_pages, window, scale_, ctx.status), "attention_prefill");
            }
            if (ctx.small_tokens)      // the decoded tokens beside them: token by token, split over their keys
                paged(ctx, qkv, cache, tables, attn, ctx.num_small, plans::attention_paged_splits(ctx.num_small, heads_, kv_heads_, longest, head_dim_), window,
                      nullptr, ctx.small_tokens);
        } else if (plans::attention_paged_takes(dtype, head_dim_, cache.page_size)) {
            paged(ctx, qkv, cache, tables, attn, T, plans::attention_paged_splits(T, heads_, kv_heads_, longest, head_dim_), window, ctx.seq_context, nullptr);
        } else {
            launch_check(eg_attention_generic(ctx.stream, (int)dtype, qkv.p, (int)qkv.ld, cache.k, cache.v, tables.block_table, tables.table_width,
                                              ctx.token_seq, ctx.positions, attn.p, (int)attn.ld, T, heads_, kv_heads_, head_dim_, cache.page_size,
                                              cache.page_stride, cache.head_stride, cache.num_pages, window, scale_, ctx.status), "attention_generic");
        }
        Delta d;
        if (follow && out_.takes_following_norm(attn)) {
            d.pre = out_.with_following_norm(ctx, attn, *follow);
            return d;
        }
        const Rows o = out_(ctx, attn);
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    static const float* rotation_table(const StepContext& ctx, const HalfRotation& rot) { return step_rotation_table(ctx, rot); }
    void paged(const StepContext& ctx, const Rows& qkv, const CacheView& cache, const GroupTables& tables, const Rows& attn, int tokens, int splits,
               int window, const int* seq_context, const int* token_list) const {
        float *acc = nullptr, *ml = nullptr;
        int* counters = nullptr;
        if (splits > 1) {
            const size_t T = (size_t)ctx.num_tokens;
            acc = ctx.take<float>(T * heads_ * splits * head_dim_);
            ml = ctx.take<float>(T * heads_ * splits * 2);
            if ((size_t)tokens * kv_heads_ * ((heads_ / kv_heads_ + 15) / 16) > KernelScratch::ATTENTION_COUNTERS)
                throw DeviceError("a step has more (token, KV head) pairs than the attention's ticket counters");
            counters = ctx.scratch->attention_counters.as<int>();
        }
        launch_check(eg_attention_paged(ctx.stream, qkv.p, (int)qkv.ld, cache.k, cache.v, tables.block_table, tables.table_width, ctx.token_seq,
                                        ctx.positions, seq_context, attn.p, (int)attn.ld, acc, ml, tokens, heads_, kv_heads_, head_dim_, cache.page_size,
                                        cache.page_stride, cache.head_stride, cache.num_pages, window, scale_, splits, ctx.status, nullptr, 0, counters,
                                        plans::use_pdl(), nullptr, token_list), "attention_paged");
    }

    int hidden_, heads_, kv_heads_, head_dim_;
    bool qkv_bias_, out_bias_;
    long long window_;
    float scale_;
    Linear qkv_, out_;
};

// ---- SwiGLU feed-forward: down( up(x) * silu(gate(x)) ) (src/models/mlp.cpp:41-49).  gate and up become one product whose
// weight rows are interleaved (gate_0, up_0, gate_1, up_1, ...), so that every tile of the product holds both halves of the
// outputs it covers and the activation can run in the product's epilogue.  Parameters: hidden_size, intermediate_size, bias,
// gate_name / up_name / down_name (tensor-name suffixes, by default those of the reference) ---
class SwiGLU : public FeedForward {
public:
    SwiGLU(const Params& p, const std::string& prefix)
        : FeedForward(p, prefix), hidden_((int)p.integer("hidden_size")), inter_((int)p.integer("intermediate_size")), bias_(p.flag("bias", false)),
          gate_name_(prefix + p.text("gate_name", ".gate_proj.weight")), up_name_(prefix + p.text("up_name", ".up_proj.weight")),
          down_name_(prefix + p.text("down_name", ".down_proj.weight")), gate_bias_name_(prefix + p.text("gate_bias_name", ".gate_proj.bias")),
          up_bias_name_(prefix + p.text("up_bias_name", ".up_proj.bias")), down_bias_name_(prefix + p.text("down_bias_name", ".down_proj.bias")),
          clamped_(p.text("activation", "swiglu") == "clamped"), limit_((float)p.real("limit", 0.0)) {
        if (p.text("activation", "swiglu") != "swiglu" && !clamped_) throw std::invalid_argument("a gated feed-forward's activation is 'swiglu' or 'clamped'");
        if (clamped_ && !(limit_ > 0.f)) throw std::invalid_argument("a clamped gate needs a positive limit");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        std::vector<TensorRequest> r = {TensorRequest::matrix(gate_name_, inter_, hidden_), TensorRequest::matrix(up_name_, inter_, hidden_),
                                        TensorRequest::matrix(down_name_, hidden_, inter_)};
        if (bias_) {
            r.push_back(TensorRequest::vector(gate_bias_name_, inter_).with_init("zero"));
            r.push_back(TensorRequest::vector(up_bias_name_, inter_).with_init("zero"));
            r.push_back(TensorRequest::vector(down_bias_name_, hidden_).with_init("zero"));
        }
        return r;
    }
    void load(const HostTensors& file, DType dtype) override {
        const std::vector<float> gate = host_floats(need_tensor(file, gate_name_)), up = host_floats(need_tensor(file, up_name_));
        std::vector<float> w((size_t)2 * inter_ * hidden_), b;
        for (int i = 0; i < inter_; ++i) {
            std::memcpy(&w[(size_t)(2 * i) * hidden_], &gate[(size_t)i * hidden_], (size_t)hidden_ * 4);
            std::memcpy(&w[(size_t)(2 * i + 1) * hidden_], &up[(size_t)i * hidden_], (size_t)hidden_ * 4);
        }
        std::vector<float> db;
        if (bias_) {
            const std::vector<float> gb = host_floats(need_tensor(file, gate_bias_name_)), ub = host_floats(need_tensor(file, up_bias_name_));
            b.resize((size_t)2 * inter_);
            for (int i = 0; i < inter_; ++i) { b[2 * i] = gb[i]; b[2 * i + 1] = ub[i]; }
            db = host_floats(need_tensor(file, down_bias_name_));
        }
        gate_up_ = Linear(w.data(), 2 * inter_, hidden_, bias_ ? b.data() : nullptr, dtype);
        down_ = Linear(need_tensor(file, down_name_), bias_ ? db.data() : nullptr, dtype);
    }
    size_t weight_bytes() const override { return gate_up_.weight_bytes() + down_.weight_bytes(); }
    bool capturable() const override { return true; }
    bool accepts_pending_norm() const override { return !clamped_; }
    bool fuses_following_norm() const override { return !clamped_; }

    // norm + gate/up + SwiGLU; down projection into the residual
    bool emit_fused(FusedBuilder& b, const float* gain, float eps) const override {
        if (b.ctx->dtype != DType::BF16 || hidden_ != b.hidden || inter_ % 8 || clamped_) return false;
        void* act = b.arena->take((size_t)b.tokens * inter_ * 2);
        EgFusedTemplate t = FusedBuilder::blank();
        t.input = EGF_IN_NORM;
        t.output = EGF_OUT_SWIGLU;
        t.N = 2 * inter_;
        t.K = hidden_;
        t.tiles_per_unit = 1;
        t.group_rows = 8;
        t.units_per_group = 1;
        t.warp_units = hidden_ <= EGF_STAGE_COLS;
        t.eps = eps;
        t.out = act;
        t.ldo = inter_;
        if (!b.linear(t, gate_up_.weight, hidden_, gate_up_.bias_f32(), gain)) return false;
        EgFusedTemplate d = FusedBuilder::blank();
        d.input = EGF_IN_ROWS;
        d.output = EGF_OUT_RESIDUAL;
        d.N = hidden_;
        d.K = inter_;
        d.tiles_per_unit = 1;
        d.group_rows = 8;
        d.units_per_group = 1;
        d.x = act;
        d.ldx = inter_;
        return b.linear(d, down_.weight, inter_, down_.bias_f32(), nullptr);
    }

    Delta forward(const StepContext& ctx, PartInput in, const FollowingNorm* follow) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        Rows act{ctx.take_rows(T, inter_, dtype), dtype, T, inter_, inter_};
        if (clamped_) {
            // g = min(gate, limit), u = clamp(up, -limit, limit): a = g sigmoid(1.702 g) (u + 1)
            const Rows x = in.pending ? in.pending->materialize() : in.rows;
            if (plans::gemm_skinny_takes(dtype, T, hidden_) && Linear::aligned(x)) {
                act = gate_up_.skinny_clamped_glu(ctx, x, limit_);
            } else if (plans::gemm_tcgen05_wide_takes(dtype, T, 2 * inter_, hidden_) && Linear::aligned(x)) {
                launch_check(eg_gemm_tcgen05_pair_glu_bias(ctx.stream, x.p, x.ld, gate_up_.weight, hidden_, gate_up_.bias_f32(), act.p, inter_, T, 2 * inter_,
                                                           hidden_, ctx.status, limit_), "gemm_tcgen05_pair_glu");
            } else {
                // the bare product in float32; biases, limits and the gate in one kernel behind it
                const Rows gu = gate_up_.without_bias_f32(ctx, x);
                launch_check(eg_clamped_glu_bias(ctx.stream, gu.p, (int)gu.dtype, gu.ld, gate_up_.bias_f32(), act.p, (int)dtype, inter_, T, inter_, limit_),
                             "clamped_glu");
            }
            Delta d;
            const Rows o = down_.f32_bias_pending(ctx, act, &d.bias);
            d.p = o.p;
            d.dtype = o.dtype;
            return d;
        }
        if (in.pending && in.pending->fusable) {
            // decode: add + norm + gate/up product + SwiGLU in one kernel
            const NormInFront norm = in.pending->fused();
            gate_up_.skinny(ctx, plans::EPI_SWIGLU, T, nullptr, &norm, act.p, inter_, nullptr, nullptr, nullptr, nullptr, nullptr);
        } else {
            const Rows x = in.pending ? in.pending->materialize() : in.rows;
            if (plans::gemm_skinny_takes(dtype, T, hidden_) && Linear::aligned(x)) {
                gate_up_.skinny(ctx, plans::EPI_SWIGLU, T, &x, nullptr, act.p, inter_, nullptr, nullptr, nullptr, nullptr, nullptr);
            } else if (plans::gemm_tcgen05_wide_takes(dtype, T, 2 * inter_, hidden_) && Linear::aligned(x)) {
                // prompts: the product on the tcgen05 tensor cores (CTA pairs, 256 x 256 tiles) with SwiGLU in its epilogue
                launch_check(eg_gemm_tcgen05_pair(ctx.stream, plans::EPI_SWIGLU, x.p, x.ld, gate_up_.weight, hidden_, gate_up_.bias_f32(), act.p, inter_, T,
                                                  2 * inter_, hidden_, 256, ctx.status, nullptr), "gemm_tcgen05_pair");
            } else {
                const Rows gu = gate_up_(ctx, x);
                launch_check(eg_swiglu(ctx.stream, (int)dtype, gu.p, (int)gu.ld, act.p, inter_, T, inter_), "swiglu");
            }
        }
        Delta d;
        if (follow && down_.takes_following_norm(act)) {
            d.pre = down_.with_following_norm(ctx, act, *follow);
            return d;
        }
        const Rows o = down_(ctx, act);
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    int hidden_, inter_;
    bool bias_;
    std::string gate_name_, up_name_, down_name_;      // the weights' tensor names (parameters gate_name / up_name / down_name: suffixes of the prefix)
    std::string gate_bias_name_, up_bias_name_, down_bias_name_;    // with bias: the biases' names (parameters *_bias_name, suffixes alike)
    bool clamped_;                                     // parameter activation "clamped" (with limit) instead of "swiglu"
    float limit_;
    Linear gate_up_, down_;
};

// ---- token embedding: residual[t] = E[id[t]] (src/models/embedding.cpp:54-76) ---------------------------------------
class TokenEmbedding : public Embedding {
public:
    TokenEmbedding(const Params& p, const std::string& prefix)
        : Embedding(p, prefix), vocab_((int)p.integer("vocab_size")), hidden_((int)p.integer("hidden_size")), weight_name_(prefix + p.text("weight_name", ".weight")),
          scale_(p.has("scale") ? (float)p.real("scale") : 1.0f) {}
    std::vector<TensorRequest> tensor_requests() const override { return {TensorRequest::matrix(weight_name_, vocab_, hidden_)}; }
    void load(const HostTensors& file, DType dtype) override {
        table_ = upload(need_tensor(file, weight_name_), dtype);
        dtype_ = dtype;
    }
    bool capturable() const override { return true; }
    void forward(const StepContext& ctx, float* residual) override {
        if (scale_ != 1.0f) {       // residual[t] = scale * E[id[t]]
            launch_check(eg_embedding_gather_scaled(ctx.stream, (int)dtype_, ctx.token_ids, table_.get(), residual, ctx.num_tokens, hidden_, vocab_, scale_,
                                                    ctx.status), "embedding_gather_scaled");
            return;
        }
        launch_check(eg_embedding_gather(ctx.stream, (int)dtype_, ctx.token_ids, table_.get(), residual, ctx.num_tokens, hidden_, vocab_, ctx.status),
                     "embedding_gather");
    }
    const void* table() const override { return table_.get(); }
    bool fused_gather(const void** table, int* vocab) const override {
        if (dtype_ != DType::BF16 || hidden_ % 4 || scale_ != 1.0f) return false;
        *table = table_.get();
        *vocab = vocab_;
        return true;
    }

private:
    int vocab_, hidden_;
    std::string weight_name_;
    float scale_;                   // parameter scale: a factor on every embedding row (default 1)
    DType dtype_ = DType::BF16;
    DeviceBuffer table_;
};

// ---- output head: logits = x E^T when tied (the reference always is, src/models/gpt_model.cpp:324-328,
// src/models/embedding.cpp:78-81) or x W_head^T with lm_head.weight when not.  Logits are float32 in both precisions.
// Parameters: vocab_size, hidden_size, tied_to (prefix of the embedding, or absent), weight_name (suffix, default
// ".weight"), softcap (c > 0: logits <- c tanh(logits / c)) -------------------------------------
class LMHead : public Head {
public:
    LMHead(const Params& p, const std::string& prefix)
        : Head(p, prefix), vocab_((int)p.integer("vocab_size")), hidden_((int)p.integer("hidden_size")), tied_(p.has("tied_to")),
          softcap_(p.has("softcap") ? (float)p.real("softcap") : 0.f), scale_(p.has("scale") ? (float)p.real("scale") : 1.0f),
          weight_name_(prefix + p.text("weight_name", ".weight")) {
        if (softcap_ < 0.f) throw std::invalid_argument("softcap must be positive");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        if (tied_) return {};
        return {TensorRequest::matrix(weight_name_, vocab_, hidden_)};
    }
    void load_head(const HostTensors& file, DType dtype, const void* tied_table) override {
        if (tied_) linear_ = Linear::sharing(tied_table, vocab_, hidden_, dtype);
        else linear_ = Linear(need_tensor(file, weight_name_), nullptr, dtype);
    }
    size_t weight_bytes() const override { return linear_.weight_bytes(); }
    bool capturable() const override { return true; }
    int vocab() const override { return vocab_; }
    bool emit_fused(FusedBuilder& b, const float* gain, float eps) const override {
        if (b.ctx->dtype != DType::BF16 || hidden_ != b.hidden || linear_.has_bias() || softcap_ > 0.f || scale_ != 1.0f) return false;
        b.logits = b.arena->take_n<float>((size_t)b.tokens * vocab_);
        EgFusedTemplate t = FusedBuilder::blank();
        t.input = EGF_IN_NORM;
        t.output = EGF_OUT_F32;
        t.N = vocab_;
        t.K = hidden_;
        t.tiles_per_unit = 1;
        t.group_rows = 8;
        t.units_per_group = 1;
        t.warp_units = hidden_ <= EGF_STAGE_COLS;
        t.eps = eps;
        t.out = b.logits;
        t.ldo = vocab_;
        return b.linear(t, linear_.weight, hidden_, nullptr, gain);
    }
    float* forward(const StepContext& ctx, PartInput in, int rows) override {
        // Thousands of CTAs share the head's rows, and each would repeat the add + norm of the few tokens in front of its
        // product: the norm runs once, in a kernel of its own.
        Rows x = in.pending ? in.pending->materialize() : in.rows;
        x.rows = rows;
        float* logits = (float*)linear_(ctx, x, /*out_f32=*/true).p;
        if (scale_ != 1.0f) launch_check(eg_scale_f32(ctx.stream, logits, (long long)rows * vocab_, scale_), "scale");
        // logits <- cap * tanh(logits / cap), where the model has such a cap
        if (softcap_ > 0.f) launch_check(eg_softcap(ctx.stream, logits, (long long)rows * vocab_, softcap_), "softcap");
        return logits;
    }

private:
    int vocab_, hidden_;
    bool tied_;
    float softcap_, scale_;         // parameter scale: logits <- scale * logits (before a soft cap), default 1
    std::string weight_name_;
    Linear linear_;
};

inline void register_builtin_parts() {
    PartRegistry& r = PartRegistry::instance();
    if (r.mixers.count("attention")) return;
    r.mixers["attention"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<Attention>(p, prefix, std::move(pos));
    };
    r.feed_forwards["swiglu"] = [](const Params& p, const std::string& prefix) { return std::make_shared<SwiGLU>(p, prefix); };
    r.norms["rmsnorm"] = [](const Params& p, const std::string& prefix) { return std::make_shared<RMSNorm>(p, prefix); };
    r.norms["layernorm"] = [](const Params& p, const std::string& prefix) { return std::make_shared<LayerNorm>(p, prefix); };
    r.stream_adds["pass_offsets"] = [](const Params& p, const std::string& prefix) { return std::make_shared<PassOffsets>(p, prefix); };
    r.positions["rope"] = [](const Params& p, const std::string& prefix) { return std::make_shared<RotaryEncoding>(p, prefix); };
    r.embeddings["embedding"] = [](const Params& p, const std::string& prefix) { return std::make_shared<TokenEmbedding>(p, prefix); };
    r.heads["lm_head"] = [](const Params& p, const std::string& prefix) { return std::make_shared<LMHead>(p, prefix); };
}

}  // namespace easygpt::engine
