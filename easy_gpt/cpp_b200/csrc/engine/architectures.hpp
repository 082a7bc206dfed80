// Architectures: the registry from an architecture's name to its model, and the one architecture the engine
// ships, the Qwen2 / Qwen2.5 dense decoder.
//
// The lookup rule is the reference's (src/models/layer_key_prefix.cpp:24-28, 92-105): lower-case
// architectures[0] and model_type; an entry matches if its key occurs in the architecture string or equals the
// model type; no match raises an error naming both strings.  (A configuration may also give the name as one string
// under "architecture".)  An entry turns the config.json object into a
// ModelSpec; loader, cache manager, step function, scheduler and replay need nothing else.
#pragma once
#include <algorithm>
#include <cctype>
#include <functional>
#include <map>

#include "json.hpp"
#include "spec.hpp"

namespace easygpt::engine {

struct ConfigError : std::invalid_argument {
    using std::invalid_argument::invalid_argument;
};

struct ArchitectureRegistry {
    using Builder = std::function<ModelSpec(const json::Value&)>;
    std::vector<std::pair<std::string, Builder>> entries;      // in the order of registration
    static ArchitectureRegistry& instance() {
        static ArchitectureRegistry r;
        return r;
    }
    void add(std::string key, Builder b) {
        std::transform(key.begin(), key.end(), key.begin(), [](unsigned char c) { return (char)std::tolower(c); });
        for (auto& e : entries)
            if (e.first == key) { e.second = std::move(b); return; }
        entries.emplace_back(std::move(key), std::move(b));
    }
    ModelSpec build(const json::Value& config) const {
        std::string arch, model_type;
        if (const json::Value* a = config.find("architectures"))
            if (a->is_array() && !a->array.empty() && a->array[0].is_string()) arch = a->array[0].string;
        if (arch.empty())                                       // some configurations name it in one string
            if (const json::Value* a = config.find("architecture"))
                if (a->is_string()) arch = a->string;
        if (const json::Value* m = config.find("model_type"))
            if (m->is_string()) model_type = m->string;
        auto lower = [](std::string s) {
            std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return (char)std::tolower(c); });
            return s;
        };
        const std::string la = lower(arch), lm = lower(model_type);
        for (auto& e : entries)
            if (la.find(e.first) != std::string::npos || lm == e.first) {
                ModelSpec spec = e.second(config);
                spec.validate();
                return spec;
            }
        throw std::invalid_argument("Unsupported model architecture/model_type: architecture='" + arch + "', model_type='" + model_type + "'");
    }
};

// ---- Qwen2 / Qwen2.5 -------------------------------------------------------------------------------------------------
// Typed configuration read from the keys of its own config.json.  The reference reads eleven keys
// (src/config.cpp:16-31) and takes the rest from the shapes of the weights or from constants in its code (eps 1e-6 at
// src/models/norm.cpp:41, head size at src/models/self_attn.cpp:169-174, intermediate size at
// src/models/model_param_validation.cpp:167-194).  Here every one of those is a key with the default the reference's
// constant implies.
struct Qwen2Config {
    long long vocab_size, hidden_size, intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads, head_dim,
        max_position_embeddings, max_window_layers, sliding_window = -1, bos_token_id = -1, eos_token_id = -1;
    double rope_theta, rms_norm_eps;
    bool tie_word_embeddings, attention_bias, attention_out_bias, mlp_bias, use_sliding_window;
    std::string hidden_act, architecture, model_type;

    static long long integer(const json::Value& d, const std::string& key) {
        const json::Value* v = d.find(key);
        if (!v || !v->is_number() || !v->is_integer) throw ConfigError(key + " must be an integer");
        return v->integer;
    }
    static bool boolean(const json::Value& d, const std::string& key, bool fallback) {
        const json::Value* v = d.find(key);
        if (!v || v->is_null()) return fallback;
        if (v->is_bool()) return v->boolean;
        if (v->is_number()) return v->number != 0;
        throw ConfigError(key + " must be true or false");
    }
    static Qwen2Config from_json(const json::Value& d) {
        if (!d.is_object()) throw ConfigError("config.json is not a JSON object");
        std::string missing;
        for (const char* k : {"vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                              "rope_theta", "max_position_embeddings"}) {
            const json::Value* v = d.find(k);
            if (!v || v->is_null()) missing += (missing.empty() ? "" : ", ") + std::string(k);
        }
        if (!missing.empty()) throw ConfigError("config.json lacks: " + missing);
        Qwen2Config c;
        c.num_attention_heads = integer(d, "num_attention_heads");
        c.hidden_size = integer(d, "hidden_size");
        if (c.num_attention_heads <= 0 || c.hidden_size <= 0) throw ConfigError("hidden_size and num_attention_heads must be > 0");
        const json::Value* hd = d.find("head_dim");
        if (hd && !hd->is_null()) c.head_dim = integer(d, "head_dim");
        else {
            if (c.hidden_size % c.num_attention_heads)      // src/models/model_param_validation.cpp:94-97
                throw ConfigError("hidden_size must be divisible by num_attention_heads when head_dim is not given");
            c.head_dim = c.hidden_size / c.num_attention_heads;
        }
        c.vocab_size = integer(d, "vocab_size");
        c.intermediate_size = integer(d, "intermediate_size");
        c.num_hidden_layers = integer(d, "num_hidden_layers");
        c.num_key_value_heads = integer(d, "num_key_value_heads");
        c.max_position_embeddings = integer(d, "max_position_embeddings");
        const json::Value* theta = d.find("rope_theta");
        if (!theta->is_number()) throw ConfigError("rope_theta must be a number");
        c.rope_theta = theta->number;
        const json::Value* eps = d.find("rms_norm_eps");
        c.rms_norm_eps = (eps && eps->is_number()) ? eps->number : 1e-6;
        c.tie_word_embeddings = boolean(d, "tie_word_embeddings", false);
        c.attention_bias = boolean(d, "attention_bias", true);
        c.attention_out_bias = boolean(d, "attention_out_bias", false);
        c.mlp_bias = boolean(d, "mlp_bias", false);
        const json::Value* act = d.find("hidden_act");
        c.hidden_act = (act && act->is_string()) ? act->string : "silu";
        c.use_sliding_window = boolean(d, "use_sliding_window", false);
        const json::Value* sw = d.find("sliding_window");
        bool window_ok = false;
        if (sw && sw->is_number() && sw->is_integer && sw->integer > 0) { c.sliding_window = sw->integer; window_ok = true; }
        const json::Value* mwl = d.find("max_window_layers");
        c.max_window_layers = (mwl && !mwl->is_null()) ? integer(d, "max_window_layers") : c.num_hidden_layers;
        const json::Value* bos = d.find("bos_token_id");
        c.bos_token_id = (bos && !bos->is_null()) ? integer(d, "bos_token_id") : -1;
        const json::Value* eos = d.find("eos_token_id");
        if (eos && eos->is_array()) c.eos_token_id = (!eos->array.empty() && eos->array[0].is_integer) ? eos->array[0].integer : -1;
        else c.eos_token_id = (eos && !eos->is_null()) ? integer(d, "eos_token_id") : -1;
        if (const json::Value* a = d.find("architectures"))
            if (a->is_array() && !a->array.empty() && a->array[0].is_string()) c.architecture = a->array[0].string;      // src/config.cpp:26-31
        if (const json::Value* m = d.find("model_type"))
            if (m->is_string()) c.model_type = m->string;
        // what cannot run is refused
        auto positive = [](long long v, const char* key) {
            if (v <= 0) throw ConfigError(std::string(key) + " must be > 0, got " + std::to_string(v));
        };
        positive(c.vocab_size, "vocab_size");
        positive(c.intermediate_size, "intermediate_size");
        positive(c.num_hidden_layers, "num_hidden_layers");
        positive(c.num_key_value_heads, "num_key_value_heads");
        positive(c.head_dim, "head_dim");
        positive(c.max_position_embeddings, "max_position_embeddings");
        if (c.num_attention_heads % c.num_key_value_heads)       // src/cuda/ops/self_attn.cu:216-218
            throw ConfigError("num_attention_heads (" + std::to_string(c.num_attention_heads) + ") must be a multiple of num_key_value_heads (" +
                              std::to_string(c.num_key_value_heads) + ")");
        if (c.head_dim % 2) throw ConfigError("head_dim must be even for the half rotation");       // src/ops.cpp:155-157
        if (c.rope_theta <= 0.0) throw ConfigError("rope_theta must be > 0");                        // src/ops.cpp:158-160
        if (c.rms_norm_eps <= 0.0) throw ConfigError("rms_norm_eps must be > 0");
        if (c.hidden_act != "silu") throw ConfigError("hidden_act '" + c.hidden_act + "' is not supported (silu only)");
        if (const json::Value* rs = d.find("rope_scaling"))
            if (!rs->is_null() && !(rs->is_object() && rs->object.empty())) throw ConfigError("rope_scaling is not supported");
        if (c.use_sliding_window) {
            if (!window_ok) throw ConfigError("use_sliding_window needs a positive integer sliding_window");
            if (c.max_window_layers < 0) throw ConfigError("max_window_layers must be >= 0");
        }
        return c;
    }
    // layers from max_window_layers on see only the last sliding_window positions when use_sliding_window is set
    long long layer_window(long long layer) const { return (use_sliding_window && layer >= max_window_layers) ? sliding_window : -1; }
};

// Tensor names are the reference's (src/models/layer_key_prefix.cpp:77-87, src/models/embedding.cpp:30) plus
// lm_head.weight for an untied head, which the reference never consumes (src/models/gpt_model.cpp:324-328).
inline ModelSpec qwen2_spec(const json::Value& config) {
    const Qwen2Config c = Qwen2Config::from_json(config);
    ModelSpec spec;
    spec.architecture = "qwen2";
    spec.vocab_size = c.vocab_size;
    spec.hidden_size = c.hidden_size;
    spec.max_positions = c.max_position_embeddings;
    spec.bos_token_id = c.bos_token_id;
    spec.eos_token_id = c.eos_token_id;
    auto norm = [&](const std::string& prefix) { return PartSpec{"rmsnorm", Params{{"size", c.hidden_size}, {"eps", c.rms_norm_eps}}, prefix, true}; };
    for (long long i = 0; i < c.num_hidden_layers; ++i) {
        const std::string prefix = "model.layers." + std::to_string(i);
        Params attention{{"hidden_size", c.hidden_size}, {"num_heads", c.num_attention_heads}, {"num_kv_heads", c.num_key_value_heads},
                         {"head_dim", c.head_dim}, {"qkv_bias", c.attention_bias}, {"out_bias", c.attention_out_bias}};
        if (c.layer_window(i) > 0) attention.set("window", c.layer_window(i));
        spec.layers.push_back(LayerSpec::pre_norm(
            PartSpec{"attention", attention, prefix + ".self_attn", true},
            PartSpec{"swiglu", Params{{"hidden_size", c.hidden_size}, {"intermediate_size", c.intermediate_size}, {"bias", c.mlp_bias}}, prefix + ".mlp", true},
            norm(prefix + ".input_layernorm"), norm(prefix + ".post_attention_layernorm"),
            PartSpec{"rope", Params{{"head_dim", c.head_dim}, {"rotary_dim", c.head_dim}, {"theta", c.rope_theta}}, "", true}));
        spec.run_order.push_back(RunEntry{(int)i, (int)i, true});
    }
    spec.embedding = PartSpec{"embedding", Params{{"vocab_size", c.vocab_size}, {"hidden_size", c.hidden_size}}, "model.embed_tokens", true};
    spec.final_norm = norm("model.norm");
    Params head{{"vocab_size", c.vocab_size}, {"hidden_size", c.hidden_size}};
    if (c.tie_word_embeddings) head.set("tied_to", "model.embed_tokens");
    spec.lm_head = PartSpec{"lm_head", head, "lm_head", true};
    return spec;
}

// ---- Gufanex ---------------------------------------------------------------------------------------------------------------
// A decoder whose config.json lists its layers one by one: each has a mixer of its own kind and sizes ("mamba1": a
// selective state-space mixer; "latent_attention": attention through a cached latent) and a routed feed-forward or none;
// mixer and feed-forward read the same stream through two layer norms, x = x + (mixer(norm1(x)) + ff(norm2(x))).  A run
// of layers ("loop": start, stop, times) is passed through several times with the same weights and a cache or state of
// its own per pass; before every pass a learned vector of that pass is added to the stream, and before every pass but
// the first also the stream as the embedding left it.  The output is a layer norm, the head, and a soft cap
// c * tanh(logits / c).  Every size and constant is a key of config.json; tensor names are "l<i>.<part>.<tensor>".
struct GufanexConfig {
    static const json::Value& need(const json::Value& d, const std::string& key, const std::string& where) {
        const json::Value* v = d.is_object() ? d.find(key) : nullptr;
        if (!v || v->is_null()) throw ConfigError("config.json lacks " + where + key);
        return *v;
    }
    static long long integer(const json::Value& d, const std::string& key, const std::string& where) {
        const json::Value& v = need(d, key, where);
        if (!v.is_number() || !v.is_integer) throw ConfigError(where + key + " must be an integer");
        return v.integer;
    }
    static long long integer_or(const json::Value& d, const std::string& key, long long fallback, const std::string& where) {
        const json::Value* v = d.is_object() ? d.find(key) : nullptr;
        return (!v || v->is_null()) ? fallback : integer(d, key, where);
    }
    static double number(const json::Value& d, const std::string& key, const std::string& where) {
        const json::Value& v = need(d, key, where);
        if (!v.is_number()) throw ConfigError(where + key + " must be a number");
        return v.number;
    }
    static bool present(const json::Value& d, const std::string& key) {
        const json::Value* v = d.is_object() ? d.find(key) : nullptr;
        return v && !v->is_null();
    }
};

inline ModelSpec gufanex_spec(const json::Value& config) {
    using C = GufanexConfig;
    if (!config.is_object()) throw ConfigError("config.json is not a JSON object");
    ModelSpec spec;
    spec.architecture = "gufanex";
    const long long width = C::integer(config, "width", ""), vocab = C::integer(config, "vocab", "");
    if (width <= 0 || vocab <= 0) throw ConfigError("width and vocab must be > 0");
    const double eps = C::number(C::need(config, "norm", ""), "eps", "norm.");
    if (eps <= 0.0) throw ConfigError("norm.eps must be > 0");
    spec.vocab_size = vocab;
    spec.hidden_size = width;
    spec.max_positions = C::integer_or(config, "max_positions", 1LL << 30, "");     // the design sets no limit; positions are 32-bit
    auto layer_norm = [&](const std::string& prefix) {
        return PartSpec{"layernorm", Params{{"size", width}, {"eps", eps}, {"weight_name", ""}, {"bias_name", ".b"}}, prefix, true};
    };
    const json::Value& layers = C::need(config, "layers", "");
    if (!layers.is_array() || layers.array.empty()) throw ConfigError("layers must be a list with at least one layer");
    for (size_t i = 0; i < layers.array.size(); ++i) {
        const json::Value& l = layers.array[i];
        const std::string where = "layers[" + std::to_string(i) + "].", prefix = "l" + std::to_string(i);
        const json::Value& type = C::need(l, "type", where);
        const json::Value& m = C::need(l, "mixer", where);
        if (!type.is_string()) throw ConfigError(where + "type must be a string");
        PartSpec mixer;
        if (type.string == "mamba1") {
            const std::string w = where + "mixer.";
            mixer = PartSpec{"selective_scan", Params{{"hidden_size", width}, {"inner", C::integer(m, "inner", w)}, {"state", C::integer(m, "state", w)},
                                                      {"dt_rank", C::integer(m, "dt_rank", w)}, {"conv", C::integer(m, "conv", w)}}, prefix + ".mix", true};
        } else if (type.string == "latent_attention") {
            const std::string w = where + "mixer.";
            const json::Value& rot = C::need(m, "rot", w);
            mixer = PartSpec{"latent_attention", Params{{"hidden_size", width}, {"heads", C::integer(m, "heads", w)}, {"dim", C::integer(m, "dim", w)},
                                                        {"rot_dim", C::integer(m, "rot_dim", w)}, {"vdim", C::integer(m, "vdim", w)},
                                                        {"kv_rank", C::integer(m, "kv_rank", w)}, {"q_rank", C::integer(m, "q_rank", w)},
                                                        {"scale", C::number(m, "scale", w)}, {"rot_base", C::number(rot, "base", w + "rot.")},
                                                        {"rot_dims", C::integer(rot, "dims", w + "rot.")}, {"eps", eps}, {"sink", true}}, prefix + ".mix", true};
        } else {
            throw ConfigError(where + "type '" + type.string + "' is no mixer of this design (mamba1, latent_attention)");
        }
        LayerSpec layer;
        layer.parallel = true;
        layer.sublayers.push_back({"mixer", mixer, layer_norm(prefix + ".norm1"), "pre", PartSpec::none()});
        if (C::present(l, "mlp")) {
            const json::Value& mlp = *l.find("mlp");
            const std::string w = where + "mlp.";
            const json::Value& kind = C::need(mlp, "kind", w);
            if (!kind.is_string() || kind.string != "moe") throw ConfigError(w + "kind must be 'moe'");
            const json::Value& router = C::need(mlp, "router", w);
            const long long experts = C::integer(router, "experts", w + "router."), identity = C::integer_or(router, "identity", 0, w + "router.");
            Params ff{{"hidden_size", width}, {"experts", experts}, {"identity", identity}, {"top", C::integer(router, "top", w + "router.")},
                      {"ff", experts > 0 ? C::integer(C::need(mlp, "expert", w), "ff", w + "expert.") : 0LL},
                      {"shared_ff", C::present(mlp, "shared") ? C::integer(*mlp.find("shared"), "ff", w + "shared.") : 0LL}};
            layer.sublayers.push_back({"feed_forward", PartSpec{"routed_experts", ff, prefix + ".mlp", true}, layer_norm(prefix + ".norm2"), "pre", PartSpec::none()});
        }
        spec.layers.push_back(std::move(layer));
    }
    // the run order: the layers in front of the loop, the loop's layers `times` times (a cache or state per pass), the rest
    const long long n = (long long)spec.layers.size();
    long long start = n, stop = n, times = 1;
    if (C::present(config, "loop")) {
        const json::Value& loop = *config.find("loop");
        start = C::integer(loop, "start", "loop.");
        stop = C::integer(loop, "stop", "loop.");
        times = C::integer(loop, "times", "loop.");
        if (start < 0 || stop < start || stop > n || times < 1) throw ConfigError("loop must have 0 <= start <= stop <= layers and times >= 1");
        if (stop > start) spec.stream_adds.push_back(PartSpec{"pass_offsets", Params{{"rows", times}, {"hidden_size", width}}, "loop.step", true});
    }
    int cache = 0;
    auto run = [&](long long layer) { spec.run_order.push_back(RunEntry{(int)layer, cache++, true}); };
    for (long long i = 0; i < std::min(start, n); ++i) run(i);
    if (stop > start)
        for (long long t = 0; t < times; ++t)
            for (long long i = start; i < stop; ++i) {
                run(i);
                if (i == start) {
                    RunEntry& e = spec.run_order.back();
                    e.stream_add = 0;
                    e.stream_add_row = (int)t;
                    e.add_embedding = t > 0;
                }
            }
    for (long long i = stop; i < n; ++i) run(i);
    spec.embedding = PartSpec{"embedding", Params{{"vocab_size", vocab}, {"hidden_size", width}, {"weight_name", ""}}, "embed", true};
    spec.final_norm = layer_norm("final.norm");
    Params head{{"vocab_size", vocab}, {"hidden_size", width}, {"weight_name", ""}};
    if (C::present(config, "logit_softcap")) {
        const double cap = C::number(config, "logit_softcap", "");
        if (cap < 0.0) throw ConfigError("logit_softcap must be positive");
        if (cap > 0.0) head.set("softcap", cap);
    }
    spec.lm_head = PartSpec{"lm_head", head, "head", true};
    return spec;
}

// ---- Lasizen ---------------------------------------------------------------------------------------------------------------
// A decoder whose config.json lists its layers one by one ("type": "attention", attention over a sliding window with a
// sink, or "delta", a gated delta-rule mixer; "mlp": a dense feed-forward, or null).  Both branches of a layer are normed
// on both sides, x = x + norm1b(mixer(shift(norm1(x)))), x = x + norm2b(ff(norm2(x))), all RMS norms; in front of the mixer
// every token's normed row is mixed with that of the token in front of it (a learned weight per channel).  A run of
// layers ("loop": start, stop, times) is passed through several times in a row with the same weights and a cache or state
// of its own per pass.  The embedding is scaled by embedding.scale, the logits by logit_scale.  Every size and constant is
// a key of config.json; tensor names are "l<i>.<part>.<tensor>".
inline ModelSpec lasizen_spec(const json::Value& config) {
    using C = GufanexConfig;        // the typed readers (a key's path goes into the refusal)
    if (!config.is_object()) throw ConfigError("config.json is not a JSON object");
    ModelSpec spec;
    spec.architecture = "lasizen";
    const long long width = C::integer(config, "width", ""), vocab = C::integer(config, "vocab", "");
    if (width <= 0 || vocab <= 0) throw ConfigError("width and vocab must be > 0");
    const double eps = C::number(C::need(config, "norm", ""), "eps", "norm.");
    if (eps <= 0.0) throw ConfigError("norm.eps must be > 0");
    spec.vocab_size = vocab;
    spec.hidden_size = width;
    spec.max_positions = C::integer_or(config, "max_positions", 1LL << 30, "");     // the design sets no limit; positions are 32-bit
    auto norm = [&](const std::string& name) { return PartSpec{"rmsnorm", Params{{"size", width}, {"eps", eps}, {"weight_name", ""}}, name, true}; };
    const json::Value& layers = C::need(config, "layers", "");
    if (!layers.is_array() || layers.array.empty()) throw ConfigError("layers must be a list with at least one layer");
    for (size_t i = 0; i < layers.array.size(); ++i) {
        const json::Value& l = layers.array[i];
        const std::string where = "layers[" + std::to_string(i) + "].", prefix = "l" + std::to_string(i), w = where + "mixer.";
        const json::Value& type = C::need(l, "type", where);
        const json::Value& m = C::need(l, "mixer", where);
        if (!type.is_string()) throw ConfigError(where + "type must be a string");
        LayerSpec layer;
        PartSpec mixer;
        const long long heads = C::integer(m, "heads", w), kv_heads = C::integer(m, "kv_heads", w), dim = C::integer(m, "dim", w), vdim = C::integer(m, "vdim", w);
        if (heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || heads % kv_heads)
            throw ConfigError(w + "heads, kv_heads, dim and vdim must be > 0, heads a multiple of kv_heads");
        if (type.string == "attention") {
            Params a{{"hidden_size", width}, {"heads", heads}, {"kv_heads", kv_heads}, {"dim", dim}, {"vdim", vdim}, {"scale", C::number(m, "scale", w)},
                     {"sink_logit", 0.0}, {"unit_eps", eps}};
            if (C::present(m, "mask")) {
                const long long size = C::integer(*m.find("mask"), "size", w + "mask.");
                if (size <= 0) throw ConfigError(w + "mask.size must be > 0");
                a.set("window", size);
            }
            mixer = PartSpec{"sink_attention", a, prefix + ".mix", true};
            if (C::present(m, "rot")) {
                const json::Value& rot = *m.find("rot");
                const long long dims = C::integer(rot, "dims", w + "rot.");
                if (dims < 0 || dims % 2 || dims > dim) throw ConfigError(w + "rot.dims must be even and within dim");
                if (dims > 0) {
                    Params r{{"head_dim", dim}, {"rotary_dim", dims}, {"theta", C::number(rot, "base", w + "rot.")}};
                    if (C::present(rot, "scaling")) {
                        const json::Value& sc = *rot.find("scaling");
                        const std::string ws = w + "rot.scaling.";
                        r.set("scaling_factor", C::number(sc, "factor", ws));
                        r.set("scaling_original", C::number(sc, "original", ws));
                        r.set("scaling_fast", C::number(sc, "fast", ws));
                        r.set("scaling_slow", C::number(sc, "slow", ws));
                    }
                    layer.position = PartSpec{"rope", r, "", true};
                }
            }
        } else if (type.string == "delta") {
            mixer = PartSpec{"gated_delta", Params{{"hidden_size", width}, {"heads", heads}, {"kv_heads", kv_heads}, {"dim", dim}, {"vdim", vdim},
                                                   {"conv", C::integer(m, "conv", w)}, {"eps", eps}, {"unit_eps", 1e-6}}, prefix + ".mix", true};
        } else {
            throw ConfigError(where + "type '" + type.string + "' is no mixer of this design (attention, delta)");
        }
        SubLayerSpec mix{"mixer", mixer, norm(prefix + ".norm1"), "pre", norm(prefix + ".norm1b")};
        mix.shift = PartSpec{"token_shift", Params{{"size", width}}, prefix + ".shift", true};
        layer.sublayers.push_back(std::move(mix));
        if (C::present(l, "mlp")) {
            const json::Value& mlp = *l.find("mlp");
            const std::string wm = where + "mlp.";
            const json::Value& kind = C::need(mlp, "kind", wm);
            if (!kind.is_string() || kind.string != "dense") throw ConfigError(wm + "kind must be 'dense'");
            const long long ff = C::integer(mlp, "ff", wm);
            if (ff <= 0) throw ConfigError(wm + "ff must be > 0");
            layer.sublayers.push_back({"feed_forward", PartSpec{"xielu", Params{{"hidden_size", width}, {"ff", ff}}, prefix + ".mlp", true}, norm(prefix + ".norm2"),
                                       "pre", norm(prefix + ".norm2b")});
        }
        spec.layers.push_back(std::move(layer));
    }
    // the run order: the layers in front of the loop, the loop's layers `times` times (a cache or state per pass), the rest
    const long long n = (long long)spec.layers.size();
    long long start = n, stop = n, times = 1;
    if (C::present(config, "loop")) {
        const json::Value& loop = *config.find("loop");
        start = C::integer(loop, "start", "loop.");
        stop = C::integer(loop, "stop", "loop.");
        times = C::integer(loop, "times", "loop.");
        if (start < 0 || stop < start || stop > n || times < 1) throw ConfigError("loop must have 0 <= start <= stop <= layers and times >= 1");
    }
    int cache = 0;
    auto run = [&](long long layer) { spec.run_order.push_back(RunEntry{(int)layer, cache++, true}); };
    for (long long i = 0; i < std::min(start, n); ++i) run(i);
    for (long long t = 0; t < times; ++t)
        for (long long i = start; i < stop; ++i) run(i);
    for (long long i = stop; i < n; ++i) run(i);
    Params embedding{{"vocab_size", vocab}, {"hidden_size", width}, {"weight_name", ""}};
    if (C::present(config, "embedding")) embedding.set("scale", C::number(*config.find("embedding"), "scale", "embedding."));
    spec.embedding = PartSpec{"embedding", embedding, "embed", true};
    spec.final_norm = norm("final.norm");
    Params head{{"vocab_size", vocab}, {"hidden_size", width}, {"weight_name", ""}};
    if (C::present(config, "logit_scale")) head.set("scale", C::number(config, "logit_scale", ""));
    spec.lm_head = PartSpec{"lm_head", head, "head", true};
    return spec;
}

// ---- Masezen ---------------------------------------------------------------------------------------------------------------
// A decoder whose config.json lists its layers one by one.  A layer has ONE norm (an RMS norm whose gain is a single number)
// that both branches read, side by side:  h = n(x);  x = x + s1 * mixer(h + conv(h)) + s2 * ff(h),  with conv a causal
// convolution over time on each channel (canon.taps taps, the last taps - 1 rows of h kept per request), s1 and s2 a gain
// per channel; behind it every layer adds a small gated map of a per-token vector (token_side.dim columns of a table that
// all layers share) through an RMS norm of its own.  The mixer ("type": "attention") is grouped-query attention whose
// values are the keys as projected, with normed and turned queries and keys, scores mixed across the heads and a gated
// output.  "mlp" is null, a dense feed-forward with a squared ReLU, or routed experts with a clamped gate whose weights
// multiply the experts' inputs, beside a shared expert.  Every size and constant is a key of config.json; tensor names are
// "l<i>.<part>.<tensor>".
inline ModelSpec masezen_spec(const json::Value& config) {
    using C = GufanexConfig;
    if (!config.is_object()) throw ConfigError("config.json is not a JSON object");
    ModelSpec spec;
    spec.architecture = "masezen";
    const long long width = C::integer(config, "width", ""), vocab = C::integer(config, "vocab", "");
    if (width <= 0 || vocab <= 0) throw ConfigError("width and vocab must be > 0");
    const double eps = C::number(C::need(config, "norm", ""), "eps", "norm.");
    if (eps <= 0.0) throw ConfigError("norm.eps must be > 0");
    spec.vocab_size = vocab;
    spec.hidden_size = width;
    spec.max_positions = C::integer_or(config, "max_positions", 1LL << 30, "");
    auto single_norm = [&](const std::string& name) {
        return PartSpec{"rmsnorm", Params{{"size", width}, {"eps", eps}, {"weight_name", ""}, {"single_gain", 1}}, name, true};
    };
    const long long taps = C::present(config, "canon") ? C::integer(*config.find("canon"), "taps", "canon.") : 0;
    if (taps < 0 || taps > 8) throw ConfigError("canon.taps must lie in 1..8");
    const long long side = C::present(config, "token_side") ? C::integer(*config.find("token_side"), "dim", "token_side.") : 0;
    if (side < 0) throw ConfigError("token_side.dim must be > 0");
    const json::Value& layers = C::need(config, "layers", "");
    if (!layers.is_array() || layers.array.empty()) throw ConfigError("layers must be a list with at least one layer");
    const long long count = (long long)layers.array.size();
    for (size_t i = 0; i < layers.array.size(); ++i) {
        const json::Value& l = layers.array[i];
        const std::string where = "layers[" + std::to_string(i) + "].", prefix = "l" + std::to_string(i), w = where + "mixer.";
        const json::Value& type = C::need(l, "type", where);
        const json::Value& m = C::need(l, "mixer", where);
        if (!type.is_string() || type.string != "attention") throw ConfigError(where + "type must be 'attention', the mixer of this design");
        LayerSpec layer;
        layer.parallel = true;
        const long long heads = C::integer(m, "heads", w), kv_heads = C::integer(m, "kv_heads", w), dim = C::integer(m, "dim", w);
        if (heads <= 0 || kv_heads <= 0 || dim <= 0 || heads % kv_heads) throw ConfigError(w + "heads, kv_heads and dim must be > 0, heads a multiple of kv_heads");
        if (C::present(m, "vdim") && C::integer(m, "vdim", w) != dim) throw ConfigError(w + "vdim must equal dim: the values are the keys");
        PartSpec mixer{"mixed_attention", Params{{"hidden_size", width}, {"heads", heads}, {"kv_heads", kv_heads}, {"dim", dim}, {"scale", C::number(m, "scale", w)},
                                                 {"norm_eps", eps}}, prefix + ".mix", true};
        if (C::present(m, "rot")) {
            const json::Value& rot = *m.find("rot");
            const long long dims = C::integer(rot, "dims", w + "rot.");
            if (dims < 0 || dims % 2 || dims > dim) throw ConfigError(w + "rot.dims must be even and within dim");
            if (dims > 0) {
                Params r{{"head_dim", dim}, {"rotary_dim", dims}, {"theta", C::number(rot, "base", w + "rot.")}};
                if (C::present(rot, "scaling")) {
                    const json::Value& sc = *rot.find("scaling");
                    const std::string ws = w + "rot.scaling.";
                    r.set("scaling_factor", C::number(sc, "factor", ws));
                    r.set("scaling_original", C::number(sc, "original", ws));
                    r.set("scaling_fast", C::number(sc, "fast", ws));
                    r.set("scaling_slow", C::number(sc, "slow", ws));
                }
                layer.position = PartSpec{"rope", r, "", true};
            }
        }
        auto gain = [&](const std::string& name) { return PartSpec{"layer_scale", Params{{"size", width}, {"weight_name", ""}}, name, true}; };
        SubLayerSpec mix{"mixer", mixer, single_norm(prefix + ".norm1"), "pre", gain(prefix + ".ls1")};
        if (taps > 0) mix.shift = PartSpec{"conv_shift", Params{{"size", width}, {"taps", taps}}, prefix + ".canon1", true};
        layer.sublayers.push_back(std::move(mix));
        if (C::present(l, "mlp")) {
            const json::Value& mlp = *l.find("mlp");
            const std::string wm = where + "mlp.";
            const json::Value& kind = C::need(mlp, "kind", wm);
            if (!kind.is_string()) throw ConfigError(wm + "kind must be a string");
            PartSpec ff;
            if (kind.string == "dense") {
                const long long f = C::integer(mlp, "ff", wm);
                if (f <= 0) throw ConfigError(wm + "ff must be > 0");
                ff = PartSpec{"squared_relu", Params{{"hidden_size", width}, {"ff", f}}, prefix + ".mlp", true};
            } else if (kind.string == "moe") {
                const json::Value& router = C::need(mlp, "router", wm);
                const json::Value& expert = C::need(mlp, "expert", wm);
                const long long experts = C::integer(router, "experts", wm + "router."), top = C::integer(router, "top", wm + "router.");
                const long long f = C::integer(expert, "ff", wm + "expert.");
                const double limit = C::number(expert, "limit", wm + "expert.");
                if (experts <= 0 || top <= 0 || top > experts || f <= 0 || limit <= 0.0)
                    throw ConfigError(wm + "needs router.experts >= router.top > 0, expert.ff > 0 and expert.limit > 0");
                Params e{{"hidden_size", width}, {"experts", experts}, {"top", top}, {"ff", f}, {"scoring", "sigmoid"}, {"correction", 0}, {"activation", "clamped"},
                         {"limit", limit}, {"weight_input", 1}, {"shared_gated", 0}};
                if (C::present(mlp, "shared")) {
                    const json::Value& shared = *mlp.find("shared");
                    const long long sf = C::integer(shared, "ff", wm + "shared.");
                    const double sl = C::number(shared, "limit", wm + "shared.");
                    if (sf <= 0 || sl <= 0.0) throw ConfigError(wm + "shared.ff and shared.limit must be > 0");
                    e.set("shared_ff", sf);
                    e.set("shared_activation", "clamped");
                    e.set("shared_limit", sl);
                }
                ff = PartSpec{"routed_experts", e, prefix + ".mlp", true};
            } else {
                throw ConfigError(wm + "kind '" + kind.string + "' is no feed-forward of this design (dense, moe)");
            }
            // no norm of its own: it reads the rows of the mixer's norm, as they are in front of the convolution
            layer.sublayers.push_back({"feed_forward", ff, PartSpec::none(), "pre", gain(prefix + ".ls2")});
        } else {
            spec.ignored_tensors.push_back(prefix + ".ls2");        // a layer without a feed-forward may still carry its gain
        }
        if (side > 0) {
            PartSpec part{"token_side", Params{{"hidden_size", width}, {"vocab_size", vocab}, {"side", side}, {"column", (long long)i * side}, {"columns", count * side},
                                               {"table", "side.embed"}}, prefix + ".side", true};
            layer.sublayers.push_back({"feed_forward", part, PartSpec::none(), "pre",
                                       PartSpec{"rmsnorm", Params{{"size", width}, {"eps", eps}, {"weight_name", ""}}, prefix + ".side.norm", true}});
            layer.sequential_tail = 1;
        }
        spec.layers.push_back(std::move(layer));
    }
    for (int i = 0; i < (int)spec.layers.size(); ++i) spec.run_order.push_back(RunEntry{i, i, true});
    spec.embedding = PartSpec{"embedding", Params{{"vocab_size", vocab}, {"hidden_size", width}, {"weight_name", ""}}, "embed", true};
    spec.final_norm = single_norm("final.norm");
    spec.lm_head = PartSpec{"lm_head", Params{{"vocab_size", vocab}, {"hidden_size", width}, {"weight_name", ""}}, "head", true};
    return spec;
}

// ---- Mozalix ---------------------------------------------------------------------------------------------------------------
// A decoder whose config.json lists its layers one by one.  A layer's branches read the stream itself and are normed on their
// way back into it, x = x + n1(mixer(x)), x = x + n2(ff(x)), with RMS norms whose tensors hold the gain minus one.  The
// mixer is one of three: "attention" (grouped heads, q and k normed per head with a shared gain and then turned, keys of the
// query's own block of mask.size positions, a learned sink per head), "attention_2" (two softmax maps a head over a sliding
// window, the second taken off the first with one weight for the layer, the difference normed per head) and "parallel" (an
// attention without positions, with unit-rms q and k, capped scores and a window that also keeps the sequence's first tokens,
// beside a gated delta-rule mixer with a decay per key channel; the two outputs are summed with a weight each).  The
// feed-forward is a gated one with clamped gate and up values and biases on all three maps, or none.  A layer with
// "weights_of": j runs layer j's tensors on a cache and state of its own.  The embedding is scaled by embedding.scale.  Every
// size and constant is a key of config.json; tensor names are "l<i>.<part>.<tensor>".
// whether two values of a configuration say the same (members of an object in any order)
inline bool same_config_value(const json::Value& a, const json::Value& b) {
    if (a.type != b.type) return false;
    switch (a.type) {
        case json::Value::Null: return true;
        case json::Value::Bool: return a.boolean == b.boolean;
        case json::Value::Number: return a.number == b.number;
        case json::Value::String: return a.string == b.string;
        case json::Value::Array:
            if (a.array.size() != b.array.size()) return false;
            for (size_t i = 0; i < a.array.size(); ++i)
                if (!same_config_value(a.array[i], b.array[i])) return false;
            return true;
        case json::Value::Object:
            if (a.object.size() != b.object.size()) return false;
            for (auto& kv : a.object) {
                const json::Value* other = b.find(kv.first);
                if (!other || !same_config_value(kv.second, *other)) return false;
            }
            return true;
    }
    return false;
}

inline ModelSpec mozalix_spec(const json::Value& config) {
    using C = GufanexConfig;        // the typed readers (a key's path goes into the refusal)
    if (!config.is_object()) throw ConfigError("config.json is not a JSON object");
    ModelSpec spec;
    spec.architecture = "mozalix";
    const long long width = C::integer(config, "width", ""), vocab = C::integer(config, "vocab", "");
    if (width <= 0 || vocab <= 0) throw ConfigError("width and vocab must be > 0");
    const double eps = C::number(C::need(config, "norm", ""), "eps", "norm.");
    if (eps <= 0.0) throw ConfigError("norm.eps must be > 0");
    spec.vocab_size = vocab;
    spec.hidden_size = width;
    spec.max_positions = C::integer_or(config, "max_positions", 1LL << 30, "");     // the design sets no limit; positions are 32-bit
    auto norm = [&](const std::string& name) {
        return PartSpec{"rmsnorm", Params{{"size", width}, {"eps", eps}, {"weight_name", ""}, {"offset", 1.0}}, name, true};
    };
    // the sizes every attention of this design has, and its mask's size if it has a mask
    auto attention = [&](const json::Value& m, const std::string& w, long long* mask_size) {
        const long long heads = C::integer(m, "heads", w), kv_heads = C::integer(m, "kv_heads", w), dim = C::integer(m, "dim", w), vdim = C::integer(m, "vdim", w);
        if (heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || heads % kv_heads)
            throw ConfigError(w + "heads, kv_heads, dim and vdim must be > 0, heads a multiple of kv_heads");
        *mask_size = 0;
        if (C::present(m, "mask")) {
            *mask_size = C::integer(*m.find("mask"), "size", w + "mask.");
            if (*mask_size <= 0) throw ConfigError(w + "mask.size must be > 0");
        }
        return Params{{"hidden_size", width}, {"heads", heads}, {"kv_heads", kv_heads}, {"dim", dim}, {"vdim", vdim}, {"scale", C::number(m, "scale", w)},
                      {"norm_eps", eps}};
    };
    auto rotation = [&](const json::Value& m, const std::string& w) {
        if (!C::present(m, "rot")) return PartSpec::none();
        const json::Value& rot = *m.find("rot");
        const long long dims = C::integer(rot, "dims", w + "rot."), dim = C::integer(m, "dim", w);
        if (dims < 0 || dims % 2 || dims > dim) throw ConfigError(w + "rot.dims must be even and within dim");
        if (dims == 0) return PartSpec::none();
        return PartSpec{"rope", Params{{"head_dim", dim}, {"rotary_dim", dims}, {"theta", C::number(rot, "base", w + "rot.")}}, "", true};
    };
    const json::Value& layers = C::need(config, "layers", "");
    if (!layers.is_array() || layers.array.empty()) throw ConfigError("layers must be a list with at least one layer");
    const long long count = (long long)layers.array.size();
    // whose tensors a layer uses: its own, or (through "weights_of", possibly in several steps) another layer's
    std::vector<long long> owner(count);
    for (long long i = 0; i < count; ++i) {
        long long j = i;
        for (long long hops = 0; C::present(layers.array[j], "weights_of"); ++hops) {
            const std::string where = "layers[" + std::to_string(j) + "].";
            j = C::integer(layers.array[j], "weights_of", where);
            if (j < 0 || j >= count || hops > count) throw ConfigError(where + "weights_of must name a layer that has tensors of its own");
        }
        owner[i] = j;
    }
    std::vector<int> built(count, -1);           // layer index -> index into spec.layers, for layers with tensors of their own
    for (long long i = 0; i < count; ++i) {
        if (owner[i] != i) continue;
        const json::Value& l = layers.array[i];
        const std::string where = "layers[" + std::to_string(i) + "].", prefix = "l" + std::to_string(i), w = where + "mixer.";
        const json::Value& type = C::need(l, "type", where);
        const json::Value& m = C::need(l, "mixer", where);
        if (!type.is_string()) throw ConfigError(where + "type must be a string");
        LayerSpec layer;
        PartSpec mixer;
        long long mask = 0;
        if (type.string == "attention") {
            Params a = attention(m, w, &mask);
            a.set("qk_norm", "gain");
            a.set("sinks", 1);
            if (mask > 0) a.set("chunk", mask);
            mixer = PartSpec{"masked_attention", a, prefix + ".mix", true};
            layer.position = rotation(m, w);
        } else if (type.string == "attention_2") {
            Params a = attention(m, w, &mask);
            a.set("qk_norm", "gain");
            a.set("maps", 2);
            a.set("diff", C::number(m, "diff", w));
            if (mask > 0) a.set("window", mask);
            mixer = PartSpec{"masked_attention", a, prefix + ".mix", true};
            layer.position = rotation(m, w);
        } else if (type.string == "parallel") {
            const json::Value& left = C::need(m, "left", w);
            const json::Value& right = C::need(m, "right", w);
            const std::string wl = w + "left.", wr = w + "right.";
            Params a = attention(left, wl, &mask);
            a.set("qk_norm", "unit");
            if (mask > 0) {
                a.set("window", mask);
                const long long keep = C::integer_or(*left.find("mask"), "keep_first", 0, wl + "mask.");
                if (keep < 0) throw ConfigError(wl + "mask.keep_first must not be negative");
                a.set("keep_first", keep);
            }
            if (C::present(left, "softcap")) {
                const double cap = C::number(left, "softcap", wl);
                if (cap <= 0.0) throw ConfigError(wl + "softcap must be > 0");
                a.set("softcap", cap);
            }
            a.set("out_scale", C::number(m, "left_scale", w));
            const long long heads = C::integer(right, "heads", wr), kv_heads = C::integer(right, "kv_heads", wr), dim = C::integer(right, "dim", wr),
                            vdim = C::integer(right, "vdim", wr), conv = C::integer(right, "conv", wr);
            if (heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || heads % kv_heads || conv < 1)
                throw ConfigError(wr + "heads, kv_heads, dim, vdim and conv must be > 0, heads a multiple of kv_heads");
            Params d{{"hidden_size", width}, {"heads", heads}, {"kv_heads", kv_heads}, {"dim", dim}, {"vdim", vdim}, {"conv", conv}, {"eps", eps}, {"unit_eps", 1e-6},
                     {"gate", "sigmoid"}, {"out_scale", C::number(m, "right_scale", w)}};
            if (C::present(right, "rank")) d.set("rank", C::integer(right, "rank", wr));        // only what random-weights mode writes: a file's tensors decide
            Params both{{"left_kind", "masked_attention"}, {"right_kind", "channel_delta"}};
            both.merge("left.", a);
            both.merge("right.", d);
            mixer = PartSpec{"side_by_side", both, prefix + ".mix", true};
        } else {
            throw ConfigError(where + "type '" + type.string + "' is no mixer of this design (attention, attention_2, parallel)");
        }
        layer.sublayers.push_back({"mixer", mixer, PartSpec::none(), "pre", norm(prefix + ".norm1")});
        if (C::present(l, "mlp")) {
            const json::Value& mlp = *l.find("mlp");
            const std::string wm = where + "mlp.";
            const json::Value& kind = C::need(mlp, "kind", wm);
            if (!kind.is_string() || kind.string != "dense") throw ConfigError(wm + "kind must be 'dense'");
            const long long ff = C::integer(mlp, "ff", wm);
            const double limit = C::number(mlp, "limit", wm);
            if (ff <= 0 || limit <= 0.0) throw ConfigError(wm + "ff and limit must be > 0");
            Params f{{"hidden_size", width}, {"intermediate_size", ff}, {"bias", true}, {"activation", "clamped"}, {"limit", limit}, {"gate_name", ".gate"},
                     {"up_name", ".up"}, {"down_name", ".down"}, {"gate_bias_name", ".gate.b"}, {"up_bias_name", ".up.b"}, {"down_bias_name", ".down.b"}};
            layer.sublayers.push_back({"feed_forward", PartSpec{"swiglu", f, prefix + ".mlp", true}, PartSpec::none(), "pre", norm(prefix + ".norm2")});
        }
        built[i] = (int)spec.layers.size();
        spec.layers.push_back(std::move(layer));
    }
    for (long long i = 0; i < count; ++i) {
        const json::Value& l = layers.array[i];
        if (owner[i] != i) {
            const json::Value &mine = C::need(l, "type", "layers[" + std::to_string(i) + "]."), &theirs = C::need(layers.array[owner[i]], "type", "");
            if (!mine.is_string() || mine.string != theirs.string)
                throw ConfigError("layers[" + std::to_string(i) + "] uses the tensors of a layer of another type");
            // one set of parts runs both layers: sizes and constants that differed would be ignored without a word
            static const json::Value none;
            for (const char* key : {"mixer", "mlp"}) {
                const json::Value *a = l.find(key), *b = layers.array[owner[i]].find(key);
                if (!same_config_value(a ? *a : none, b ? *b : none))
                    throw ConfigError("layers[" + std::to_string(i) + "]." + key + " differs from that of the layer whose tensors it uses");
            }
        }
        spec.run_order.push_back(RunEntry{built[owner[i]], (int)i, true});
    }
    Params embedding{{"vocab_size", vocab}, {"hidden_size", width}, {"weight_name", ""}};
    if (C::present(config, "embedding")) embedding.set("scale", C::number(*config.find("embedding"), "scale", "embedding."));
    spec.embedding = PartSpec{"embedding", embedding, "embed", true};
    spec.final_norm = norm("final.norm");
    spec.lm_head = PartSpec{"lm_head", Params{{"vocab_size", vocab}, {"hidden_size", width}, {"weight_name", ""}}, "head", true};
    return spec;
}

inline void register_builtin_architectures() {
    ArchitectureRegistry& r = ArchitectureRegistry::instance();
    for (auto& e : r.entries)
        if (e.first == "qwen2") return;
    r.add("qwen2", qwen2_spec);
    r.add("gufanex", gufanex_spec);
    r.add("lasizen", lasizen_spec);
    r.add("masezen", masezen_spec);
    r.add("mozalix", mozalix_spec);
}

}  // namespace easygpt::engine
