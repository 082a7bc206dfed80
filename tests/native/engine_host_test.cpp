// The native engine's host-only parts from C++ alone (no GPU, no CUDA headers): the JSON reader, the safetensors
// reader with every malformed file refused, the one error that lists missing / unexpected / wrongly shaped tensors, the
// typed Qwen2 configuration with what cannot run refused, the architecture registry's rule, and the run order's checks.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <iostream>

#include "architectures.hpp"
#include "weights.hpp"

using namespace easygpt;
using namespace easygpt::engine;

static int failures = 0;
#define CHECK(cond)                                                                 \
    do {                                                                            \
        if (!(cond)) {                                                              \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);           \
            ++failures;                                                             \
        }                                                                           \
    } while (0)

template <class E> static bool throws(const std::function<void()>& f, const std::string& part) {
    try {
        f();
    } catch (const E& e) {
        if (std::string(e.what()).find(part) != std::string::npos) return true;
        std::printf("  message was: %s\n", e.what());
        return false;
    } catch (...) {
        return false;
    }
    return false;
}

static std::string safetensors_bytes(const std::string& header, const std::string& data) {
    std::string out(8, '\0');
    const uint64_t n = header.size();
    for (int i = 0; i < 8; ++i) out[i] = (char)(n >> (8 * i));
    return out + header + data;
}
static std::string write_file(const std::string& dir, const std::string& name, const std::string& bytes) {
    const std::string path = dir + "/" + name;
    std::ofstream(path, std::ios::binary).write(bytes.data(), (std::streamsize)bytes.size());
    return path;
}

static const char* kConfig = R"({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 3, "hidden_size": 80,
  "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 208, "vocab_size": 391, "rope_theta": 1000000.0,
  "rms_norm_eps": 1e-5, "tie_word_embeddings": false, "max_position_embeddings": 2048, "bos_token_id": null, "eos_token_id": [7, 9],
  "use_sliding_window": true, "sliding_window": 24, "max_window_layers": 1})";

// The configuration text with `key` dropped (value empty) or set to `value`.
static std::string with(const std::string& config, const std::string& key, const std::string& value) {
    std::string text = config;
    const std::string needle = "\"" + key + "\":";
    size_t at = text.find(needle);
    if (at != std::string::npos) {
        size_t end = at + needle.size();
        int depth = 0;
        while (end < text.size() && !((text[end] == ',' || text[end] == '}') && depth == 0)) {
            if (text[end] == '[') ++depth;
            if (text[end] == ']') --depth;
            ++end;
        }
        if (text[end] == ',') ++end;
        text.erase(at, end - at);
    }
    if (!value.empty()) {
        const size_t brace = text.rfind('}');
        std::string head = text.substr(0, brace);
        while (!head.empty() && (head.back() == ' ' || head.back() == '\n' || head.back() == ',')) head.pop_back();
        text = head + ", \"" + key + "\": " + value + "}";
    } else {
        const size_t brace = text.rfind('}');
        std::string head = text.substr(0, brace);
        while (!head.empty() && (head.back() == ' ' || head.back() == '\n' || head.back() == ',')) head.pop_back();
        text = head + "}";
    }
    return text;
}

int main(int argc, char** argv) {
    const std::string dir = argc > 1 ? argv[1] : ".";

    // ---- JSON ----------------------------------------------------------------------------------------------------
    {
        const json::Value v = json::parse(R"({"a": [1, 2.5, -3e2, true, null], "s": "x\né😀\"", "o": {"k": 12345678901234}})");
        CHECK(v.find("a")->array.size() == 5 && v.find("a")->array[0].is_integer && v.find("a")->array[0].integer == 1);
        CHECK(!v.find("a")->array[1].is_integer && v.find("a")->array[1].number == 2.5 && v.find("a")->array[2].number == -300.0);
        CHECK(v.find("a")->array[3].boolean && v.find("a")->array[4].is_null());
        CHECK(v.find("s")->string == "x\n\xc3\xa9\xf0\x9f\x98\x80\"");
        CHECK(v.find("o")->find("k")->integer == 12345678901234LL && v.object[0].first == "a" && !v.contains("missing"));
        CHECK(throws<json::ParseError>([] { json::parse("{\"a\": }"); }, "byte"));
        CHECK(throws<json::ParseError>([] { json::parse("[1, 2] x"); }, "after the JSON value"));
        CHECK(throws<json::ParseError>([] { json::parse("\"abc"); }, "unterminated"));
    }

    // ---- safetensors: what is malformed is refused (src/models/loader.cpp:79-140, 214-252) ------------------------------
    {
        CHECK(throws<SafetensorsError>([&] { SafetensorsFile f(dir + "/nowhere.safetensors"); }, "cannot open"));
        CHECK(throws<SafetensorsError>([&] { SafetensorsFile f(write_file(dir, "short", "abc")); }, "smaller than the 8-byte"));
        CHECK(throws<SafetensorsError>([&] { SafetensorsFile f(write_file(dir, "long", std::string("\xff\xff\0\0\0\0\0\0", 8) + "{}")); }, "exceeds the file size"));
        CHECK(throws<SafetensorsError>([&] { SafetensorsFile f(write_file(dir, "nojson", safetensors_bytes("{not json", ""))); }, "not JSON"));
        CHECK(throws<SafetensorsError>([&] { SafetensorsFile f(write_file(dir, "array", safetensors_bytes("[1]", ""))); }, "not a JSON object"));
        auto one = [&](const std::string& meta, const std::string& data = std::string(8, '\0')) {
            return [=] { SafetensorsFile f(write_file(dir, "one", safetensors_bytes("{\"t\": " + meta + "}", data))); };
        };
        CHECK(throws<SafetensorsError>(one(R"({"shape": [2], "data_offsets": [0, 8]})"), "missing dtype"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F64", "shape": [1], "data_offsets": [0, 8]})"), "Unsupported dtype F64"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [], "data_offsets": [0, 8]})"), "needs 4"));       // no dimensions: one number
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [2, 0], "data_offsets": [0, 8]})"), "bad dimension"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [2.5], "data_offsets": [0, 8]})"), "bad dimension"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [2], "data_offsets": [8, 0]})"), "bad data_offsets"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [2], "data_offsets": [0, 16]})"), "past the end"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [3], "data_offsets": [0, 8]})"), "8 bytes stored"));
        // a good file: F32, BF16 and F16 values read as float32; __metadata__ skipped
        const float f32[2] = {1.5f, -2.0f};
        const uint16_t bf[2] = {0x3fc0, 0xc000}, fh[3] = {0x3e00, 0xc000, 0x0001};
        std::string data((const char*)f32, 8);
        data += std::string((const char*)bf, 4) + std::string((const char*)fh, 6);
        SafetensorsFile good(write_file(dir, "good", safetensors_bytes(
            R"({"__metadata__": {"format": "pt"}, "a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},)"
            R"( "b": {"dtype": "BF16", "shape": [2, 1], "data_offsets": [8, 12]}, "c": {"dtype": "F16", "shape": [3], "data_offsets": [12, 18]}})", data)));
        CHECK(good.entries().size() == 3 && !good.find("__metadata__"));
        float out[3];
        good.find("a")->to_float(out);
        CHECK(out[0] == 1.5f && out[1] == -2.0f);
        good.find("b")->to_float(out);
        CHECK(out[0] == 1.5f && out[1] == -2.0f && good.find("b")->shape.size() == 2);
        good.find("c")->to_float(out);
        CHECK(out[0] == 1.5f && out[1] == -2.0f && out[2] > 0 && out[2] < 1e-7f);
        CHECK(float_to_bf16(1.5f) == 0x3fc0 && float_to_bf16(1.00390625f) == 0x3f80 && float_to_bf16(1.01171875f) == 0x3f82);      // ties to even
        // one error for everything: missing, unexpected, wrong shape; [n, 1] accepted like [n]
        std::vector<TensorRequest> wanted = {TensorRequest::vector("a", 2), TensorRequest::vector("b", 2), TensorRequest::matrix("c", 3, 1),
                                             TensorRequest::matrix("d", 4, 4), TensorRequest::vector("e", 4)};
        CHECK(throws<WeightError>([&] { check_manifest(wanted, good); }, "Missing required model weights: d, e"));
        CHECK(throws<WeightError>([&] { check_manifest(wanted, good); }, "Invalid tensor shape for key 'c': expected [3, 1], got [3]"));
        CHECK(throws<WeightError>([&] { check_manifest({TensorRequest::vector("a", 2)}, good); }, "Unexpected tensors in the file: b, c"));
        check_manifest({TensorRequest::vector("a", 2), TensorRequest::vector("b", 2), TensorRequest::vector("c", 3)}, good);
    }

    // ---- the typed configuration and the registry ------------------------------------------------------------------------
    {
        register_builtin_architectures();
        const ModelSpec spec = ArchitectureRegistry::instance().build(json::parse(kConfig));
        CHECK(spec.architecture == "qwen2" && spec.layers.size() == 3 && spec.run_order.size() == 3 && spec.vocab_size == 391);
        CHECK(spec.eos_token_id == 7 && spec.bos_token_id == -1 && spec.max_positions == 2048);
        const SubLayerSpec& mixer = spec.layers[1].sublayers[0];
        CHECK(mixer.role == "mixer" && mixer.part.kind == "attention" && mixer.part.params.integer("window") == 24 &&
              mixer.part.params.integer("head_dim") == 32 && mixer.part.prefix == "model.layers.1.self_attn");       // src/models/layer_key_prefix.cpp:77-87
        CHECK(!spec.layers[0].sublayers[0].part.params.has("window"));                                                // windows from layer 1 on
        CHECK(spec.layers[1].sublayers[1].part.kind == "swiglu" && spec.layers[1].sublayers[1].part.params.integer("intermediate_size") == 208);
        CHECK(mixer.norm.params.real("eps") == 1e-5 && spec.layers[1].position.params.real("theta") == 1e6);
        CHECK(!spec.lm_head.params.has("tied_to") && spec.lm_head.prefix == "lm_head");
        const ModelSpec tied = ArchitectureRegistry::instance().build(json::parse(with(kConfig, "tie_word_embeddings", "true")));
        CHECK(tied.lm_head.params.text("tied_to") == "model.embed_tokens");
        // the reference's rule: the key occurs in architectures[0], or equals model_type (src/models/layer_key_prefix.cpp:92-105)
        ArchitectureRegistry::instance().build(json::parse(with(with(kConfig, "architectures", "[\"MyQwen2Thing\"]"), "model_type", "\"other\"")));
        ArchitectureRegistry::instance().build(json::parse(with(with(kConfig, "architectures", ""), "model_type", "\"QWEN2\"")));
        CHECK(throws<std::invalid_argument>([&] {
            ArchitectureRegistry::instance().build(json::parse(with(with(kConfig, "architectures", "[\"LlamaForCausalLM\"]"), "model_type", "\"llama\"")));
        }, "Unsupported model architecture/model_type: architecture='LlamaForCausalLM', model_type='llama'"));
        auto refuse = [&](const std::string& key, const std::string& value, const std::string& message) {
            const bool ok = throws<ConfigError>([&] { ArchitectureRegistry::instance().build(json::parse(with(kConfig, key, value))); }, message);
            if (!ok) std::printf("  (%s = %s)\n", key.c_str(), value.c_str());
            return ok;
        };
        CHECK(refuse("vocab_size", "", "config.json lacks: vocab_size"));
        CHECK(refuse("hidden_size", "\"80\"", "hidden_size must be an integer"));
        CHECK(refuse("num_key_value_heads", "4", "must be a multiple of num_key_value_heads"));
        CHECK(refuse("head_dim", "31", "head_dim must be even"));
        CHECK(refuse("rope_theta", "0", "rope_theta must be > 0"));
        CHECK(refuse("rms_norm_eps", "0", "rms_norm_eps must be > 0"));
        CHECK(refuse("hidden_act", "\"gelu\"", "is not supported (silu only)"));
        CHECK(refuse("rope_scaling", "{\"type\": \"yarn\"}", "rope_scaling is not supported"));
        CHECK(refuse("sliding_window", "null", "needs a positive integer sliding_window"));
        CHECK(refuse("num_hidden_layers", "0", "num_hidden_layers must be > 0"));
        const ModelSpec derived = ArchitectureRegistry::instance().build(json::parse(with(with(kConfig, "head_dim", ""), "num_attention_heads", "4")));
        CHECK(derived.layers[0].sublayers[0].part.params.integer("head_dim") == 20);                               // hidden / heads when no key
        CHECK(refuse("head_dim", "", "hidden_size must be divisible by num_attention_heads"));                       // 80 / 6
        // the run order is data and is checked
        ModelSpec bad = spec;
        bad.run_order = {RunEntry{0, 0, true}, RunEntry{5, 1, true}};
        CHECK(throws<std::invalid_argument>([&] { bad.validate(); }, "names layer 5"));
        bad.run_order = {RunEntry{0, 0, true}, RunEntry{1, 0, true}};
        CHECK(throws<std::invalid_argument>([&] { bad.validate(); }, "is written by run entries 0 and 1"));
        bad.run_order = {RunEntry{0, 1, false}, RunEntry{1, 1, true}};
        CHECK(throws<std::invalid_argument>([&] { bad.validate(); }, "before entry 1 has written it"));
        bad.run_order = {RunEntry{0, 0, true}, RunEntry{1, 1, true}, RunEntry{0, 2, true}, RunEntry{1, 1, false}};
        bad.validate();                                                                                             // a layer twice, a shared cache: fine
    }


    // ---- a design whose config.json lists its layers: mixers by type, a repeated run of layers, parallel sub-layers --------------
    {
        const char* kListed = R"({"architecture": "Gufanex", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "logit_softcap": 12.5,
          "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [
            {"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 20, "q_rank": 24, "scale": 0.3,
                                                   "rot": {"base": 500.0, "dims": 4}}, "mlp": null},
            {"type": "mamba1", "mixer": {"inner": 48, "state": 5, "dt_rank": 3, "conv": 3},
             "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 5, "identity": 2, "top": 2}, "shared": {"ff": 24}}},
            {"type": "latent_attention", "mixer": {"heads": 1, "dim": 16, "rot_dim": 8, "vdim": 16, "kv_rank": 12, "q_rank": 8, "scale": 0.25,
                                                   "rot": {"base": 10000.0, "dims": 8}},
             "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 2, "identity": 0, "top": 1}}},
            {"type": "mamba1", "mixer": {"inner": 16, "state": 2, "dt_rank": 1, "conv": 2}, "mlp": null}]})";
        const ModelSpec spec = ArchitectureRegistry::instance().build(json::parse(kListed));
        CHECK(spec.architecture == "gufanex" && spec.layers.size() == 4 && spec.vocab_size == 97 && spec.hidden_size == 40);
        // layer 0, then layers 1 and 2 twice with a cache each, then layer 3
        CHECK(spec.run_order.size() == 6);
        const int layers[] = {0, 1, 2, 1, 2, 3};
        for (size_t i = 0; i < spec.run_order.size(); ++i) CHECK(spec.run_order[i].layer == layers[i] && spec.run_order[i].cache == (int)i && spec.run_order[i].writes_cache);
        // a pass starts with the pass's learned vector; every pass but the first also adds the embedding's output
        CHECK(spec.stream_adds.size() == 1 && spec.stream_adds[0].prefix == "loop.step" && spec.stream_adds[0].params.integer("rows") == 2);
        CHECK(spec.run_order[1].stream_add == 0 && spec.run_order[1].stream_add_row == 0 && !spec.run_order[1].add_embedding);
        CHECK(spec.run_order[3].stream_add == 0 && spec.run_order[3].stream_add_row == 1 && spec.run_order[3].add_embedding);
        CHECK(spec.run_order[0].stream_add < 0 && spec.run_order[2].stream_add < 0 && spec.run_order[4].stream_add < 0 && spec.run_order[5].stream_add < 0);
        CHECK(spec.layers[0].parallel && spec.layers[0].sublayers.size() == 1 && spec.layers[1].sublayers.size() == 2);
        const PartSpec& latent = spec.layers[0].sublayers[0].part;
        CHECK(latent.kind == "latent_attention" && latent.prefix == "l0.mix" && latent.params.integer("kv_rank") == 20 && latent.params.real("scale") == 0.3 &&
              latent.params.real("rot_base") == 500.0 && latent.params.integer("rot_dims") == 4 && latent.params.real("eps") == 1e-5);
        const PartSpec& scan = spec.layers[1].sublayers[0].part;
        CHECK(scan.kind == "selective_scan" && scan.params.integer("inner") == 48 && scan.params.integer("state") == 5 && scan.params.integer("conv") == 3);
        const PartSpec& routed = spec.layers[1].sublayers[1].part;
        CHECK(routed.kind == "routed_experts" && routed.prefix == "l1.mlp" && routed.params.integer("experts") == 5 && routed.params.integer("identity") == 2 &&
              routed.params.integer("top") == 2 && routed.params.integer("ff") == 16 && routed.params.integer("shared_ff") == 24);
        CHECK(spec.layers[2].sublayers[1].part.params.integer("shared_ff") == 0);
        CHECK(spec.layers[1].sublayers[1].norm.kind == "layernorm" && spec.layers[1].sublayers[1].norm.prefix == "l1.norm2" &&
              spec.layers[1].sublayers[1].norm.params.text("bias_name") == ".b");
        CHECK(spec.lm_head.params.real("softcap") == 12.5 && spec.embedding.prefix == "embed" && spec.final_norm.prefix == "final.norm");
        auto listed = [&](const std::string& from, const std::string& to) {
            std::string text = kListed;
            const size_t at = text.find(from);
            if (at == std::string::npos) throw std::logic_error("the test's configuration has no " + from);
            text.replace(at, from.size(), to);
            return ArchitectureRegistry::instance().build(json::parse(text));
        };
        const std::string loop = "\"loop\": {\"start\": 1, \"stop\": 3, \"times\": 2},";
        CHECK(listed(loop, "").run_order.size() == 4 && listed(loop, "").stream_adds.empty());          // no loop: every layer once
        CHECK(listed(loop, "\"loop\": {\"start\": 0, \"stop\": 4, \"times\": 3},").run_order.size() == 12);
        CHECK(listed(loop, "\"loop\": {\"start\": 2, \"stop\": 2, \"times\": 3},").run_order.size() == 4);    // an empty run of layers
        CHECK(!listed("\"logit_softcap\": 12.5,", "").lm_head.params.has("softcap"));
        CHECK(throws<ConfigError>([&] { listed(loop, "\"loop\": {\"start\": 2, \"stop\": 5, \"times\": 2},"); }, "loop must have"));
        CHECK(throws<ConfigError>([&] { listed("\"width\": 40,", ""); }, "config.json lacks width"));
        CHECK(throws<ConfigError>([&] { listed("{\"eps\": 1e-5}", "{}"); }, "config.json lacks norm.eps"));
        CHECK(throws<ConfigError>([&] { listed("\"inner\": 48", "\"inner\": \"48\""); }, "layers[1].mixer.inner must be an integer"));
        CHECK(throws<ConfigError>([&] { listed("\"type\": \"mamba1\"", "\"type\": \"lstm\""); }, "is no mixer of this design"));
        // a parallel layer's sub-layers all have their norm in front
        ModelSpec bad = spec;
        bad.layers[1].sublayers[1].norm_placement = "post";
        CHECK(throws<std::invalid_argument>([&] { bad.validate(); }, "a parallel layer's sub-layers"));
        bad = spec;
        bad.run_order[2].stream_add = 3;
        CHECK(throws<std::invalid_argument>([&] { bad.validate(); }, "names stream addition 3"));
    }

    // ---- a fourth listed design: branches normed on their way back, masks of three kinds, two mixers side by side, shared tensors ----
    {
        const char* kMasks = R"({"architecture": "Mozalix", "vocab": 77, "width": 56, "norm": {"eps": 4e-6}, "embedding": {"scale": 0.25},
          "layers": [
            {"type": "attention_2", "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.2, "diff": 0.3, "mask": {"size": 21},
                                              "rot": {"base": 7000.0, "dims": 6}},
             "mlp": {"kind": "dense", "ff": 72, "limit": 2.25}},
            {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 4, "dim": 8, "vdim": 12, "scale": 0.35, "softcap": 11.0, "mask": {"size": 17, "keep_first": 3}},
                                           "right": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "conv": 3}, "left_scale": 0.75, "right_scale": 1.5},
             "mlp": null},
            {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.5, "mask": {"size": 13}}, "mlp": {"kind": "dense", "ff": 40, "limit": 1.0}},
            {"type": "parallel", "weights_of": 1,
             "mixer": {"left": {"heads": 4, "kv_heads": 4, "dim": 8, "vdim": 12, "scale": 0.35, "softcap": 11.0, "mask": {"size": 17, "keep_first": 3}},
                       "right": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "conv": 3}, "left_scale": 0.75, "right_scale": 1.5},
             "mlp": null},
            {"type": "attention_2", "weights_of": 0, "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.2, "diff": 0.3, "mask": {"size": 21},
                                                               "rot": {"base": 7000.0, "dims": 6}},
             "mlp": {"kind": "dense", "ff": 72, "limit": 2.25}}]})";
        const ModelSpec spec = ArchitectureRegistry::instance().build(json::parse(kMasks));
        // three layers have tensors; five run, each with a cache of its own
        CHECK(spec.architecture == "mozalix" && spec.layers.size() == 3 && spec.vocab_size == 77 && spec.hidden_size == 56 && spec.run_order.size() == 5);
        const int layers[] = {0, 1, 2, 1, 0};
        for (int i = 0; i < 5; ++i) CHECK(spec.run_order[i].layer == layers[i] && spec.run_order[i].cache == i && spec.run_order[i].writes_cache);
        CHECK(spec.embedding.params.real("scale") == 0.25 && spec.final_norm.params.real("offset") == 1.0 && spec.final_norm.prefix == "final.norm");
        // no norm in front of a branch, one with the gain kept as its distance from one behind it
        const SubLayerSpec& mix = spec.layers[0].sublayers[0];
        CHECK(!mix.norm.present && mix.output_norm.kind == "rmsnorm" && mix.output_norm.prefix == "l0.norm1" && mix.output_norm.params.real("offset") == 1.0 &&
              mix.output_norm.params.real("eps") == 4e-6 && !spec.layers[0].parallel);
        CHECK(mix.part.kind == "masked_attention" && mix.part.prefix == "l0.mix" && mix.part.params.integer("maps") == 2 && mix.part.params.integer("window") == 21 &&
              !mix.part.params.has("chunk") && mix.part.params.real("diff") == 0.3 && mix.part.params.text("qk_norm") == "gain" && mix.part.params.real("norm_eps") == 4e-6 &&
              mix.part.params.integer("heads") == 6 && mix.part.params.integer("kv_heads") == 2 && mix.part.params.integer("vdim") == 24);
        CHECK(spec.layers[0].position.present && spec.layers[0].position.params.integer("rotary_dim") == 6 && spec.layers[0].position.params.real("theta") == 7000.0);
        const SubLayerSpec& ff = spec.layers[0].sublayers[1];
        CHECK(ff.part.kind == "swiglu" && ff.part.params.text("activation") == "clamped" && ff.part.params.real("limit") == 2.25 && ff.part.params.flag("bias", false) &&
              ff.part.params.integer("intermediate_size") == 72 && ff.part.params.text("gate_bias_name") == ".gate.b" && !ff.norm.present &&
              ff.output_norm.prefix == "l0.norm2");
        // the two mixers side by side carry their own parameters, the sum's weights among them
        const PartSpec& both = spec.layers[1].sublayers[0].part;
        CHECK(spec.layers[1].sublayers.size() == 1 && both.kind == "side_by_side" && both.params.text("left_kind") == "masked_attention" &&
              both.params.text("right_kind") == "channel_delta");
        const Params left = both.params.sub("left."), right = both.params.sub("right.");
        CHECK(left.integer("window") == 17 && left.integer("keep_first") == 3 && left.real("softcap") == 11.0 && left.text("qk_norm") == "unit" &&
              left.real("out_scale") == 0.75 && !left.has("maps") && !left.has("sinks") && !spec.layers[1].position.present);
        CHECK(right.integer("heads") == 4 && right.integer("kv_heads") == 2 && right.integer("dim") == 12 && right.integer("vdim") == 20 && right.integer("conv") == 3 &&
              right.real("out_scale") == 1.5 && right.text("gate") == "sigmoid" && right.real("unit_eps") == 1e-6 && !right.has("rank"));
        const PartSpec& chunks = spec.layers[2].sublayers[0].part;
        CHECK(chunks.params.integer("chunk") == 13 && !chunks.params.has("window") && chunks.params.integer("sinks") == 1 && !spec.layers[2].position.present);
        auto changed = [&](const std::string& from, const std::string& to) {
            std::string text = kMasks;
            const size_t at = text.find(from);
            CHECK(at != std::string::npos);
            text.replace(at, from.size(), to);
            return text;
        };
        // no mask: all keys; no embedding entry: no scale
        const ModelSpec open_mask = ArchitectureRegistry::instance().build(json::parse(changed(R"(, "mask": {"size": 13})", "")));
        CHECK(!open_mask.layers[2].sublayers[0].part.params.has("chunk"));
        const ModelSpec unscaled = ArchitectureRegistry::instance().build(json::parse(changed(R"("embedding": {"scale": 0.25},)", "")));
        CHECK(!unscaled.embedding.params.has("scale"));
        for (const auto& wrong : {changed(R"("weights_of": 1)", R"("weights_of": 0)"), changed(R"("weights_of": 1)", R"("weights_of": 9)"),
                                  changed(R"("type": "attention",)", R"("type": "attention_3",)"), changed(R"("limit": 1.0)", R"("limit": 0)"),
                                  // the entry of a layer that runs another's tensors must equal that layer's (here the first of the two is changed)
                                  changed(R"("size": 17, "keep_first": 3)", R"("size": 18, "keep_first": 3)")}) {
            bool refused = false;
            try {
                ArchitectureRegistry::instance().build(json::parse(wrong));
            } catch (const std::exception&) {
                refused = true;
            }
            CHECK(refused);
        }
    }

    // ---- a third listed design: one norm a layer read by two branches side by side, a convolution in front of the mixer, a token input behind --
    {
        const char* kSide = R"({"architecture": "Masezen", "vocab": 91, "width": 40, "norm": {"eps": 3e-6}, "canon": {"taps": 5}, "token_side": {"dim": 7},
          "layers": [
            {"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 16, "vdim": 16, "scale": 0.25,
                                            "rot": {"base": 7000.0, "dims": 12, "scaling": {"factor": 2.0, "original": 128, "fast": 8.0, "slow": 2.0}}},
             "mlp": {"kind": "dense", "ff": 56}},
            {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "scale": 0.5},
             "mlp": {"kind": "moe", "router": {"experts": 5, "top": 3}, "expert": {"ff": 24, "limit": 2.5}, "shared": {"ff": 32, "limit": 1.25}}},
            {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 8, "scale": 0.3}, "mlp": null}]})";
        const ModelSpec spec = ArchitectureRegistry::instance().build(json::parse(kSide));
        CHECK(spec.architecture == "masezen" && spec.layers.size() == 3 && spec.vocab_size == 91 && spec.hidden_size == 40 && spec.run_order.size() == 3);
        const LayerSpec& first = spec.layers[0];
        CHECK(first.parallel && first.sublayers.size() == 3 && first.sequential_tail == 1);
        const SubLayerSpec& mix = first.sublayers[0];
        CHECK(mix.part.kind == "mixed_attention" && mix.part.prefix == "l0.mix" && mix.part.params.integer("heads") == 6 && mix.part.params.integer("kv_heads") == 3 &&
              mix.part.params.integer("dim") == 16 && mix.part.params.real("scale") == 0.25 && mix.part.params.real("norm_eps") == 3e-6);
        CHECK(mix.norm.kind == "rmsnorm" && mix.norm.prefix == "l0.norm1" && mix.norm.params.integer("single_gain") == 1 && mix.norm.params.real("eps") == 3e-6 &&
              mix.output_norm.present && mix.output_norm.kind == "layer_scale" && mix.output_norm.prefix == "l0.ls1");
        CHECK(mix.shift.present && mix.shift.kind == "conv_shift" && mix.shift.prefix == "l0.canon1" && mix.shift.params.integer("taps") == 5 &&
              mix.shift.params.integer("size") == 40);
        CHECK(first.position.present && first.position.params.integer("rotary_dim") == 12 && first.position.params.real("theta") == 7000.0 &&
              first.position.params.real("scaling_factor") == 2.0 && first.position.params.real("scaling_original") == 128.0);
        // the feed-forward has no norm of its own (it reads the mixer's), and a gain on its output
        const SubLayerSpec& ff = first.sublayers[1];
        CHECK(ff.part.kind == "squared_relu" && ff.part.prefix == "l0.mlp" && ff.part.params.integer("ff") == 56 && !ff.norm.present && !ff.shift.present &&
              ff.output_norm.kind == "layer_scale" && ff.output_norm.prefix == "l0.ls2");
        // every layer reads its own columns of the one table
        const SubLayerSpec& side = spec.layers[1].sublayers[2];
        CHECK(side.part.kind == "token_side" && side.part.prefix == "l1.side" && side.part.params.integer("side") == 7 && side.part.params.integer("column") == 7 &&
              side.part.params.integer("columns") == 21 && side.part.params.text("table") == "side.embed" && !side.norm.present &&
              side.output_norm.kind == "rmsnorm" && side.output_norm.prefix == "l1.side.norm");
        const PartSpec& routed = spec.layers[1].sublayers[1].part;
        CHECK(routed.kind == "routed_experts" && routed.params.integer("experts") == 5 && routed.params.integer("top") == 3 && routed.params.integer("ff") == 24 &&
              routed.params.real("limit") == 2.5 && routed.params.integer("weight_input") == 1 && routed.params.integer("shared_ff") == 32 &&
              routed.params.real("shared_limit") == 1.25 && routed.params.text("scoring") == "sigmoid");
        // no rotation where the keys say nothing of one; a layer without a feed-forward has the mixer and the token input
        CHECK(!spec.layers[1].position.present && spec.layers[2].sublayers.size() == 2 && spec.layers[2].sequential_tail == 1 &&
              spec.layers[2].sublayers[0].part.kind == "mixed_attention" && spec.layers[2].sublayers[1].part.kind == "token_side");
        auto changed = [&](const std::string& from, const std::string& to) {
            std::string text = kSide;
            const size_t at = text.find(from);
            CHECK(at != std::string::npos);
            text.replace(at, from.size(), to);
            return text;
        };
        // neither a convolution nor a token input: the layers are the two branches alone
        const ModelSpec bare = ArchitectureRegistry::instance().build(json::parse(changed(R"("canon": {"taps": 5}, "token_side": {"dim": 7},)", "")));
        CHECK(bare.layers[0].sublayers.size() == 2 && bare.layers[0].sequential_tail == 0 && !bare.layers[0].sublayers[0].shift.present);
        bool refused = false;
        try {
            ArchitectureRegistry::instance().build(json::parse(changed(R"("vdim": 16)", R"("vdim": 24)")));
        } catch (const std::exception&) {
            refused = true;
        }
        CHECK(refused);       // the values are the keys: another size for them is no model of this design
    }

    // ---- a second listed design: branches normed on both sides, a shift in front of the mixer, a loop without additions -----------
    {
        const char* kListed = R"({"architecture": "Lasizen", "vocab": 83, "width": 48, "norm": {"eps": 2e-6}, "embedding": {"scale": 3.0},
          "logit_scale": 0.5, "loop": {"start": 0, "stop": 2, "times": 3},
          "layers": [
            {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.2, "mask": {"size": 20},
                                            "rot": {"base": 5000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}}},
             "mlp": {"kind": "dense", "ff": 72}},
            {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "conv": 3}, "mlp": null},
            {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.35}, "mlp": {"kind": "dense", "ff": 40}}]})";
        const ModelSpec spec = ArchitectureRegistry::instance().build(json::parse(kListed));
        CHECK(spec.architecture == "lasizen" && spec.layers.size() == 3 && spec.vocab_size == 83 && spec.hidden_size == 48);
        // layers 0 and 1 three times in a row with a cache or state of their own each time, then layer 2; nothing is added between passes
        CHECK(spec.run_order.size() == 7 && spec.stream_adds.empty());
        const int layers[] = {0, 1, 0, 1, 0, 1, 2};
        for (size_t i = 0; i < spec.run_order.size(); ++i)
            CHECK(spec.run_order[i].layer == layers[i] && spec.run_order[i].cache == (int)i && spec.run_order[i].writes_cache && spec.run_order[i].stream_add < 0);
        const SubLayerSpec& mix = spec.layers[0].sublayers[0];
        CHECK(!spec.layers[0].parallel && spec.layers[0].sublayers.size() == 2 && spec.layers[1].sublayers.size() == 1);
        CHECK(mix.part.kind == "sink_attention" && mix.part.prefix == "l0.mix" && mix.part.params.integer("heads") == 6 && mix.part.params.integer("kv_heads") == 2 &&
              mix.part.params.integer("dim") == 16 && mix.part.params.integer("vdim") == 24 && mix.part.params.real("scale") == 0.2 &&
              mix.part.params.integer("window") == 20 && mix.part.params.real("sink_logit") == 0.0 && mix.part.params.real("unit_eps") == 2e-6);
        CHECK(mix.norm.kind == "rmsnorm" && mix.norm.prefix == "l0.norm1" && mix.norm.params.text("weight_name", "x") == "" && mix.norm_placement == "pre" &&
              mix.output_norm.present && mix.output_norm.prefix == "l0.norm1b" && mix.output_norm.params.real("eps") == 2e-6);
        CHECK(mix.shift.present && mix.shift.kind == "token_shift" && mix.shift.prefix == "l0.shift" && mix.shift.params.integer("size") == 48);
        const PartSpec& rope = spec.layers[0].position;
        CHECK(rope.present && rope.kind == "rope" && rope.params.integer("rotary_dim") == 8 && rope.params.integer("head_dim") == 16 && rope.params.real("theta") == 5000.0 &&
              rope.params.real("scaling_factor") == 4.0 && rope.params.real("scaling_original") == 64.0 && rope.params.real("scaling_fast") == 16.0 &&
              rope.params.real("scaling_slow") == 2.0);
        const SubLayerSpec& ff = spec.layers[0].sublayers[1];
        CHECK(ff.part.kind == "xielu" && ff.part.prefix == "l0.mlp" && ff.part.params.integer("ff") == 72 && ff.norm.prefix == "l0.norm2" &&
              ff.output_norm.prefix == "l0.norm2b" && !ff.shift.present);
        const PartSpec& delta = spec.layers[1].sublayers[0].part;
        CHECK(delta.kind == "gated_delta" && delta.params.integer("heads") == 4 && delta.params.integer("kv_heads") == 2 && delta.params.integer("dim") == 12 &&
              delta.params.integer("vdim") == 20 && delta.params.integer("conv") == 3 && delta.params.real("eps") == 2e-6 && delta.params.real("unit_eps") == 1e-6);
        CHECK(spec.layers[1].sublayers[0].shift.present && !spec.layers[1].position.present);
        // no window, no rotation: the keys say so by their absence
        CHECK(!spec.layers[2].sublayers[0].part.params.has("window") && !spec.layers[2].position.present);
        CHECK(spec.embedding.params.real("scale") == 3.0 && spec.lm_head.params.real("scale") == 0.5 && spec.embedding.prefix == "embed" &&
              spec.final_norm.kind == "rmsnorm" && spec.final_norm.prefix == "final.norm" && spec.lm_head.prefix == "head");
        auto listed = [&](const std::string& from, const std::string& to) {
            std::string text = kListed;
            const size_t at = text.find(from);
            if (at == std::string::npos) throw std::logic_error("the test's configuration has no " + from);
            text.replace(at, from.size(), to);
            return ArchitectureRegistry::instance().build(json::parse(text));
        };
        const std::string loop = "\"loop\": {\"start\": 0, \"stop\": 2, \"times\": 3},";
        CHECK(listed(loop, "").run_order.size() == 3);
        CHECK(listed(loop, "\"loop\": {\"start\": 1, \"stop\": 3, \"times\": 2},").run_order.size() == 5);
        CHECK(listed(loop, "\"loop\": {\"start\": 1, \"stop\": 1, \"times\": 4},").run_order.size() == 3);
        CHECK(!listed("\"logit_scale\": 0.5,", "").lm_head.params.has("scale"));
        CHECK(!listed(", \"scaling\": {\"factor\": 4.0, \"original\": 64, \"fast\": 16.0, \"slow\": 2.0}", "").layers[0].position.params.has("scaling_factor"));
        CHECK(throws<ConfigError>([&] { listed(loop, "\"loop\": {\"start\": 2, \"stop\": 1, \"times\": 2},"); }, "loop must have"));
        CHECK(throws<ConfigError>([&] { listed("\"heads\": 6", "\"heads\": 5"); }, "heads a multiple of kv_heads"));
        CHECK(throws<ConfigError>([&] { listed("\"dims\": 8", "\"dims\": 7"); }, "rot.dims must be even"));
        CHECK(throws<ConfigError>([&] { listed("\"conv\": 3", "\"conv\": 3.5"); }, "layers[1].mixer.conv must be an integer"));
        CHECK(throws<ConfigError>([&] { listed("\"kind\": \"dense\", \"ff\": 72", "\"kind\": \"moe\", \"ff\": 72"); }, "kind must be 'dense'"));
        CHECK(throws<ConfigError>([&] { listed("\"type\": \"delta\"", "\"type\": \"mamba1\""); }, "is no mixer of this design"));
        CHECK(throws<ConfigError>([&] { listed("{\"size\": 20}", "{\"size\": 0}"); }, "mask.size must be > 0"));
        // a shift belongs in front of a mixer, behind the norm in front of it
        ModelSpec bad = spec;
        bad.layers[0].sublayers[1].shift = bad.layers[0].sublayers[0].shift;
        CHECK(throws<std::invalid_argument>([&] { bad.validate(); }, "a shift stands in front of a mixer"));
    }

    if (failures) {
        std::printf("%d checks failed\n", failures);
        return 1;
    }
    std::printf("native engine, host side: all checks passed\n");
    return 0;
}
