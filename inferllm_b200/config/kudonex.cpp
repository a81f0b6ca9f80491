#include "config/kudonex.h"

#include <cmath>

namespace illm {

namespace {
const Json& need_obj(const Json& d, const std::string& key, const std::string& where) {
    if (!d.is_object() || !d.has(key) || !d.at(key).is_object()) throw ConfigError("config.json: " + where + "'" + key + "' must be an object");
    return d.at(key);
}
bool given(const Json& d, const std::string& key) { return d.is_object() && d.has(key) && !d.at(key).is_null(); }
Json obj(std::initializer_list<std::pair<const char*, Json>> kv) {
    Json o = Json::object();
    for (auto& p : kv) o.set(p.first, p.second);
    return o;
}
Json name_map(std::initializer_list<std::pair<const char*, const char*>> kv) {
    Json o = Json::object();
    for (auto& p : kv) o.set(p.first, std::string(p.second));
    return o;
}
// The sinusoid position vector's base is fixed by the design.
constexpr double kSinusoidBase = 10000.0;
}  // namespace

std::unique_ptr<ArchConfig> KudonexConfig::from_json(const Json& d) {
    std::unique_ptr<KudonexConfig> c(new KudonexConfig);
    c->raw = d;
    c->width = take_int(d, "width");
    c->vocab = take_int(d, "vocab");
    c->max_positions = take_int(d, "max_positions", 131072);
    c->norm_eps = take_double(need_obj(d, "norm", ""), "eps", 1e-5);
    if (given(d, "embedding")) c->embedding_scale = take_double(need_obj(d, "embedding", ""), "scale", 1.0);
    if (given(d, "canon")) {
        c->canon_taps = take_int(need_obj(d, "canon", ""), "taps");
        if (c->canon_taps < 1) throw ConfigError("config.json: canon.taps must be at least 1");
    }
    if (c->width <= 0 || c->vocab <= 0 || c->max_positions <= 0) throw ConfigError("config.json: width, vocab and max_positions must be positive");
    if (!(c->norm_eps > 0)) throw ConfigError("config.json: norm.eps must be positive");
    if (!d.has("layers") || !d.at("layers").is_array() || d.at("layers").size() == 0)
        throw ConfigError("config.json: 'layers' must be a list with at least one layer");
    c->model_spec();        // every layer is checked now, not at the first use
    return std::unique_ptr<ArchConfig>(c.release());
}

ModelSpec KudonexConfig::model_spec() const {
    ModelSpec s;
    s.hidden_size = width;
    s.vocab_size = vocab;
    s.max_positions = max_positions;
    const Json& layers = raw.at("layers");
    size_t i = 0;
    auto norm = [&](bool f32_out) {
        Json p = obj({{"size", width}, {"eps", norm_eps}, {"tensor", std::string("")}});
        if (f32_out) p.set("output_dtype", std::string("float32"));
        return PartSpec("layernorm", p);
    };
    for (const Json& L : layers.items()) {
        const std::string where = "layer " + std::to_string(i) + ": ";
        if (!L.is_object()) throw ConfigError("config.json: " + where + "must be an object");
        const std::string type = take_string(L, "type", "");
        const Json& m = need_obj(L, "mixer", where);
        LayerSpec l;
        l.prefix = "l" + std::to_string(i) + ".";
        const bool has_ffn = given(L, "mlp");
        l.block = has_ffn ? "sandwich" : "sandwich_mixer";
        l.names = {{"mixer", "mix."}, {"ffn", "mlp."}, {"norm1", "norm1"}, {"norm1b", "norm1b"}, {"norm2", "norm2"}, {"norm2b", "norm2b"}};
        // the input convolution reads the normed rows in float32
        l.norms["norm1"] = norm(canon_taps > 0);
        l.norms["norm1b"] = norm(false);
        if (has_ffn) {
            l.norms["norm2"] = norm(false);
            l.norms["norm2b"] = norm(false);
        }
        const long long heads = take_int(m, "heads");
        PartSpec mixer;
        if (type == "mlstm") {
            // the matrix memory with exponential input and forget gates (soft-capped), a running maximum that starts
            // at 0, a normaliser state, per-head unit RMS, a weight over all heads and a sigmoid gate
            Json p = obj({{"hidden_size", width}, {"n_heads", heads}, {"head_dim", take_int(m, "dim")}, {"v_head_dim", take_int(m, "vdim")},
                          {"gate_cap", take_double(m, "gate_cap", 0.0)}, {"norm_eps", norm_eps}, {"output_dtype", std::string("float32")},
                          {"names", name_map({{"q", "q"}, {"k", "k"}, {"v", "v"}, {"gate", "g"}, {"o", "o"}, {"norm", "norm"}, {"i", "i"},
                                              {"i_bias", "i.b"}, {"f", "f"}, {"f_bias", "f.b"}})}});
            mixer = PartSpec("mlstm", p);
        } else if (type == "mamba2") {
            // the selective state space with a scalar decay per head: one input matrix [z | x | B | C | dt], a short
            // convolution with bias and silu over x, B and C, heads sharing B and C in groups, a skip weight per head,
            // the silu(z) gate before an RMS norm in equal parts
            Json p = obj({{"hidden_size", width}, {"n_heads", heads}, {"v_head_dim", take_int(m, "vdim")}, {"state", take_int(m, "state")},
                          {"groups", take_int(m, "groups", 1)}, {"norm_groups", take_int(m, "norm_groups", 1)}, {"conv", take_int(m, "conv", 1)},
                          {"norm_eps", norm_eps}, {"output_dtype", std::string("float32")},
                          {"names", name_map({{"in", "in"}, {"conv", "conv"}, {"conv_bias", "conv.b"}, {"dt_bias", "dt_bias"}, {"a_log", "A_log"},
                                              {"skip", "D"}, {"norm", "norm"}, {"o", "o"}})}});
            mixer = PartSpec("mamba2", p);
        } else if (type == "attention") {
            // softmax attention over a sliding window without any rotation: the values are the keys, a logarithmic
            // distance term is subtracted from the scores, the heads' scores are mixed before the softmax, and a full-width
            // sigmoid gate multiplies the concatenated heads
            const long long dim = take_int(m, "dim"), vdim = take_int(m, "vdim", dim);
            if (vdim != dim) throw ConfigError("config.json: " + where + "the values are the keys, so vdim must equal dim");
            long long window = 0;
            if (given(m, "mask")) {
                window = take_int(need_obj(m, "mask", where), "size", 0);
                if (window < 0) throw ConfigError("config.json: " + where + "mask.size must not be negative");
            }
            Json p = obj({{"hidden_size", width}, {"n_heads", heads}, {"n_kv_heads", take_int(m, "kv_heads", heads)}, {"head_dim", dim},
                          {"v_head_dim", vdim}, {"window", window}, {"scale", take_double(m, "scale", 1.0 / std::sqrt((double)dim))},
                          {"values", std::string("keys")}, {"distance_bias", std::string("log1p")}, {"head_mix", true},
                          {"out_gate", std::string("sigmoid")}, {"output_dtype", std::string("float32")},
                          {"position", PartSpec("none", Json::object()).to_json()},
                          {"names", name_map({{"q", "q"}, {"k", "k"}, {"o", "o"}, {"gate", "g"}, {"r1", "r1"}, {"r2", "r2"}, {"mix", "talk"}})}});
            mixer = PartSpec("attention", p);
        } else {
            throw ConfigError("config.json: " + where + "unknown type '" + type + "' (mlstm, mamba2, attention)");
        }
        if (canon_taps > 0) {
            // what the mixer reads is h + conv(h); the wrapper owns the layer's tensor beside the mixer's prefix
            l.names["mixer"] = "";
            l.mixer = PartSpec("input_conv", obj({{"width", width}, {"taps", canon_taps}, {"tensor", std::string("canon1")},
                                                  {"inner_prefix", std::string("mix.")}, {"inner", mixer.to_json()}}));
        } else {
            l.mixer = mixer;
        }
        if (has_ffn) {
            const Json& mlp = need_obj(L, "mlp", where);
            const std::string kind = take_string(mlp, "kind", "moe");
            if (kind != "moe") throw ConfigError("config.json: " + where + "mlp.kind '" + kind + "' is not supported (moe)");
            const Json& router = need_obj(mlp, "router", where);
            Json p = obj({{"hidden_size", width}, {"intermediate_size", take_int(need_obj(mlp, "expert", where), "ff")},
                          {"experts", take_int(router, "experts")}, {"top", take_int(router, "top")}, {"activation", std::string("silu")},
                          {"scoring", std::string("softmax_all")}, {"choice_correction", true}, {"renormalize", false},
                          {"names", name_map({{"router", "router"}, {"correction", "correction"}, {"expert", "e"}, {"gate", "gate"}, {"up", "up"},
                                              {"down", "down"}})}});
            if (given(router, "groups")) {
                const Json& g = need_obj(router, "groups", where);
                p.set("groups", obj({{"count", take_int(g, "count")}, {"keep", take_int(g, "keep")}}));
            }
            if (given(mlp, "shared")) {
                p.set("shared", obj({{"intermediate_size", take_int(need_obj(mlp, "shared", where), "ff")}, {"activation", std::string("silu")},
                                     {"names", name_map({{"gate", "gate"}, {"up", "up"}, {"down", "down"}})}}));
                p.set("shared_prefix", std::string("shared."));
            }
            l.ffn = PartSpec("routed_mlp", p);
        }
        s.layers.push_back(l);
        i++;
    }
    for (int k = 0; k < (int)s.layers.size(); k++) s.schedule.push_back(ScheduleEntry{k, k, true, false});
    s.embedding = PartSpec("embedding", obj({{"name", std::string("embed")}, {"tensor", std::string("")}, {"vocab_size", vocab}, {"hidden_size", width},
                                             {"scale", embedding_scale}, {"sinusoid_base", kSinusoidBase}}));
    s.final_norm = PartSpec("layernorm", obj({{"name", std::string("final.norm")}, {"tensor", std::string("")}, {"size", width}, {"eps", norm_eps}}));
    s.head = PartSpec("lm_head", obj({{"name", std::string("head")}, {"tensor", std::string("")}, {"tied", true}, {"vocab_size", vocab},
                                      {"hidden_size", width}}));
    return s;
}

void register_kudonex_architecture() { register_architecture("Kudonex", &KudonexConfig::from_json, {"kudonex"}); }

}  // namespace illm
