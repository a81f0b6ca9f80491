#include "config/tukulorn.h"

#include <cmath>

namespace illm {

namespace {
const Json& need_obj(const Json& d, const std::string& key, const std::string& where) {
    if (!d.is_object() || !d.has(key) || !d.at(key).is_object()) throw ConfigError("config.json: " + where + "'" + key + "' must be an object");
    return d.at(key);
}
bool given(const Json& d, const std::string& key) { return d.is_object() && d.has(key) && !d.at(key).is_null(); }
double need_number(const Json& d, const std::string& key, const std::string& where) {
    if (!d.is_object() || !d.has(key) || !d.at(key).is_number()) throw ConfigError("config.json: " + where + "'" + key + "' must be a number");
    return d.at(key).as_double();
}
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
}  // namespace

std::unique_ptr<ArchConfig> TukulornConfig::from_json(const Json& d) {
    std::unique_ptr<TukulornConfig> c(new TukulornConfig);
    c->raw = d;
    c->width = take_int(d, "width");
    c->vocab = take_int(d, "vocab");
    c->max_positions = take_int(d, "max_positions", 131072);
    c->norm_eps = take_double(need_obj(d, "norm", ""), "eps", 1e-6);
    if (c->width <= 0 || c->vocab <= 0 || c->max_positions <= 0) throw ConfigError("config.json: width, vocab and max_positions must be positive");
    if (!(c->norm_eps > 0)) throw ConfigError("config.json: norm.eps must be positive");
    if (!d.has("layers") || !d.at("layers").is_array() || d.at("layers").size() == 0)
        throw ConfigError("config.json: 'layers' must be a list with at least one layer");
    if (given(d, "loop")) {
        const Json& l = need_obj(d, "loop", "");
        c->has_loop = true;
        c->loop_start = take_int(l, "start");
        c->loop_stop = take_int(l, "stop");
        c->loop_times = take_int(l, "times", 1);
        const long long n = (long long)d.at("layers").size();
        if (c->loop_start < 0 || c->loop_stop <= c->loop_start || c->loop_stop > n || c->loop_times < 1)
            throw ConfigError("config.json: loop needs 0 <= start < stop <= the number of layers and times >= 1");
    }
    c->model_spec();        // every layer is checked now, not at the first use
    return std::unique_ptr<ArchConfig>(c.release());
}

ModelSpec TukulornConfig::model_spec() const {
    ModelSpec s;
    s.hidden_size = width;
    s.vocab_size = vocab;
    s.max_positions = max_positions;
    // RMS norm whose weight is stored around zero: x / sqrt(mean(x^2) + eps) * (1 + w)
    auto norm = [&]() {
        return PartSpec("rmsnorm", obj({{"size", width}, {"eps", norm_eps}, {"weight_offset", 1.0}, {"tensor", std::string("")}}));
    };
    auto layer_scale = [&]() { return PartSpec("layer_scale", obj({{"size", width}, {"tensor", std::string("")}})); };
    const Json& layers = raw.at("layers");
    size_t i = 0;
    for (const Json& L : layers.items()) {
        const std::string where = "layer " + std::to_string(i) + ": ";
        if (!L.is_object()) throw ConfigError("config.json: " + where + "must be an object");
        const std::string type = take_string(L, "type", "");
        const Json& m = need_obj(L, "mixer", where);
        const bool has_mlp = given(L, "mlp");
        LayerSpec l;
        l.prefix = "l" + std::to_string(i) + ".";
        l.block = has_mlp ? "prenorm_scaled" : "prenorm_scaled_mixer";
        l.names = {{"mixer", "mix."}, {"ffn", "mlp."}, {"norm1", "norm1"}, {"ls1", "ls1"}};
        l.norms["norm1"] = norm();
        l.norms["ls1"] = layer_scale();
        if (has_mlp) {
            l.names["norm2"] = "norm2";
            l.names["ls2"] = "ls2";
            l.norms["norm2"] = norm();
            l.norms["ls2"] = layer_scale();
        }
        const long long heads = take_int(m, "heads"), dim = take_int(m, "dim"), vdim = take_int(m, "vdim");
        if (heads <= 0 || dim <= 0 || vdim <= 0) throw ConfigError("config.json: " + where + "heads, dim and vdim must be positive");
        const double scale = need_number(m, "scale", where);
        if (type == "attention") {
            // differential attention: two score maps per head over the same values, o = a1 - lambda a2 with one lambda for the
            // layer, a unit norm per head and the factor 1 - diff; biases on q, k, v and the output; no rotation; the queries
            // grow with the position by steps (the temperature); causal, all earlier positions (or `mask.size` of them)
            const long long kvh = take_int(m, "kv_heads", heads);
            if (kvh <= 0 || heads % kvh) throw ConfigError("config.json: " + where + "heads must be a multiple of kv_heads");
            long long window = 0;
            if (given(m, "mask")) {
                window = take_int(need_obj(m, "mask", where), "size", 0);
                if (window < 0) throw ConfigError("config.json: " + where + "mask.size must not be negative");
            }
            Json p = obj({{"hidden_size", width}, {"n_heads", heads}, {"n_kv_heads", kvh}, {"head_dim", dim}, {"v_head_dim", vdim}, {"window", window},
                          {"scale", scale}, {"norm_eps", norm_eps}, {"qkv_bias", true}, {"o_bias", true}, {"score_maps", 2},
                          {"diff", need_number(m, "diff", where)}, {"output_dtype", std::string("float32")},
                          {"position", PartSpec("none", Json::object()).to_json()},
                          {"names", name_map({{"q", "q"}, {"k", "k"}, {"v", "v"}, {"o", "o"}, {"q_bias", "q.b"}, {"k_bias", "k.b"}, {"v_bias", "v.b"},
                                              {"o_bias", "o.b"}, {"lq1", "lq1"}, {"lk1", "lk1"}, {"lq2", "lq2"}, {"lk2", "lk2"}})}});
            if (given(m, "q_temp")) {
                const Json& qt = need_obj(m, "q_temp", where);
                const long long every = take_int(qt, "every");
                if (every < 1) throw ConfigError("config.json: " + where + "q_temp.every must be at least 1");
                p.set("q_temperature", obj({{"coef", need_number(qt, "coef", where + "q_temp: ")}, {"every", every}}));
            }
            l.mixer = PartSpec("attention", p);
        } else if (type == "latent_attention") {
            // attention whose keys and values are maps of one normed latent per token (the only thing cached, beside one
            // rotated key part that all heads share); queries straight from the input, `dim` channels against the latent's keys
            // and `rot_dim` rotated channels against the shared part; a sliding window; a sigmoid gate per head
            const long long kv_rank = take_int(m, "kv_rank"), rot_dim = take_int(m, "rot_dim", 0);
            if (kv_rank <= 0 || rot_dim < 0) throw ConfigError("config.json: " + where + "kv_rank must be positive and rot_dim not negative");
            long long window = 0;
            if (given(m, "mask")) {
                window = take_int(need_obj(m, "mask", where), "size", 0);
                if (window < 0) throw ConfigError("config.json: " + where + "mask.size must not be negative");
            }
            Json p = obj({{"hidden_size", width}, {"n_heads", heads}, {"head_dim", dim}, {"v_head_dim", vdim}, {"q_rank", 0}, {"kv_rank", kv_rank},
                          {"rot_head_dim", rot_dim}, {"window", window}, {"scale", scale}, {"norm_eps", norm_eps}, {"out_gate", std::string("head_sigmoid")},
                          {"output_dtype", std::string("float32")},
                          {"names", name_map({{"q", "q"}, {"kv_down", "dkv"}, {"kv_norm", "dkv.norm"}, {"k_up", "uk"}, {"v_up", "uv"}, {"gate", "g"},
                                              {"o", "o"}})}});
            if (rot_dim > 0) {
                const Json& rot = need_obj(m, "rot", where);
                const long long dims = take_int(rot, "dims", rot_dim);
                const double base = need_number(rot, "base", where + "rot: ");
                if (dims <= 0 || dims % 2 || dims > rot_dim) throw ConfigError("config.json: " + where + "rot.dims must be even and at most rot_dim");
                if (!(base > 0)) throw ConfigError("config.json: " + where + "rot.base must be positive");
                p.set("position", PartSpec("rope_pairs", obj({{"head_dim", rot_dim}, {"rot_dim", dims}, {"theta", base}, {"max_positions", max_positions}}))
                                      .to_json());
            }
            l.mixer = PartSpec("latent_attention", p);
        } else {
            throw ConfigError("config.json: " + where + "unknown type '" + type + "' (attention, latent_attention)");
        }
        if (has_mlp) {
            const Json& mlp = need_obj(L, "mlp", where);
            const std::string kind = take_string(mlp, "kind", "dense");
            if (kind == "dense") {
                l.ffn = PartSpec("gated_mlp", obj({{"hidden_size", width}, {"intermediate_size", take_int(mlp, "ff")}, {"activation", std::string("silu")},
                                                   {"output_dtype", std::string("float32")},
                                                   {"names", name_map({{"gate", "gate"}, {"up", "up"}, {"down", "down"}})}}));
            } else if (kind == "moe") {
                // sigmoid scores; a group's score is the sum of its two largest; weights over their sum (+ 1e-20) times router.scale;
                // experts with the clamped activation
                const Json& router = need_obj(mlp, "router", where);
                const Json& ex = need_obj(mlp, "expert", where);
                Json p = obj({{"hidden_size", width}, {"intermediate_size", take_int(ex, "ff")}, {"experts", take_int(router, "experts")},
                              {"top", take_int(router, "top")}, {"scoring", std::string("sigmoid")}, {"renormalize", true}, {"sum_eps", 1e-20},
                              {"weight_scale", take_double(router, "scale", 1.0)}, {"group_score_top", 2},
                              {"activation", std::string("swish_clamped")}, {"activation_limit", need_number(ex, "limit", where + "expert: ")},
                              {"names", name_map({{"router", "router"}, {"expert", "e"}, {"gate", "gate"}, {"up", "up"}, {"down", "down"}})}});
                if (given(router, "groups")) {
                    const Json& g = need_obj(router, "groups", where);
                    p.set("groups", obj({{"count", take_int(g, "count")}, {"keep", take_int(g, "keep")}}));
                }
                l.ffn = PartSpec("routed_mlp", p);
            } else {
                throw ConfigError("config.json: " + where + "mlp.kind '" + kind + "' is not supported (dense, moe)");
            }
        }
        s.layers.push_back(l);
        i++;
    }
    // the order of execution: the looped layers run `times` times, every pass with cache entries of its own; every pass but
    // the first begins by adding the embedding output to the stream
    const long long n = (long long)s.layers.size();
    int cache = 0;
    auto run = [&](long long layer, bool reenter) { s.schedule.push_back(ScheduleEntry{(int)layer, cache++, true, reenter}); };
    if (!has_loop) {
        for (long long k = 0; k < n; k++) run(k, false);
    } else {
        for (long long k = 0; k < loop_start; k++) run(k, false);
        for (long long pass = 0; pass < loop_times; pass++)
            for (long long k = loop_start; k < loop_stop; k++) run(k, pass > 0 && k == loop_start);
        for (long long k = loop_stop; k < n; k++) run(k, false);
        if (loop_times > 1) s.reentry = PartSpec("add_embedding", Json::object());
    }
    s.embedding = PartSpec("embedding", obj({{"name", std::string("embed")}, {"tensor", std::string("")}, {"vocab_size", vocab}, {"hidden_size", width}}));
    s.final_norm = PartSpec("rmsnorm", obj({{"name", std::string("final.norm")}, {"tensor", std::string("")}, {"size", width}, {"eps", norm_eps},
                                            {"weight_offset", 1.0}}));
    s.head = PartSpec("lm_head", obj({{"name", std::string("head")}, {"tensor", std::string("")}, {"tied", false}, {"vocab_size", vocab},
                                      {"hidden_size", width}}));
    return s;
}

void register_tukulorn_architecture() { register_architecture("Tukulorn", &TukulornConfig::from_json, {"tukulorn"}); }

}  // namespace illm
