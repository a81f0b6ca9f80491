// Routed feed-forward (mixture of experts): the feed-forward "routed_mlp".
//
//     z = W_r h (+ b_r)  [experts], float32;   the `top` experts with the largest z;   weights = softmax over the chosen z
//     y = sum over the chosen experts of weight * W_down,e ( act(W_gate,e h) * (W_up,e h) )
//
// Experts have no biases.  Their matrices are packed at load: gate and up rows of an expert in turn (row 2i the gate
// row and row 2i + 1 the up row of output i, so that a product's epilogue can apply the activation) in one
// [experts * 2 ff, hidden] matrix, the down matrices in one [experts * hidden, ff].  The tokens of a step are
// grouped by expert on the device (nothing of the routing comes back to the host), so a step launches the same
// kernels whatever the router decides.  Tensor names: `names` gives "router", "router_bias", the experts' prefix
// "expert" (followed by the expert's number and a dot) and "gate", "up", "down" below it.
//
// A second way to choose, `scoring` = "softmax_all": the scores are s = softmax(z) over ALL experts; the `top` experts
// with the largest s + correction are chosen (the correction, tensor "correction" [experts], present if
// `choice_correction`, never enters the weights); with `groups` {count, keep} the experts form `count` equal runs of
// adjacent experts (groups), a group's score is its largest corrected score, and only experts of the `keep` best groups can be
// chosen; the weights are the chosen experts' s, as they are unless `renormalize`.  `shared` {intermediate_size,
// activation, names} adds a gated feed-forward that every token goes through (a "gated_mlp" part below the prefix
// `shared_prefix`), its float32 output summed with the experts' in the kernel that combines them.
//
// A third way, `scoring` = "sigmoid": s_e = sigmoid(z_e), every expert by itself; choice, groups and weights as for
// softmax_all.  Three more parameters of the scored ways: `group_score_top` n (a group's score is the sum of its n largest
// choice scores; 1 if not given), `weight_scale` (the weights are multiplied by it at the end) and `sum_eps` (added to the
// sum the weights are divided by).  And one more activation of the experts, "swish_clamped" with `activation_limit` L:
// g = min(W_gate h, L), u = clamp(W_up h, -L, L), y = g sigmoid(1.702 g) (u + 1).
#include "parts/parts.h"

namespace illm {

namespace {

struct RoutedMLP : FeedForward {
    long long hidden, inter;
    int experts, top, act;
    bool has_bias;
    bool score_all, score_sigmoid, has_correction, renorm;
    int groups = 1, keep = 1, group_top = 1;
    float weight_scale = 1.f, sum_eps = 0.f, act_limit = 0.f;
    std::unique_ptr<FeedForward> shared;
    std::string shared_prefix;
    OwnedMat correction;
    std::map<std::string, std::string> names;
    DeviceBuffer gu_buf, down_buf;
    Mat w_gate_up, w_down;
    OwnedMat w_router, b_router;

    RoutedMLP(const PartSpec& s, Runtime* rt)
            : FeedForward(s, rt), hidden(s.get_int("hidden_size")), inter(s.get_int("intermediate_size")), experts((int)s.get_int("experts")),
              top((int)s.get_int("top")), act(ops::gate_act_from_name(s.get_string("activation", "silu"))), has_bias(s.get_bool("router_bias", false)),
              score_all(s.get_string("scoring", "softmax_chosen") == "softmax_all"), score_sigmoid(s.get_string("scoring", "softmax_chosen") == "sigmoid"),
              has_correction(s.get_bool("choice_correction", false)),
              renorm(s.get_bool("renormalize", false)), shared_prefix(s.get_string("shared_prefix", "shared.")) {
        const std::string sc = s.get_string("scoring", "softmax_chosen");
        if (sc != "softmax_chosen" && sc != "softmax_all" && sc != "sigmoid")
            throw ConfigError("routed_mlp: scoring '" + sc + "' is not supported (softmax_chosen, softmax_all, sigmoid)");
        const bool scored = score_all || score_sigmoid;
        if (!scored && (has_correction || s.has("groups") || s.has("group_score_top") || s.has("weight_scale") || s.has("sum_eps")))
            throw ConfigError("routed_mlp: a choice correction, groups, weight_scale and sum_eps need scoring = softmax_all or sigmoid");
        if (scored && has_bias) throw ConfigError("routed_mlp: scoring = " + sc + " takes a choice correction, not a router bias");
        group_top = (int)s.get_int("group_score_top", 1);
        weight_scale = (float)s.get_double("weight_scale", 1.0);
        sum_eps = (float)s.get_double("sum_eps", 0.0);
        if (group_top < 1 || group_top > 4) throw ConfigError("routed_mlp: group_score_top must be 1 to 4");
        if (act == ops::kActSwishClamped) {
            act_limit = (float)s.get_double("activation_limit");
            if (!(act_limit > 0.f)) throw ConfigError("routed_mlp: activation_limit must be positive");
        }
        if (s.has("groups")) {
            const Json& g = s.params.at("groups");
            if (!g.is_object() || !g.has("count") || !g.has("keep") || !g.at("count").is_int() || !g.at("keep").is_int())
                throw ConfigError("routed_mlp: groups must be {count, keep}");
            groups = (int)g.at("count").as_int();
            keep = (int)g.at("keep").as_int();
            if (groups < 1 || groups > 32 || s.get_int("experts") % groups || keep < 1 || keep > groups ||
                (long long)keep * (s.get_int("experts") / groups) < s.get_int("top"))
                throw ConfigError("routed_mlp: the experts must form 1 to 32 equal groups, and the groups kept must hold at least `top` experts");
        }
        if (s.has("shared")) {
            PartSpec sh("gated_mlp", s.params.at("shared"));
            sh.params.set("hidden_size", s.get_int("hidden_size"));
            sh.params.set("output_dtype", std::string("float32"));
            shared = build_feed_forward(sh, rt);
        }
        if (hidden <= 0 || inter <= 0 || experts <= 0 || top <= 0 || top > experts)
            throw ConfigError("routed_mlp: sizes must be positive and top at most the number of experts");
        if (act < 0) throw ConfigError("routed_mlp: activation '" + s.get_string("activation", "silu") + "' is not supported (silu, relu, gelu_tanh, swish_clamped)");
        names = {{"router", "router.weight"}, {"router_bias", "router.bias"}, {"correction", "correction"}, {"expert", "experts."}, {"gate", "gate_proj.weight"},
                 {"up", "up_proj.weight"}, {"down", "down_proj.weight"}};
        if (s.has("names"))
            for (auto& m : s.params.at("names").members()) names[m.first] = m.second.as_string();
    }
    std::string expert_tensor(int e, const char* role) const { return names.at("expert") + std::to_string(e) + "." + names.at(role); }
    TensorDecls tensors() const override {
        TensorDecls d = {{names.at("router"), TensorDecl{{(long long)experts, hidden}}}};
        if (has_bias) d.push_back({names.at("router_bias"), TensorDecl{{(long long)experts}}});
        if (has_correction) d.push_back({names.at("correction"), TensorDecl{{(long long)experts}}});
        for (int e = 0; e < experts; e++) {
            d.push_back({expert_tensor(e, "gate"), TensorDecl{{inter, hidden}}});
            d.push_back({expert_tensor(e, "up"), TensorDecl{{inter, hidden}}});
            d.push_back({expert_tensor(e, "down"), TensorDecl{{hidden, inter}}});
        }
        if (shared)
            for (auto& t : shared->tensors()) d.push_back({shared_prefix + t.first, t.second});
        return d;
    }
    void load(TensorSource& src) override {
        const size_t es = dtype_size(rt->dtype);
        w_router = fetch_owned(rt, src, names.at("router"), rt->dtype, "a router's matrix");
        if (has_bias) b_router = fetch_owned(rt, src, names.at("router_bias"), DType::F32, "a router's bias");
        if (has_correction) correction = fetch_owned(rt, src, names.at("correction"), DType::F32, "a router's choice correction");
        if (shared) {
            struct Below : TensorSource {
                TensorSource& src;
                std::string prefix;
                Below(TensorSource& s, std::string p) : src(s), prefix(std::move(p)) {}
                DType kept_dtype(const std::string& n) override { return src.kept_dtype(prefix + n); }
                void fetch_into(const std::string& n, void* dst, DType want, long long ld) override { src.fetch_into(prefix + n, dst, want, ld); }
                std::vector<long long> shape(const std::string& n) override { return src.shape(prefix + n); }
                bool has(const std::string& n) override { return src.has(prefix + n); }
            } below(src, shared_prefix);
            shared->load(below);
        }
        gu_buf = DeviceBuffer(rt->dev, (size_t)experts * 2 * inter * hidden * es, "the experts' packed gate/up matrices");
        down_buf = DeviceBuffer(rt->dev, (size_t)experts * hidden * inter * es, "the experts' down matrices");
        w_gate_up = Mat{gu_buf.get(), (long long)experts * 2 * inter, hidden, rt->dtype, (long long)experts * 2 * inter};
        w_down = Mat{down_buf.get(), (long long)experts * hidden, inter, rt->dtype, (long long)experts * hidden};
        for (int e = 0; e < experts; e++) {
            char* gu = (char*)w_gate_up.p + (size_t)e * 2 * inter * hidden * es;
            src.fetch_into(expert_tensor(e, "gate"), gu, rt->dtype, 2 * hidden);              // rows 2i
            src.fetch_into(expert_tensor(e, "up"), gu + (size_t)hidden * es, rt->dtype, 2 * hidden);  // rows 2i + 1
            src.fetch_into(expert_tensor(e, "down"), (char*)w_down.p + (size_t)e * hidden * inter * es, rt->dtype);
        }
    }
    MatOrPartials forward(const Mat& h, const StepContext& ctx, bool) override {
        Device& dev = *rt->dev;
        Mat logits = ops::linear(dev, rt->gemm, h, w_router.m, DType::F32, false).m;
        ops::MoeRouting route;
        route.scoring = score_all ? 1 : score_sigmoid ? 2 : 0;
        route.groups = groups;
        route.keep = keep;
        route.group_top = group_top;
        route.weight_scale = weight_scale;
        route.sum_eps = sum_eps;
        route.act_limit = act_limit;
        route.renorm = (score_all || score_sigmoid) ? renorm : true;
        route.bias = has_bias ? (const float*)b_router.m.p : has_correction ? (const float*)correction.m.p : nullptr;
        Mat plus;
        if (shared) {
            plus = shared->forward(h, ctx, false).m;
            route.plus = &plus;
        }
        MatOrPartials r;
        r.m = ops::moe_forward_ex(dev, h, logits, route, experts, top, w_gate_up, w_down, act);
        return r;
    }
};

}  // namespace

void register_routed_parts(std::map<std::string, PartFactory<FeedForward>>& ffs) {
    ffs["routed_mlp"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<FeedForward>(new RoutedMLP(s, rt)); };
}

}  // namespace illm
