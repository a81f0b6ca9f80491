// Parts of a block that norms every sublayer on both sides:
//
//     x <- x + norm1b(mixer(norm1(x)));   x <- x + norm2b(ffn(norm2(x)))
//
// "layernorm": the norm with a weight and no bias, (v - mean) / sqrt(mean squared deviation + eps) * w, float32.
// It can stand in front of a sublayer (Norm::forward) and behind one (add_normed_pending); where one of each follow
// one another (a sublayer's output norm, then the next sublayer's input norm) both run in one kernel.
//
// "sandwich" / "sandwich_mixer": the block above, with and without a feed-forward.
//
// "input_conv": a mixer around another mixer: what the inner mixer reads is h + conv(h), a causal convolution over
// time with one filter of `taps` taps per channel (tensor `tensor` [width, taps], no bias).  The last taps - 1 rows of
// h are per-sequence state: the part asks for a second cache entry beside the inner mixer's own.  It takes h in
// float32 (its norm's `output_dtype`), convolves in float32 and hands the inner mixer the compute dtype.
#include "parts/parts.h"

namespace illm {

namespace {

struct LayerNorm : Norm {
    long long size;
    float eps;
    std::string tensor;
    bool out_f32;
    OwnedMat weight;
    LayerNorm(const PartSpec& s, Runtime* rt)
            : Norm(s, rt), size(s.get_int("size")), eps((float)s.get_double("eps")), tensor(s.get_string("tensor", "weight")),
              out_f32(s.get_string("output_dtype", "compute") == "float32") {
        if (size <= 0 || !(eps > 0)) throw ConfigError("layernorm: size and eps must be positive");
    }
    TensorDecls tensors() const override { return {{tensor, TensorDecl{{size}, "norm"}}}; }
    void load(TensorSource& src) override { weight = fetch_owned(rt, src, tensor, DType::F32, "a norm weight"); }
    DType out_dtype() const { return out_f32 ? DType::F32 : rt->dtype; }

    Mat forward(ResidualStream& stream, const int* rows, long long n_rows) override {
        // a sublayer's output that still has to pass a layer norm of its own on its way into the stream is normed,
        // added and normed again here; anything else that is pending is added first
        LayerNorm* post = stream.has_pending && !stream.has_pending2 ? dynamic_cast<LayerNorm*>(stream.pending_post) : nullptr;
        if (post && !stream.pending.is_partials() && stream.pending.m.dtype == DType::F32 && post->eps == eps) {
            Mat y = ops::layernorm_sandwich(*rt->dev, stream.x, &stream.pending.m, &post->weight.m, &weight.m, eps, out_dtype(), rows, n_rows);
            if (rows == nullptr) {
                stream.has_pending = false;
                stream.pending_post = nullptr;
            }
            return y;
        }
        if (stream.has_pending || stream.has_pending2) stream.flush();
        return ops::layernorm_sandwich(*rt->dev, stream.x, nullptr, nullptr, &weight.m, eps, out_dtype(), rows, n_rows);
    }
    void add_normed_pending(ResidualStream& stream) override {
        Mat y = stream.pending.is_partials() ? ops::materialize(*rt->dev, stream.pending.part, DType::F32) : ops::cast(*rt->dev, stream.pending.m, DType::F32);
        ops::layernorm_sandwich(*rt->dev, stream.x, &y, &weight.m, nullptr, eps, DType::F32, nullptr, 0);
        stream.has_pending = false;
    }
};

struct SandwichBlock : Block {
    void forward(ResidualStream& stream, const StepContext& ctx, const CacheView& cache, bool writes) override {
        Mat h = norms.at("norm1")->forward(stream, nullptr, 0);
        stream.add_normed(mixer->forward(h, ctx, cache, writes, false), norms.at("norm1b"));
        if (!ffn) return;
        h = norms.at("norm2")->forward(stream, nullptr, 0);
        stream.add_normed(ffn->forward(h, ctx, false), norms.at("norm2b"));
    }
};

// the tensors of an inner part, below a prefix
struct PrefixedSource : TensorSource {
    TensorSource& src;
    std::string prefix;
    PrefixedSource(TensorSource& s, std::string p) : src(s), prefix(std::move(p)) {}
    DType kept_dtype(const std::string& name) override { return src.kept_dtype(prefix + name); }
    void fetch_into(const std::string& name, void* dst, DType want, long long ld) override { src.fetch_into(prefix + name, dst, want, ld); }
    std::vector<long long> shape(const std::string& name) override { return src.shape(prefix + name); }
    bool has(const std::string& name) override { return src.has(prefix + name); }
};

struct InputConv : Mixer {
    long long width;
    int taps;
    std::string tensor, inner_prefix;
    std::unique_ptr<Mixer> inner;
    OwnedMat w;
    InputConv(const PartSpec& s, Runtime* rt)
            : Mixer(s, rt), width(s.get_int("width")), taps((int)s.get_int("taps")), tensor(s.get_string("tensor", "conv.weight")),
              inner_prefix(s.get_string("inner_prefix", "inner.")), inner(build_mixer(s.get_part("inner"), rt)) {
        if (width <= 0 || taps < 1) throw ConfigError("input_conv: width and taps must be positive");
        if (inner->aux_cache_request().kind != CacheRequest::None) throw ConfigError("input_conv: the inner mixer must not ask for a second cache entry");
    }
    bool graph_safe() const override { return inner->graph_safe(); }
    bool pad_safe() const override { return false; }       // tokens behind the real ones would enter the convolution's rows
    CacheRequest cache_request() const override { return inner->cache_request(); }
    CacheRequest aux_cache_request() const override {
        return taps > 1 ? CacheRequest::state({(long long)taps - 1, width}, DType::F32) : CacheRequest();
    }
    TensorDecls tensors() const override {
        TensorDecls d = {{tensor, TensorDecl{{width, (long long)taps}}}};
        for (auto& t : inner->tensors()) d.push_back({inner_prefix + t.first, t.second});
        return d;
    }
    void load(TensorSource& src) override {
        w = fetch_owned(rt, src, tensor, DType::F32, "an input convolution's taps");
        PrefixedSource below(src, inner_prefix);
        inner->load(below);
    }
    MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool may_defer) override {
        if (taps > 1 && !cache.has_aux) throw EngineError("input_conv: the layer has no cache entry for the convolution's rows");
        if (!writes) throw EngineError("input_conv: the convolution's rows belong to one layer");
        Device& dev = *rt->dev;
        Mat hf = ops::cast(dev, h, DType::F32);
        Mat y = ops::new_mat(dev, h.rows, h.cols, rt->dtype);
        ops::ShortConv p;
        p.C = (int)width;
        p.taps = taps;
        p.w = (const float*)w.m.p;
        p.residual = true;
        ops::short_conv(dev, hf, p, ctx, cache.aux, y, 0);
        CacheView below = cache;
        below.has_aux = false;
        return inner->forward(y, ctx, below, writes, may_defer);
    }
};

}  // namespace

void register_sandwich_parts(std::map<std::string, PartFactory<Norm>>& norms, std::map<std::string, PartFactory<Mixer>>& mixers,
                             std::map<std::string, BlockKind>& blocks) {
    norms["layernorm"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Norm>(new LayerNorm(s, rt)); };
    mixers["input_conv"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new InputConv(s, rt)); };
    blocks["sandwich"] = BlockKind{{"norm1", "norm1b", "norm2", "norm2b"}, [] { return std::unique_ptr<Block>(new SandwichBlock); }};
    blocks["sandwich_mixer"] = BlockKind{{"norm1", "norm1b"}, [] { return std::unique_ptr<Block>(new SandwichBlock); }};
}

}  // namespace illm
