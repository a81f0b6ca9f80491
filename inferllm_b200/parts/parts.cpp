#include "parts/parts.h"

#include <cmath>

namespace illm {

void register_decay_parts(std::map<std::string, PartFactory<Mixer>>& mixers);      // parts/decay_mixer.cpp
void register_delta_parts(std::map<std::string, PartFactory<Mixer>>& mixers);      // parts/delta_mixer.cpp
void register_latent_parts(std::map<std::string, PartFactory<Mixer>>& mixers);     // parts/latent_mixer.cpp
void register_routed_parts(std::map<std::string, PartFactory<FeedForward>>& ffs);  // parts/routed_mlp.cpp
void register_gated_state_parts(std::map<std::string, PartFactory<Mixer>>& mixers);   // parts/gated_mixers.cpp
void register_sandwich_parts(std::map<std::string, PartFactory<Norm>>& norms, std::map<std::string, PartFactory<Mixer>>& mixers,
                             std::map<std::string, BlockKind>& blocks);               // parts/sandwich.cpp

// ---- registries

namespace {
template <typename T> std::map<std::string, PartFactory<T>>& reg() {
    static std::map<std::string, PartFactory<T>> r;
    return r;
}
std::map<std::string, BlockKind>& block_reg() {
    static std::map<std::string, BlockKind> r;
    return r;
}
void register_builtin_parts();
void ensure_builtin() {
    static bool done = false;
    if (!done) {
        done = true;
        register_builtin_parts();
    }
}
template <typename T> std::unique_ptr<T> build(const char* family, const PartSpec& s, Runtime* rt) {
    ensure_builtin();
    auto it = reg<T>().find(s.kind);
    if (it == reg<T>().end()) {
        std::string known;
        for (auto& k : reg<T>()) known += (known.empty() ? "" : ", ") + k.first;
        throw ConfigError(std::string("unknown ") + family + " kind '" + s.kind + "'; registered: " + known);
    }
    return it->second(s, rt);
}
}  // namespace

void register_mixer(const std::string& kind, PartFactory<Mixer> f) { ensure_builtin(); reg<Mixer>()[kind] = std::move(f); }
void register_feed_forward(const std::string& kind, PartFactory<FeedForward> f) { ensure_builtin(); reg<FeedForward>()[kind] = std::move(f); }
void register_norm(const std::string& kind, PartFactory<Norm> f) { ensure_builtin(); reg<Norm>()[kind] = std::move(f); }
void register_position(const std::string& kind, PartFactory<PositionEncoding> f) { ensure_builtin(); reg<PositionEncoding>()[kind] = std::move(f); }
void register_embedding(const std::string& kind, PartFactory<EmbeddingPart> f) { ensure_builtin(); reg<EmbeddingPart>()[kind] = std::move(f); }
void register_head(const std::string& kind, PartFactory<HeadPart> f) { ensure_builtin(); reg<HeadPart>()[kind] = std::move(f); }
void register_block(const std::string& kind, BlockKind k) { ensure_builtin(); block_reg()[kind] = std::move(k); }

void unregister_part(const std::string& family, const std::string& kind) {
    ensure_builtin();
    if (family == "mixer") reg<Mixer>().erase(kind);
    else if (family == "feed_forward") reg<FeedForward>().erase(kind);
    else if (family == "norm") reg<Norm>().erase(kind);
    else if (family == "position") reg<PositionEncoding>().erase(kind);
    else if (family == "embedding") reg<EmbeddingPart>().erase(kind);
    else if (family == "head") reg<HeadPart>().erase(kind);
    else if (family == "block") block_reg().erase(kind);
    else throw ConfigError("unknown family of parts '" + family + "'");
}
std::vector<std::string> registered_parts(const std::string& family) {
    ensure_builtin();
    std::vector<std::string> out;
    auto names = [&](auto& m) { for (auto& k : m) out.push_back(k.first); };
    if (family == "mixer") names(reg<Mixer>());
    else if (family == "feed_forward") names(reg<FeedForward>());
    else if (family == "norm") names(reg<Norm>());
    else if (family == "position") names(reg<PositionEncoding>());
    else if (family == "embedding") names(reg<EmbeddingPart>());
    else if (family == "head") names(reg<HeadPart>());
    else if (family == "block") names(block_reg());
    else throw ConfigError("unknown family of parts '" + family + "'");
    return out;
}

std::unique_ptr<Mixer> build_mixer(const PartSpec& s, Runtime* rt) { return build<Mixer>("mixer", s, rt); }
std::unique_ptr<FeedForward> build_feed_forward(const PartSpec& s, Runtime* rt) { return build<FeedForward>("feed_forward", s, rt); }
std::unique_ptr<Norm> build_norm(const PartSpec& s, Runtime* rt) { return build<Norm>("norm", s, rt); }
std::unique_ptr<PositionEncoding> build_position(const PartSpec& s, Runtime* rt) { return build<PositionEncoding>("position", s, rt); }
std::unique_ptr<EmbeddingPart> build_embedding(const PartSpec& s, Runtime* rt) { return build<EmbeddingPart>("embedding", s, rt); }
std::unique_ptr<HeadPart> build_head(const PartSpec& s, Runtime* rt) { return build<HeadPart>("head", s, rt); }
const BlockKind& lookup_block(const std::string& kind) {
    ensure_builtin();
    auto it = block_reg().find(kind);
    if (it == block_reg().end()) {
        std::string known;
        for (auto& k : block_reg()) known += (known.empty() ? "" : ", ") + k.first;
        throw ConfigError("unknown block kind '" + kind + "'; registered: " + known);
    }
    return it->second;
}

OwnedMat fetch_owned(Runtime* rt, TensorSource& src, const std::string& name, DType want, const char* what) {
    std::vector<long long> shape = src.shape(name);
    OwnedMat o;
    o.m.rows = shape.size() >= 2 ? shape[0] : 1;
    o.m.cols = shape.empty() ? 1 : shape.back();
    if (shape.size() > 2)
        for (size_t i = 1; i + 1 < shape.size(); i++) o.m.rows *= shape[i];
    o.m.rows_held = o.m.rows;
    o.m.dtype = want;
    o.buf = DeviceBuffer(rt->dev, (size_t)o.m.rows * o.m.cols * dtype_size(want), what);
    o.m.p = o.buf.get();
    src.fetch_into(name, o.m.p, want, 0);
    return o;
}

std::vector<double> rotary_frequencies(double theta, int rot_dim, const Json* scaling, double* magnitude) {
    const int half = rot_dim / 2;
    std::vector<double> f((size_t)half);
    for (int j = 0; j < half; j++) f[j] = std::pow(theta, -2.0 * j / rot_dim);
    *magnitude = 1.0;
    if (!scaling || !scaling->is_object()) return f;
    auto num = [&](const char* key) {
        if (!scaling->has(key) || !scaling->at(key).is_number()) throw ConfigError(std::string("rotary scaling: '") + key + "' must be a number");
        return scaling->at(key).as_double();
    };
    const double factor = num("factor"), original = num("original"), fast = num("fast"), slow = num("slow");
    if (!(factor > 0) || !(original > 0) || !(fast > 0) || !(slow > 0)) throw ConfigError("rotary scaling: all four numbers must be positive");
    // the (real-valued) pair index whose wave turns `turns` times within `original` positions
    auto pair_of = [&](double turns) { return rot_dim * std::log(original / (2.0 * M_PI * turns)) / (2.0 * std::log(theta)); };
    const double lo = std::max(std::floor(pair_of(fast)), 0.0), hi = std::min(std::ceil(pair_of(slow)), (double)rot_dim - 1.0);
    for (int j = 0; j < half; j++) {
        const double ramp = std::min(1.0, std::max(0.0, ((double)j - lo) / std::max(hi - lo, 0.001)));
        f[j] = f[j] / factor * ramp + f[j] * (1.0 - ramp);
    }
    *magnitude = 0.1 * std::log(factor) + 1.0;
    return f;
}

std::shared_ptr<PositionTable> shared_position_table(Runtime* rt, double theta, int rot_dim, long long positions) {
    double one;
    return shared_position_table(rt, rotary_frequencies(theta, rot_dim, nullptr, &one), 1.0, positions);
}

std::shared_ptr<PositionTable> shared_position_table(Runtime* rt, const std::vector<double>& freqs, double magnitude, long long positions) {
    std::string key = std::to_string(positions);
    char word[40];
    snprintf(word, sizeof word, "/%.17g", magnitude);
    key += word;
    for (double f : freqs) {
        snprintf(word, sizeof word, "/%.17g", f);
        key += word;
    }
    auto it = rt->position_tables.find(key);
    if (it != rt->position_tables.end()) return it->second;
    const int half = (int)freqs.size(), rot_dim = 2 * half;
    std::vector<float> host((size_t)positions * half * 2);
    for (long long p = 0; p < positions; p++)
        for (int j = 0; j < half; j++) {
            const double ang = (double)p * freqs[j];
            host[((size_t)p * half + j) * 2] = (float)(std::cos(ang) * magnitude);
            host[((size_t)p * half + j) * 2 + 1] = (float)(std::sin(ang) * magnitude);
        }
    auto t = std::make_shared<PositionTable>();
    t->positions = positions;
    t->rot_dim = rot_dim;
    t->buf = DeviceBuffer(rt->dev, host.size() * sizeof(float), "a position table");
    check_cuda(cudaMemcpyAsync(t->buf.get(), host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice, rt->dev->stream()),
               "uploading a position table");
    rt->dev->synchronize();        // `host` goes away
    rt->position_tables[key] = t;
    return t;
}

// ---- the parts of the LLaMA decoder

namespace {

// RMSNorm with a weight, fused with the residual addition that precedes it.  Formula of the reference
// (src/kern/naive/naive.cpp:186-207, weight multiply :138-149): y = x / sqrt(mean(x^2) + eps) * w.  The
// reference fixes eps in code (1e-6 in the layers, src/graph/llama_like.cpp:77-78; 1e-5 in the head,
// src/core/graph.h:160-163); here it is a parameter of the part.
//
// Three parameters beyond the reference's norm: `weight_offset` (a weight stored as w - offset, e.g.
// around zero for offset 1; the offset is added once, in float32, when the weight is loaded),
// `residual_scale` (the factor on the stream in the norm-after-the-sum arrangement, see
// forward_into_stream) and `tensor` (the weight's name below the part's prefix, "weight" if not given).
struct RMSNorm : Norm {
    long long size;
    float eps, weight_offset, residual_scale;
    std::string tensor;
    bool optional, absent = false;
    OwnedMat weight;
    RMSNorm(const PartSpec& s, Runtime* rt)
            : Norm(s, rt), size(s.get_int("size")), eps((float)s.get_double("eps")), weight_offset((float)s.get_double("weight_offset", 0.0)),
              residual_scale((float)s.get_double("residual_scale", 1.0)), tensor(s.get_string("tensor", "weight")),
              optional(s.get_bool("optional", false)) {
        if (size <= 0 || !(eps > 0)) throw ConfigError("rmsnorm: size and eps must be positive");
    }
    bool keeps_f32() const { return weight_offset != 0.f || spec.get_bool("float32_weight", false); }
    TensorDecls tensors() const override {
        TensorDecl d{{size}, weight_offset == 1.f ? "matrix" : "norm"};
        d.optional = optional;
        return {{tensor, d}};
    }
    bool present() const override { return !absent; }
    void load(TensorSource& src) override {
        if (optional && !src.has(tensor)) {        // `optional`: the file may leave the weight out, and the norm with it
            absent = true;
            return;
        }
        if (!keeps_f32()) {
            // a weight stored in 32-bit stays 32-bit; bfloat16 stays bfloat16 (the kernel takes both)
            weight = fetch_owned(rt, src, tensor, src.kept_dtype(tensor), "a norm weight");
            return;
        }
        weight = fetch_owned(rt, src, tensor, DType::F32, "a norm weight");
        if (weight_offset != 0.f) {
            std::vector<float> host((size_t)size);
            rt->dev->synchronize();
            check_cuda(cudaMemcpy(host.data(), weight.m.p, host.size() * sizeof(float), cudaMemcpyDeviceToHost), "reading a norm weight");
            for (float& v : host) v = weight_offset + v;
            check_cuda(cudaMemcpy(weight.m.p, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice), "writing a norm weight");
        }
    }
    Mat forward_into_stream(ResidualStream& stream) override {
        if (stream.has_pending2) stream.flush();
        if (weight.m.dtype != DType::F32) throw EngineError("rmsnorm: the norm after the sum needs its weight in float32 (float32_weight)");
        const MatOrPartials* d = stream.has_pending ? &stream.pending : nullptr;      // unreduced slices are added up by the kernel
        stream.has_pending = false;
        return ops::scale_add_rmsnorm(*rt->dev, stream.x, d, weight.m, residual_scale, eps, rt->dtype);
    }
    Mat forward(ResidualStream& stream, const int* rows, long long n_rows) override {
        // an addition that passes a layer scale on its way into the stream: x + factors * pending and the norm in one kernel
        if (stream.has_pending && stream.pending_post) {
            const Mat* ls = stream.pending_post->channel_scale();
            if (ls && rows == nullptr && !stream.has_pending2 && !stream.pending.is_partials() && stream.pending.m.dtype == DType::F32 &&
                weight.m.dtype == DType::F32) {
                Mat y = ops::scaled_add_rmsnorm(*rt->dev, stream.x, stream.pending.m, (const float*)ls->p, &weight.m, eps, rt->dtype);
                stream.has_pending = false;
                stream.pending_post = nullptr;
                return y;
            }
            stream.flush();
        }
        // float32 additions (one or two finished matrices) fold into one kernel with the norm; what that kernel does not
        // take (a second addition otherwise, a float32 addition beside a 16-bit output, gathered rows) is added first
        const bool f32_pending = stream.has_pending && !stream.pending.is_partials() && stream.pending.m.dtype == DType::F32;
        if (f32_pending && rows == nullptr && weight.m.dtype == DType::F32 &&
            (!stream.has_pending2 || (!stream.pending2.is_partials() && stream.pending2.m.dtype == DType::F32))) {
            Mat y = ops::add2_rmsnorm(*rt->dev, stream.x, stream.pending.m, stream.has_pending2 ? &stream.pending2.m : nullptr, weight.m, eps, rt->dtype);
            stream.has_pending = stream.has_pending2 = false;
            return y;
        }
        if (stream.has_pending2 || (f32_pending && rt->dtype != DType::F32)) stream.flush();
        Mat y = ops::add_rmsnorm(*rt->dev, stream.x, stream.has_pending ? &stream.pending : nullptr, weight.m, eps, rt->dtype, rows, n_rows,
                                 rows == nullptr);
        if (rows == nullptr) stream.has_pending = false;
        return y;
    }
};

// "layer_scale": a learned factor per channel on a sublayer's output before it joins the stream, x <- x + s * f(..).  It
// stands where a block puts a norm behind a sublayer (ResidualStream::add_normed); the next RMS norm folds it into its
// own kernel (channel_scale), flush() applies it alone.  `tensor`: the factors' name below the part's prefix.
struct LayerScale : Norm {
    long long size;
    std::string tensor;
    OwnedMat factors;
    LayerScale(const PartSpec& s, Runtime* rt) : Norm(s, rt), size(s.get_int("size")), tensor(s.get_string("tensor", "weight")) {
        if (size <= 0) throw ConfigError("layer_scale: size must be positive");
    }
    TensorDecls tensors() const override { return {{tensor, TensorDecl{{size}, "norm"}}}; }
    void load(TensorSource& src) override { factors = fetch_owned(rt, src, tensor, DType::F32, "a layer scale"); }
    const Mat* channel_scale() const override { return &factors.m; }
    Mat forward(ResidualStream&, const int*, long long) override { throw EngineError("layer_scale: stands behind a sublayer, not in front of one"); }
    void add_normed_pending(ResidualStream& stream) override {
        Mat y = stream.pending.is_partials() ? ops::materialize(*rt->dev, stream.pending.part, DType::F32) : ops::cast(*rt->dev, stream.pending.m, DType::F32);
        ops::scaled_add_rmsnorm(*rt->dev, stream.x, y, (const float*)factors.m.p, nullptr, 0.f, DType::F32);
        stream.has_pending = false;
    }
};

// "rope_half" is the reference's RotMode::ModelRotHalf (src/kern/naive/naive.cpp:389-414): pair
// (j, j + rot/2) of every Q and K head is rotated by the angle p * theta^(-2j/rot).  The reference
// computes the trigonometry per element (in double on the CPU, with powf/sinf/cosf on the GPU,
// src/kern/gpu/kernel_gpu.cu:343-371); here a table [position, rot/2, (cos, sin)] is computed once in
// float64 and stored in float32, and the rotation is done in float32 inside the kernel that also
// writes K and V into the cache.  theta (fixed to 10000 in the reference) and rot_dim are parameters.
//
// "rope_pairs" is the same rotation with channel 2j paired with 2j + 1 (the interleaved layout).  Both
// take an optional `scaling` {factor, original, fast, slow}: the frequencies are blended with the
// stretched ones and cos and sin carry a magnitude factor (rotary_frequencies).
struct RopeTable : PositionEncoding {
    int head_dim, rot_dim;
    double theta, magnitude = 1.0;
    long long max_positions;
    bool pairs, scaled;
    std::vector<double> freqs;
    std::shared_ptr<PositionTable> table;
    RopeTable(const PartSpec& s, Runtime* rt, bool pairs_)
            : PositionEncoding(s, rt), head_dim((int)s.get_int("head_dim")), rot_dim((int)s.get_int("rot_dim", s.get_int("head_dim"))),
              theta(s.get_double("theta")), max_positions(s.get_int("max_positions")), pairs(pairs_), scaled(s.has("scaling")) {
        if (rot_dim % 2 || rot_dim <= 0 || rot_dim > head_dim)
            throw ConfigError(s.kind + ": rot_dim " + std::to_string(rot_dim) + " must be even and in (0, head_dim]");
        if (!(theta > 0) || max_positions <= 0) throw ConfigError(s.kind + ": theta and max_positions must be positive");
        const Json* sc = scaled ? &s.params.at("scaling") : nullptr;
        freqs = rotary_frequencies(theta, rot_dim, sc, &magnitude);
    }
    bool takes_partials() const override { return !pairs; }
    void prepare() override { table = shared_position_table(rt, freqs, magnitude, max_positions); }
    bool rotation_table(const float** t, int* rot, long long* n_pos) const override {
        if (pairs) return false;
        *t = table ? table->data() : nullptr;
        *rot = rot_dim;
        *n_pos = max_positions;
        return true;
    }
    bool table_rotation(const float** t, int* rot, long long* n_pos, bool* is_pairs) const override {
        *t = table ? table->data() : nullptr;
        *rot = rot_dim;
        *n_pos = max_positions;
        *is_pairs = pairs;
        return true;
    }
    Mat encode_and_store(const MatOrPartials& qkv, ops::Geometry g, const StepContext& ctx, const KVView& kv) override {
        if (!pairs) return ops::rope_kv_write(*rt->dev, qkv, table->data(), rot_dim, max_positions, ctx, kv, g);
        ops::QkPrep p;
        p.q_off = 0;
        p.k_off = g.n_heads * g.head_dim;
        p.v_off = (g.n_heads + g.n_kv_heads) * g.head_dim;
        p.cos_sin = table->data();
        p.rot_dim = rot_dim;
        p.pairs = true;
        p.n_pos = max_positions;
        return ops::qk_prep(*rt->dev, qkv.is_partials() ? ops::materialize(*rt->dev, qkv.part, rt->dtype) : qkv.m, p, g, ctx, kv, rt->dtype);
    }
};

// "none" encodes nothing and only stores K and V.
struct NoPosition : PositionEncoding {
    using PositionEncoding::PositionEncoding;
    bool takes_partials() const override { return true; }
    bool rotation_table(const float** t, int* rot, long long* n_pos) const override {
        *t = nullptr;
        *rot = 0;
        *n_pos = 0;
        return true;
    }
    Mat encode_and_store(const MatOrPartials& qkv, ops::Geometry g, const StepContext& ctx, const KVView& kv) override {
        if (kv.writes) return ops::rope_kv_write(*rt->dev, qkv, nullptr, 0, 0, ctx, kv, g);
        return qkv.is_partials() ? ops::materialize(*rt->dev, qkv.part, rt->dtype) : qkv.m;
    }
};

// Causal self-attention with grouped heads over the paged cache: the mixer of LLaMA.
//
// Order of operations of the reference's LlamaAttention::execute (src/core/op.cpp:348-500): Q, K, V
// projections without bias; position encoding of Q and of the new K rows; K and V go into the cache;
// scores of every query against all cached keys of its sequence, scaled by 1/sqrt(head size) (:488)
// and masked causally; softmax; weighted values; then the output projection (AttentionModule,
// src/core/graph.h:106-111).  The reference has separate [H, H] matrices and one KV head per query
// head (src/core/op.h:327-332); here the three matrices are stacked into one
// [(heads + 2 kv heads) * d, H] at load so that one product feeds the rotation kernel, and the number
// of KV heads, the head size and an optional window are parameters.
//
// Options beyond the reference's attention, each a parameter that is off unless given: `v_head_dim`
// (values of another size than keys), `qkv_bias` (biases on the three projections), `qk_norm` =
// "projection" (an RMS norm with a weight over the token's whole q projection, all heads together, and
// likewise over k, before the rotation; `norm_eps`), `sink` (one learned number per head whose
// exponential joins the softmax denominator without a value), `out_gate` = "head_sigmoid" (a
// projection of the mixer's input to one number per head; the head's output is multiplied by its
// sigmoid before the output projection), `own_kv` = false (the layer has no key and value
// projections and attends to the keys and values another layer wrote into the cache entry it
// reads), `scale`, `output_dtype` = "float32" (the output projection is not rounded to the compute
// dtype, for a block that adds it to a float32 stream itself) and `names` (the tensors' names below
// the part's prefix).  With any of the first six the layer takes the general path: one float32
// product for q, k, v and the gate, one kernel for biases, norms, rotation and the cache write
// (ops::qk_prep), and the general attention kernel, which knows sinks, gates and value sizes.
//
// A second family of options changes the scores themselves and takes a kernel of its own (ops::attention_mixed):
// `values` = "keys" (there is no value projection: the values are the keys as projected, and the cache entry keeps
// keys only), `distance_bias` = "log1p" (r1_h ln(1 + r2_h (i - j)) is subtracted from the score of query i and key j; two
// numbers per head, tensors "r1" and "r2"), `head_mix` = true (before the softmax the heads' scores are mixed,
// score_h <- sum_g M[h, g] score_g, tensor "mix" [heads, heads]) and `out_gate` = "sigmoid" (a full-width gate
// projection of the mixer's input; the concatenated heads are multiplied by its sigmoid element by element).  The
// last three need the first.
//
// A third family: `score_maps` = 2 (differential attention: a head's query row is [q_1, q_2] and a key head's row
// [k_1, k_2], `head_dim` the size of ONE map; both maps are softmax attentions of their own over the same values and
// o = a_1 - lambda a_2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + `diff`, four vectors of head_dim entries and one
// number for the layer, made once at load; then o / sqrt(mean(o^2) + norm_eps) over the head's values, times 1 - diff;
// ops::attention_diff), `q_temperature` {coef, every} (the queries of position p are multiplied by
// 1 + coef ln(floor((p + 1) / every) + 1), behind the bias) and `o_bias` (a bias on the output projection).
struct Attention : Mixer {
    long long hidden;
    int n_heads, n_kv_heads, head_dim, v_head_dim, window;
    float scale, norm_eps;
    bool qkv_bias, proj_norm, has_sink, has_gate, own_kv, out_f32;
    bool values_are_keys, log_distance, head_mix, wide_gate;
    int maps = 1;                     // score maps per head (2: differential attention)
    bool o_bias = false;
    float diff = 0.f, lambda = 0.f, q_temp_coef = 0.f;
    int q_temp_every = 0;
    std::map<std::string, std::string> names;
    std::unique_ptr<PositionEncoding> position;
    DeviceBuffer qkv_buf, o_buf;
    Mat w_qkv, w_o;
    OwnedMat b_q, b_k, b_v, b_o, n_q, n_k, sinks, dist_r1, dist_r2, mix;
    Attention(const PartSpec& s, Runtime* rt)
            : Mixer(s, rt), hidden(s.get_int("hidden_size")), n_heads((int)s.get_int("n_heads")), n_kv_heads((int)s.get_int("n_kv_heads")),
              head_dim((int)s.get_int("head_dim")), v_head_dim((int)s.get_int("v_head_dim", s.get_int("head_dim"))),
              window((int)s.get_int("window", 0)), norm_eps((float)s.get_double("norm_eps", 1e-6)), qkv_bias(s.get_bool("qkv_bias", false)),
              proj_norm(s.get_string("qk_norm", "none") == "projection"), has_sink(s.get_bool("sink", false)),
              has_gate(s.get_string("out_gate", "none") == "head_sigmoid"), own_kv(s.get_bool("own_kv", true)),
              out_f32(s.get_string("output_dtype", "compute") == "float32"), values_are_keys(s.get_string("values", "own") == "keys"),
              log_distance(s.get_string("distance_bias", "none") == "log1p"), head_mix(s.get_bool("head_mix", false)),
              wide_gate(s.get_string("out_gate", "none") == "sigmoid") {
        if (hidden <= 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || v_head_dim <= 0 || window < 0)
            throw ConfigError("attention: sizes must be positive");
        if (n_heads % n_kv_heads) throw ConfigError("attention: n_heads must be a multiple of n_kv_heads");
        const std::string qn = s.get_string("qk_norm", "none"), og = s.get_string("out_gate", "none");
        if (qn != "none" && qn != "projection") throw ConfigError("attention: qk_norm '" + qn + "' is not supported (none, projection)");
        if (og != "none" && og != "head_sigmoid" && og != "sigmoid")
            throw ConfigError("attention: out_gate '" + og + "' is not supported (none, head_sigmoid, sigmoid)");
        const std::string vs = s.get_string("values", "own"), db = s.get_string("distance_bias", "none");
        if (vs != "own" && vs != "keys") throw ConfigError("attention: values '" + vs + "' is not supported (own, keys)");
        if (db != "none" && db != "log1p") throw ConfigError("attention: distance_bias '" + db + "' is not supported (none, log1p)");
        if ((log_distance || head_mix || wide_gate) && !values_are_keys)
            throw ConfigError("attention: distance_bias, head_mix and the element-wise gate run on the kernel for values = keys only");
        if (values_are_keys && (v_head_dim != head_dim || !own_kv || qkv_bias || proj_norm || has_sink || has_gate))
            throw ConfigError("attention: values = keys needs key and value heads of one size and takes no biases, projection norms, sinks or head gates");
        maps = (int)s.get_int("score_maps", 1);
        o_bias = s.get_bool("o_bias", false);
        if (maps != 1 && maps != 2) throw ConfigError("attention: score_maps must be 1 or 2");
        if (maps == 2) {
            diff = (float)s.get_double("diff");
            if (values_are_keys || has_sink || has_gate || !own_kv)
                throw ConfigError("attention: two score maps take no sinks and no head gates, and need keys and values of their own");
        }
        if (s.has("q_temperature")) {
            const Json& qt = s.params.at("q_temperature");
            if (!qt.is_object() || !qt.has("coef") || !qt.has("every") || !qt.at("coef").is_number() || !qt.at("every").is_int() || qt.at("every").as_int() < 1)
                throw ConfigError("attention: q_temperature must be {coef, every} with every >= 1");
            if (values_are_keys) throw ConfigError("attention: values = keys takes no query temperature");
            q_temp_coef = (float)qt.at("coef").as_double();
            q_temp_every = (int)qt.at("every").as_int();
        }
        if (rt && values_are_keys && !ops::attention_mixed_supported(rt->dtype, n_heads, n_kv_heads, head_dim))
            throw ConfigError("attention: " + std::to_string(n_heads) + " heads of " + std::to_string(head_dim) +
                              " channels are beyond the kernel for mixed scores (heads x head size up to 8192)");
        names = {{"q", "q_proj.weight"}, {"k", "k_proj.weight"}, {"v", "v_proj.weight"}, {"o", "o_proj.weight"},
                 {"q_bias", "q_proj.bias"}, {"k_bias", "k_proj.bias"}, {"v_bias", "v_proj.bias"}, {"q_norm", "q_norm.weight"},
                 {"k_norm", "k_norm.weight"}, {"sink", "sinks"}, {"gate", "gate_proj.weight"}, {"r1", "r1"}, {"r2", "r2"}, {"mix", "mix"},
                 {"o_bias", "o_proj.bias"}, {"lq1", "lambda_q1"}, {"lk1", "lambda_k1"}, {"lq2", "lambda_q2"}, {"lk2", "lambda_k2"}};
        if (s.has("names"))
            for (auto& m : s.params.at("names").members()) names[m.first] = m.second.as_string();
        // the attention kernels read heads 16 bytes at a time: said when the model is built, not at its first step
        if (rt && !general() && !values_are_keys && head_dim % 8)
            throw ConfigError("attention: head size " + std::to_string(head_dim) +
                              " is not supported by the kernels (multiples of 8 up to " + std::to_string(ops::kMaxHeadDimGeneric) + ")");
        if (rt && (head_dim > ops::kMaxHeadDimGeneric || v_head_dim > ops::kMaxHeadDimGeneric) && !(head_dim == 64 || head_dim == 128))
            throw ConfigError("attention: head size " + std::to_string(head_dim) + " is not supported by the kernels (up to " +
                              std::to_string(ops::kMaxHeadDimGeneric) + ")");
        scale = s.has("scale") ? (float)s.get_double("scale") : (float)(1.0 / std::sqrt((double)head_dim));
        position = build_position(s.get_part("position"), rt);
        if (rt) position->prepare();
    }
    // true if the layer needs the general path (see above)
    bool general() const {
        return v_head_dim != head_dim || qkv_bias || proj_norm || has_sink || has_gate || !own_kv || out_f32 || maps == 2 || q_temp_every > 0 || o_bias;
    }
    long long gate_rows() const { return has_gate ? n_heads : wide_gate ? (long long)n_heads * v_head_dim : 0; }
    bool graph_safe() const override { return true; }     // a decode step's launches depend only on the batch size
    // Causal attention: tokens behind a sequence's real ones are seen by none of them.  Said only for
    // the plain case: no window, and a position encoding that is nothing but the table rotation (any
    // other runs code of its own, which is not known to launch the same kernels).
    bool pad_safe() const override {
        const float* t;
        int rot;
        long long n;
        return window == 0 && !values_are_keys && position->rotation_table(&t, &rot, &n);
    }
    TensorDecls tensors() const override {
        const long long q = (long long)n_heads * maps * head_dim, k = (long long)n_kv_heads * maps * head_dim, v = (long long)n_kv_heads * v_head_dim;
        const long long o = (long long)n_heads * v_head_dim;
        TensorDecls d;
        auto nm = [&](const char* role) { return names.at(role); };
        d.push_back({nm("q"), TensorDecl{{q, hidden}}});
        if (qkv_bias) d.push_back({nm("q_bias"), TensorDecl{{q}}});
        if (own_kv) {
            d.push_back({nm("k"), TensorDecl{{k, hidden}}});
            if (qkv_bias) d.push_back({nm("k_bias"), TensorDecl{{k}}});
            if (!values_are_keys) d.push_back({nm("v"), TensorDecl{{v, hidden}}});
            if (qkv_bias) d.push_back({nm("v_bias"), TensorDecl{{v}}});
        }
        if (proj_norm) {
            d.push_back({nm("q_norm"), TensorDecl{{q}, "norm"}});
            if (own_kv) d.push_back({nm("k_norm"), TensorDecl{{k}, "norm"}});
        }
        if (has_sink) d.push_back({nm("sink"), TensorDecl{{(long long)n_heads}}});
        if (has_gate || wide_gate) d.push_back({nm("gate"), TensorDecl{{gate_rows(), hidden}}});
        if (log_distance) {
            d.push_back({nm("r1"), TensorDecl{{(long long)n_heads}}});
            d.push_back({nm("r2"), TensorDecl{{(long long)n_heads}}});
        }
        if (head_mix) d.push_back({nm("mix"), TensorDecl{{(long long)n_heads, (long long)n_heads}}});
        if (maps == 2)
            for (const char* role : {"lq1", "lk1", "lq2", "lk2"}) d.push_back({nm(role), TensorDecl{{(long long)head_dim}}});
        d.push_back({nm("o"), TensorDecl{{hidden, o}}});
        if (o_bias) d.push_back({nm("o_bias"), TensorDecl{{hidden}}});
        return d;
    }
    // rows of the packed matrix: q, then k and v (a layer with keys and values of its own), then the gate
    long long q_rows() const { return (long long)n_heads * maps * head_dim; }
    long long k_rows() const { return own_kv ? (long long)n_kv_heads * maps * head_dim : 0; }
    long long v_rows() const { return own_kv && !values_are_keys ? (long long)n_kv_heads * v_head_dim : 0; }
    long long packed_rows() const { return q_rows() + k_rows() + v_rows() + gate_rows(); }
    void load(TensorSource& src) override {
        const long long q = q_rows(), k = k_rows(), v = v_rows(), all = packed_rows();
        const size_t es = dtype_size(rt->dtype);
        qkv_buf = DeviceBuffer(rt->dev, (size_t)all * hidden * es, "the packed Q/K/V matrix");
        w_qkv = Mat{qkv_buf.get(), all, hidden, rt->dtype, all};
        src.fetch_into(names.at("q"), w_qkv.p, rt->dtype);
        if (own_kv) {
            src.fetch_into(names.at("k"), (char*)w_qkv.p + (size_t)q * hidden * es, rt->dtype);
            if (!values_are_keys) src.fetch_into(names.at("v"), (char*)w_qkv.p + (size_t)(q + k) * hidden * es, rt->dtype);
        }
        if (has_gate || wide_gate) src.fetch_into(names.at("gate"), (char*)w_qkv.p + (size_t)(q + k + v) * hidden * es, rt->dtype);
        const long long o = (long long)n_heads * v_head_dim;
        o_buf = DeviceBuffer(rt->dev, (size_t)hidden * o * es, "the output matrix of an attention layer");
        w_o = Mat{o_buf.get(), hidden, o, rt->dtype, hidden};
        src.fetch_into(names.at("o"), w_o.p, rt->dtype);
        // the small vectors are used in float32 arithmetic and kept so
        if (qkv_bias) {
            b_q = fetch_owned(rt, src, names.at("q_bias"), DType::F32, "an attention bias");
            if (own_kv) {
                b_k = fetch_owned(rt, src, names.at("k_bias"), DType::F32, "an attention bias");
                b_v = fetch_owned(rt, src, names.at("v_bias"), DType::F32, "an attention bias");
            }
        }
        if (proj_norm) {
            n_q = fetch_owned(rt, src, names.at("q_norm"), DType::F32, "a projection norm's weight");
            if (own_kv) n_k = fetch_owned(rt, src, names.at("k_norm"), DType::F32, "a projection norm's weight");
        }
        if (has_sink) sinks = fetch_owned(rt, src, names.at("sink"), DType::F32, "the attention sinks");
        if (log_distance) {
            dist_r1 = fetch_owned(rt, src, names.at("r1"), DType::F32, "an attention layer's distance factors");
            dist_r2 = fetch_owned(rt, src, names.at("r2"), DType::F32, "an attention layer's distance factors");
        }
        if (head_mix) mix = fetch_owned(rt, src, names.at("mix"), DType::F32, "an attention layer's head-mixing matrix");
        if (o_bias) b_o = fetch_owned(rt, src, names.at("o_bias"), DType::F32, "an attention bias");
        if (maps == 2) {
            // lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff: one number for the layer, made once in float32
            std::vector<float> v[4];
            const char* roles[4] = {"lq1", "lk1", "lq2", "lk2"};
            for (int i = 0; i < 4; i++) {
                OwnedMat t = fetch_owned(rt, src, names.at(roles[i]), DType::F32, "a lambda vector");
                v[i].resize((size_t)head_dim);
                rt->dev->synchronize();
                check_cuda(cudaMemcpy(v[i].data(), t.m.p, v[i].size() * sizeof(float), cudaMemcpyDeviceToHost), "reading a lambda vector");
            }
            float d1 = 0.f, d2 = 0.f;
            for (int c = 0; c < head_dim; c++) {
                d1 = std::fmaf(v[0][c], v[1][c], d1);
                d2 = std::fmaf(v[2][c], v[3][c], d2);
            }
            lambda = std::exp(d1) - std::exp(d2) + diff;
        }
    }
    CacheRequest cache_request() const override {
        if (values_are_keys) return CacheRequest::paged_keys_only(n_kv_heads, head_dim, window);
        return own_kv ? CacheRequest::paged(n_kv_heads, maps * head_dim, window, v_head_dim) : CacheRequest();
    }

    // values = keys: one float32 product for q, k and the gate; q out and k into the pages (with the table rotation,
    // if the layer has one); the kernel for mixed scores
    MatOrPartials forward_mixed(const Mat& h, const StepContext& ctx, KVView kv, bool may_defer) {
        Device& dev = *rt->dev;
        const ops::Geometry g{n_heads, n_kv_heads, head_dim};
        Mat x = ops::linear(dev, rt->gemm, h, w_qkv, DType::F32, false).m;
        ops::QkPrep p;
        p.q_off = 0;
        p.k_off = (int)q_rows();
        p.v_off = -1;
        const float* table = nullptr;
        int rot = 0;
        long long n_pos = 0;
        bool pairs = false;
        if (!position->table_rotation(&table, &rot, &n_pos, &pairs))
            throw EngineError("attention: with values = keys the position encoding must be none or a table rotation");
        p.cos_sin = table;
        p.rot_dim = rot;
        p.pairs = pairs;
        p.n_pos = n_pos;
        Mat q = ops::qk_prep(dev, x, p, g, ctx, kv, rt->dtype);
        ops::MixedAttention m;
        m.r1 = (const float*)dist_r1.m.p;
        m.r2 = (const float*)dist_r2.m.p;
        m.mix = (const float*)mix.m.p;
        if (wide_gate) {
            m.gate = (const float*)x.p + (q_rows() + k_rows());
            m.gate_stride = (int)x.cols;
        }
        Mat o = ops::attention_mixed(dev, q, kv, ctx, g, scale, m);
        return ops::linear(dev, rt->gemm, o, w_o, out_f32 ? DType::F32 : rt->dtype, may_defer);
    }

    MatOrPartials forward_general(const Mat& h, const StepContext& ctx, KVView kv, bool may_defer) {
        Device& dev = *rt->dev;
        const ops::Geometry g{n_heads, n_kv_heads, maps * head_dim};      // with two maps a head's row is [map 1, map 2]
        if (kv.n_kv_heads != n_kv_heads || kv.head_dim != maps * head_dim || (kv.v_head_dim > 0 ? kv.v_head_dim : kv.head_dim) != v_head_dim)
            throw EngineError("attention: the cache entry's keys and values do not have this layer's head count and sizes");
        if (!own_kv && kv.writes) throw EngineError("attention: a layer without key and value projections cannot write a cache entry");
        Mat x = ops::linear(dev, rt->gemm, h, w_qkv, DType::F32, false).m;
        ops::QkPrep p;
        p.q_off = 0;
        if (own_kv) {
            p.k_off = (int)q_rows();
            p.v_off = (int)(q_rows() + k_rows());
        }
        p.q_bias = (const float*)b_q.m.p;
        p.k_bias = (const float*)b_k.m.p;
        p.v_bias = (const float*)b_v.m.p;
        p.q_norm = (const float*)n_q.m.p;
        p.k_norm = (const float*)n_k.m.p;
        p.eps = norm_eps;
        const float* table = nullptr;
        int rot = 0;
        long long n_pos = 0;
        bool pairs = false;
        if (!position->table_rotation(&table, &rot, &n_pos, &pairs))
            throw EngineError("attention: with biases, norms, sinks or gates the position encoding must be a table rotation");
        p.cos_sin = table;
        p.rot_dim = rot;
        p.pairs = pairs;
        p.n_pos = n_pos;
        p.q_temp_coef = q_temp_coef;
        p.q_temp_every = q_temp_every;
        Mat q = ops::qk_prep(dev, x, p, g, ctx, kv, rt->dtype);
        if (maps == 2) {
            ops::DiffAttention da;
            da.lambda = lambda;
            da.eps = norm_eps;
            da.out_scale = 1.f - diff;
            Mat o = ops::attention_diff(dev, q, kv, ctx, ops::Geometry{n_heads, n_kv_heads, head_dim}, scale, da);
            return project_out(o, may_defer);
        }
        ops::AttentionExtras ex;
        ex.sinks = (const float*)sinks.m.p;
        if (has_gate) {
            ex.gate = (const float*)x.p + (q_rows() + k_rows() + v_rows());
            ex.gate_stride = (int)x.cols;
        }
        ex.wide_weights = true;       // the softmax weights are not to be rounded to eight bits
        Mat o = ops::attention_ex(dev, q, kv, ctx, g, scale, ex);
        return project_out(o, may_defer);
    }
    // W_o o (+ b_o); with a bias the product is finished here, since the bias joins a finished row
    MatOrPartials project_out(const Mat& o, bool may_defer) {
        MatOrPartials y = ops::linear(*rt->dev, rt->gemm, o, w_o, out_f32 ? DType::F32 : rt->dtype, may_defer && !o_bias);
        if (o_bias) ops::add_bias(*rt->dev, y.m, (const float*)b_o.m.p);
        return y;
    }

    MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool may_defer) override {
        if (cache.kind != CacheView::KV) throw EngineError("attention: the layer's cache entry holds no keys and values");
        Device& dev = *rt->dev;
        KVView kv = cache.kv;
        kv.writes = writes;
        if (values_are_keys) return forward_mixed(h, ctx, kv, may_defer);
        if (general()) return forward_general(h, ctx, kv, may_defer);
        const ops::Geometry g{n_heads, n_kv_heads, head_dim};
        const float* table = nullptr;
        int rot = 0;
        long long n_pos = 0;
        const bool rotation = position->rotation_table(&table, &rot, &n_pos);
        if (ctx.is_decode && rotation && rot % 16 == 0 && ops::attention_decode_ring_supported(h.dtype, n_heads, n_kv_heads, head_dim, kv.page_size)) {
            // one token per sequence: the attention kernel itself adds up the K slices of the projection,
            // rotates Q and the new K row and writes K and V into the cache
            MatOrPartials qkv = ops::linear(dev, rt->gemm, h, w_qkv, rt->dtype, true);
            ops::FusedRope fr{table, rot, n_pos, writes, ctx.err};
            Mat o = ops::attention_decode_ring(dev, qkv, kv, ctx, g, scale, ctx.max_seq_len, 0, &fr);
            return ops::linear(dev, rt->gemm, o, w_o, rt->dtype, may_defer);
        }
        // the packed projection may stay in K slices if the position encoding's kernel adds them up
        MatOrPartials qkv = ops::linear(dev, rt->gemm, h, w_qkv, rt->dtype, position->takes_partials());
        Mat q = position->encode_and_store(qkv, g, ctx, kv);
        Mat o = ops::attention(dev, q, kv, ctx, g, scale);
        return ops::linear(dev, rt->gemm, o, w_o, rt->dtype, may_defer);
    }
};

// Gated feed-forward (SwiGLU): down( act(gate(h)) * up(h) ), no biases.  The reference's
// LlamaFFNModule (src/core/graph.cpp:57-79) runs w3 (up), w1 (gate), Silu, Mul, w2 (down) as five
// operators; silu(x) = x / (1 + exp(-x)) (src/kern/naive/naive.cpp:80-89).  Here gate and up are packed
// into one [2I, H] matrix at load, row 2i the gate row and row 2i + 1 the up row of output i, so that
// one product feeds the activation, and where the package's own kernels run that product the
// activation is their epilogue (ops::linear_gated).
// `names` renames the three tensors; `output_dtype` = "float32" leaves the down projection unrounded;
// `activation` is "silu" (default), "relu" or "gelu_tanh" (each the epilogue of the package's own product kernels).
struct GatedMLP : FeedForward {
    long long hidden, inter;
    bool out_f32;
    int act;
    std::string n_gate = "gate_proj.weight", n_up = "up_proj.weight", n_down = "down_proj.weight";
    DeviceBuffer gu_buf, down_buf;
    Mat w_gate_up, w_down;
    GatedMLP(const PartSpec& s, Runtime* rt)
            : FeedForward(s, rt), hidden(s.get_int("hidden_size")), inter(s.get_int("intermediate_size")),
              out_f32(s.get_string("output_dtype", "compute") == "float32") {
        act = ops::gate_act_from_name(s.get_string("activation", "silu"));
        if (act < 0 || act == ops::kActSwishClamped)
            throw ConfigError("gated_mlp: activation '" + s.get_string("activation", "silu") + "' is not supported (silu, relu, gelu_tanh)");
        if (hidden <= 0 || inter <= 0) throw ConfigError("gated_mlp: sizes must be positive");
        if (s.has("names")) {
            const Json& n = s.params.at("names");
            if (n.has("gate")) n_gate = n.at("gate").as_string();
            if (n.has("up")) n_up = n.at("up").as_string();
            if (n.has("down")) n_down = n.at("down").as_string();
        }
    }
    TensorDecls tensors() const override {
        return {{n_gate, TensorDecl{{inter, hidden}}}, {n_up, TensorDecl{{inter, hidden}}}, {n_down, TensorDecl{{hidden, inter}}}};
    }
    void load(TensorSource& src) override {
        const size_t es = dtype_size(rt->dtype);
        gu_buf = DeviceBuffer(rt->dev, (size_t)2 * inter * hidden * es, "the packed gate/up matrix");
        w_gate_up = Mat{gu_buf.get(), 2 * inter, hidden, rt->dtype, 2 * inter};
        src.fetch_into(n_gate, w_gate_up.p, rt->dtype, 2 * hidden);
        src.fetch_into(n_up, (char*)w_gate_up.p + (size_t)hidden * es, rt->dtype, 2 * hidden);
        down_buf = DeviceBuffer(rt->dev, (size_t)hidden * inter * es, "the down matrix of a feed-forward layer");
        w_down = Mat{down_buf.get(), hidden, inter, rt->dtype, hidden};
        src.fetch_into(n_down, w_down.p, rt->dtype);
    }
    MatOrPartials forward(const Mat& h, const StepContext&, bool may_defer) override {
        Device& dev = *rt->dev;
        return ops::linear(dev, rt->gemm, ops::linear_gated(dev, rt->gemm, h, w_gate_up, act), w_down, out_f32 ? DType::F32 : rt->dtype,
                           may_defer);
    }
};

// Token embedding: x[t] = W[id[t]] (src/kern/naive/naive.cpp:43-54; EmbdModule, src/core/graph.cpp:143-151),
// written as the float32 residual stream.
// Two parameters beyond the gather: `scale` (the row times a constant) and `sinusoid_base` (a position vector is added:
// entry 2i is sin(p base^(-2i / hidden)) and entry 2i + 1 the cosine of the same angle; the frequencies are made in
// float64 once, angle and functions are float32).  A tied head still reads the table itself, without the scale.
struct Embedding : EmbeddingPart {
    long long vocab, hidden;
    std::string tensor;         // the table's name below the part's prefix
    double scale, sinusoid_base;
    OwnedMat weight;
    DeviceBuffer freq_buf;
    Embedding(const PartSpec& s, Runtime* rt)
            : EmbeddingPart(s, rt), vocab(s.get_int("vocab_size")), hidden(s.get_int("hidden_size")), tensor(s.get_string("tensor", "weight")),
              scale(s.get_double("scale", 1.0)), sinusoid_base(s.get_double("sinusoid_base", 0.0)) {
        if (sinusoid_base < 0 || (s.has("sinusoid_base") && !(sinusoid_base > 0))) throw ConfigError("embedding: sinusoid_base must be positive");
    }
    TensorDecls tensors() const override { return {{tensor, TensorDecl{{vocab, hidden}}}}; }
    void load(TensorSource& src) override {
        weight = fetch_owned(rt, src, tensor, rt->dtype, "the embedding table");
        if (sinusoid_base > 0) {
            std::vector<float> f((size_t)(hidden + 1) / 2);
            for (size_t i = 0; i < f.size(); i++) f[i] = (float)std::pow(sinusoid_base, -2.0 * (double)i / (double)hidden);
            freq_buf = DeviceBuffer(rt->dev, f.size() * sizeof(float), "the frequencies of a sinusoid position vector");
            rt->dev->synchronize();
            check_cuda(cudaMemcpy(freq_buf.get(), f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice), "uploading the frequencies");
        }
    }
    ResidualStream forward(const StepContext& ctx) override {
        ResidualStream s;
        s.dev = rt->dev;
        if (scale != 1.0 || sinusoid_base > 0)
            s.x = ops::embedding_scaled(*rt->dev, ctx, weight.m, (float)scale, (const float*)freq_buf.get());
        else
            s.x = ops::embedding(*rt->dev, ctx.ids, ctx.T, weight.m, ctx.err);
        return s;
    }
    const Mat* table() const override { return &weight.m; }
};

// A plain linear map y = W x without bias, as a feed-forward part: "linear" with `in_size`, `out_size`, the tensor's
// name `tensor` and `output_dtype`.  A model's re-entry map (ModelSpec::reentry) is one.
struct LinearMap : FeedForward {
    long long n_in, n_out;
    bool out_f32;
    std::string tensor;
    OwnedMat w;
    LinearMap(const PartSpec& s, Runtime* rt)
            : FeedForward(s, rt), n_in(s.get_int("in_size")), n_out(s.get_int("out_size")),
              out_f32(s.get_string("output_dtype", "compute") == "float32"), tensor(s.get_string("tensor", "weight")) {
        if (n_in <= 0 || n_out <= 0) throw ConfigError("linear: sizes must be positive");
    }
    TensorDecls tensors() const override { return {{tensor, TensorDecl{{n_out, n_in}}}}; }
    void load(TensorSource& src) override { w = fetch_owned(rt, src, tensor, rt->dtype, "a linear map's matrix"); }
    MatOrPartials forward(const Mat& h, const StepContext&, bool may_defer) override {
        return ops::linear(*rt->dev, rt->gemm, h, w.m, out_f32 ? DType::F32 : rt->dtype, may_defer);
    }
};

// Token embedding plus a hashed bigram table: x[t] = W[id_t] + G[(id_{t-1} * mul_prev + id_t * mul_cur) mod buckets],
// and G's last row (number `buckets`) for a sequence's first token.  The previous token of a step's first token is
// per-sequence state: one int32 per slot in a cache entry of the embedding's own.
struct BigramEmbedding : EmbeddingPart {
    long long vocab, hidden;
    ops::BigramHash hash;
    std::string tensor, bigram_tensor;
    OwnedMat weight, bigram;
    BigramEmbedding(const PartSpec& s, Runtime* rt)
            : EmbeddingPart(s, rt), vocab(s.get_int("vocab_size")), hidden(s.get_int("hidden_size")), tensor(s.get_string("tensor", "weight")),
              bigram_tensor(s.get_string("bigram_tensor", "bigram.weight")) {
        hash.buckets = s.get_int("buckets");
        hash.mul_prev = s.get_int("mul_prev");
        hash.mul_cur = s.get_int("mul_cur");
        if (hash.buckets <= 0 || hash.buckets >= (1LL << 31) || hash.mul_prev < 0 || hash.mul_cur < 0)
            throw ConfigError("bigram_embedding: buckets must be positive and the multipliers not negative");
    }
    TensorDecls tensors() const override {
        return {{tensor, TensorDecl{{vocab, hidden}}}, {bigram_tensor, TensorDecl{{hash.buckets + 1, hidden}}}};
    }
    void load(TensorSource& src) override {
        weight = fetch_owned(rt, src, tensor, rt->dtype, "the embedding table");
        bigram = fetch_owned(rt, src, bigram_tensor, rt->dtype, "the bigram table");
    }
    CacheRequest cache_request() const override { return CacheRequest::state({1}, DType::I32); }
    bool pad_safe() const override { return false; }
    ResidualStream forward(const StepContext&) override { throw EngineError("bigram_embedding: needs its per-sequence state"); }
    ResidualStream forward_with_state(const StepContext& ctx, const CacheView& cache) override {
        if (cache.kind != CacheView::State) throw EngineError("bigram_embedding: the embedding's cache entry holds no state");
        ResidualStream s;
        s.dev = rt->dev;
        s.x = ops::bigram_embedding(*rt->dev, ctx, weight.m, bigram.m, hash, cache.st);
        return s;
    }
    const Mat* table() const override { return &weight.m; }
};

// Output head: logits = y . W_out^T in float32 (src/core/op.cpp:230-247 computes it for the last row
// only and not at all on prefill, src/core/graph.cpp:132-141; here for the rows the caller wants).  A
// tied head uses the embedding table (the reference has no tying).
struct LMHead : HeadPart {
    long long vocab, hidden;
    bool is_tied;
    std::string tensor;
    OwnedMat own;
    Mat weight;
    LMHead(const PartSpec& s, Runtime* rt)
            : HeadPart(s, rt), vocab(s.get_int("vocab_size")), hidden(s.get_int("hidden_size")), is_tied(s.get_bool("tied", false)),
              tensor(s.get_string("tensor", "weight")) {}
    TensorDecls tensors() const override {
        if (is_tied) return {};
        return {{tensor, TensorDecl{{vocab, hidden}}}};
    }
    void load(TensorSource& src) override {
        if (is_tied) return;
        own = fetch_owned(rt, src, tensor, rt->dtype, "the output matrix");
        weight = own.m;
    }
    bool tied() const override { return is_tied; }
    void tie(const EmbeddingPart& e) override {
        if (!e.table()) throw ConfigError("lm_head: tied to an embedding that has no table");
        weight = *e.table();
    }
    Mat forward(const Mat& y, const StepContext&) override { return ops::linear(*rt->dev, rt->gemm, y, weight, DType::F32, false).m; }
};

// "prenorm" is the reference's layer (src/graph/llama_like.cpp:69-105):
//     x = x + mixer(norm1(x));  x = x + ffn(norm2(x))
// with the residual taken from the un-normed stream.
struct PreNormBlock : Block {
    void forward(ResidualStream& stream, const StepContext& ctx, const CacheView& cache, bool writes) override {
        // the outputs only go into the residual stream, so they may stay unreduced: the next norm adds
        // the slices while it reads the row anyway
        Mat h = norms.at("norm1")->forward(stream, nullptr, 0);
        stream.add(mixer->forward(h, ctx, cache, writes, true));
        h = norms.at("norm2")->forward(stream, nullptr, 0);
        stream.add(ffn->forward(h, ctx, true));
    }
};

// "prenorm_scaled" is the same layer with a learned factor per channel on each sublayer's output (a layer scale):
//     x = x + ls1 * mixer(norm1(x));  x = x + ls2 * ffn(norm2(x))
// the roles "ls1" and "ls2" are parts that give a channel_scale ("layer_scale").  "prenorm_scaled_mixer" is the layer
// without a feed-forward (roles norm1, ls1).
struct PreNormScaledBlock : Block {
    void forward(ResidualStream& stream, const StepContext& ctx, const CacheView& cache, bool writes) override {
        Mat h = norms.at("norm1")->forward(stream, nullptr, 0);
        stream.add_normed(mixer->forward(h, ctx, cache, writes, false), norms.at("ls1"));
        if (!ffn) return;
        h = norms.at("norm2")->forward(stream, nullptr, 0);
        stream.add_normed(ffn->forward(h, ctx, false), norms.at("ls2"));
    }
};

// "postnorm" is the norm-after-the-sum layer:
//     x = norm1(a x + mixer(x));  x = norm2(a x + ffn(x))
// The sublayers read the stream itself, and the normed sum replaces it; the factor a is the norms'
// `residual_scale`.  "postnorm_mixer" is the same layer without a feed-forward; its norm2 is given as an
// optional norm and used only if the weight file has it: x = norm2(a x).
struct PostNormBlock : Block {
    void forward(ResidualStream& stream, const StepContext& ctx, const CacheView& cache, bool writes) override {
        if (!stream.h.p) {      // the first layer: the embedding's rows in the compute dtype
            stream.flush();
            stream.h = ops::cast(*stream.dev, stream.x, ctx.rt->dtype);
        }
        // the outputs only go into the norm's sum, so they may stay unreduced K slices
        stream.add(mixer->forward(stream.h, ctx, cache, writes, true));
        stream.h = norms.at("norm1")->forward_into_stream(stream);
        if (!ffn) {
            // no feed-forward: the layer ends here, unless the weight file holds a second norm all the same, which then
            // norms the scaled stream alone
            auto n2 = norms.find("norm2");
            if (n2 != norms.end() && n2->second->present()) stream.h = n2->second->forward_into_stream(stream);
            return;
        }
        stream.add(ffn->forward(stream.h, ctx, true));
        stream.h = norms.at("norm2")->forward_into_stream(stream);
    }
};

// "parallel": one norm, and both sublayers read its output:
//     h = norm1(x);  x = x + mixer(h) + ffn(h)
// (a layer without a feed-forward adds the mixer alone).  The sublayers' outputs stay pending in the stream, and the next
// layer's norm adds them, the mixer's first, to the float32 stream in the kernel that norms it, unrounded if they come in
// float32.
struct ParallelBlock : Block {
    void forward(ResidualStream& stream, const StepContext& ctx, const CacheView& cache, bool writes) override {
        Mat h = norms.at("norm1")->forward(stream, nullptr, 0);       // folds in what the layer before left pending
        stream.add(mixer->forward(h, ctx, cache, writes, false));
        if (ffn) stream.add_second(ffn->forward(h, ctx, false));
    }
};

void register_builtin_parts() {
    register_decay_parts(reg<Mixer>());
    register_delta_parts(reg<Mixer>());
    register_latent_parts(reg<Mixer>());
    register_routed_parts(reg<FeedForward>());
    register_gated_state_parts(reg<Mixer>());
    register_sandwich_parts(reg<Norm>(), reg<Mixer>(), block_reg());
    block_reg()["parallel"] = BlockKind{{"norm1"}, [] { return std::unique_ptr<Block>(new ParallelBlock); }};
    reg<FeedForward>()["linear"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<FeedForward>(new LinearMap(s, rt)); };
    reg<EmbeddingPart>()["bigram_embedding"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<EmbeddingPart>(new BigramEmbedding(s, rt)); };
    block_reg()["postnorm"] = BlockKind{{"norm1", "norm2"}, [] { return std::unique_ptr<Block>(new PostNormBlock); }};
    block_reg()["postnorm_mixer"] = BlockKind{{"norm1", "norm2"}, [] { return std::unique_ptr<Block>(new PostNormBlock); }};
    reg<Norm>()["rmsnorm"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Norm>(new RMSNorm(s, rt)); };
    reg<PositionEncoding>()["rope_half"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<PositionEncoding>(new RopeTable(s, rt, false)); };
    reg<PositionEncoding>()["rope_pairs"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<PositionEncoding>(new RopeTable(s, rt, true)); };
    reg<PositionEncoding>()["none"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<PositionEncoding>(new NoPosition(s, rt)); };
    reg<Mixer>()["attention"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new Attention(s, rt)); };
    reg<FeedForward>()["gated_mlp"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<FeedForward>(new GatedMLP(s, rt)); };
    reg<EmbeddingPart>()["embedding"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<EmbeddingPart>(new Embedding(s, rt)); };
    reg<HeadPart>()["lm_head"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<HeadPart>(new LMHead(s, rt)); };
    block_reg()["prenorm"] = BlockKind{{"norm1", "norm2"}, [] { return std::unique_ptr<Block>(new PreNormBlock); }};
    block_reg()["prenorm_scaled"] = BlockKind{{"norm1", "norm2", "ls1", "ls2"}, [] { return std::unique_ptr<Block>(new PreNormScaledBlock); }};
    block_reg()["prenorm_scaled_mixer"] = BlockKind{{"norm1", "ls1"}, [] { return std::unique_ptr<Block>(new PreNormScaledBlock); }};
    reg<Norm>()["layer_scale"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Norm>(new LayerScale(s, rt)); };
}

}  // namespace

}  // namespace illm
