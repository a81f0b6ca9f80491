// Softmax attention through low-rank latents: the mixer "latent_attention".
//
//     c_q = rmsnorm(W_dq h) * w_q;   q_h = U_q,h c_q  [heads x d]
//     c   = rmsnorm(W_dkv h) * w_kv  [kv_rank]                    the only thing cached
//     k_h = U_k,h c,  v_h = U_v,h c;   score = (q_h . k_h) * scale over the visible positions (all before, or the
//     last `window`);   softmax;   y = W_o [sum_j p_j v_h,j]_h
//
// No position encoding.  It is computed in the absorbed form: score = (U_k,h^T q_h) . c and
// o_h = U_v,h (sum_j p_j c_j), so the attention kernels see ONE key/value head of kv_rank channels (the cached c is
// key and value at once: a keys-only cache entry) and `heads` query heads, and the per-head maps U_k,h^T and U_v,h run
// before and after them (ops::head_linear).  A step's keys and values are never expanded per head.
//
// Options: `q_rank` 0 (the queries come straight from the mixer's input, q = W_q h, no query latent);
// `rot_head_dim` dr > 0 with a `position` part (a table rotation): every query head has dr more channels behind its d, the
// key/value down-projection dr more rows behind the latent's (not normed), both are rotated by the position, and
//     score = (q_h[0:d] . k_h + rot(q_h[d:d+dr]) . rot(kr)) * scale
// with the ONE rotated key part kr shared by all heads.  The cache row is then [c, rot(kr)] (kv_rank + dr channels), the
// absorbed query [U_k,h^T q_h[0:d], rot(q_h[d:])], and the attention kernels' values are the whole row, of which U_v,h
// reads the first kv_rank channels;  `out_gate` = "head_sigmoid" (a projection of the mixer's input to one number per
// head, whose sigmoid multiplies the head's output).  These three run on a path of their own (forward_direct).
#include <cmath>

#include "parts/parts.h"

namespace illm {

namespace {

struct LatentAttention : Mixer {
    long long hidden;
    int n_heads, head_dim, v_head_dim, q_rank, kv_rank, window;
    int rot_head_dim = 0;
    float scale, norm_eps;
    bool out_f32, has_gate = false;
    std::map<std::string, std::string> names;
    std::unique_ptr<PositionEncoding> position;
    DeviceBuffer w_buf;
    Mat w_down;
    OwnedMat w_uq, w_uk, w_uv, w_o, n_q, n_kv;

    LatentAttention(const PartSpec& s, Runtime* rt)
            : Mixer(s, rt), hidden(s.get_int("hidden_size")), n_heads((int)s.get_int("n_heads")), head_dim((int)s.get_int("head_dim")),
              v_head_dim((int)s.get_int("v_head_dim", s.get_int("head_dim"))), q_rank((int)s.get_int("q_rank")), kv_rank((int)s.get_int("kv_rank")),
              window((int)s.get_int("window", 0)), norm_eps((float)s.get_double("norm_eps", 1e-6)),
              out_f32(s.get_string("output_dtype", "compute") == "float32") {
        if (hidden <= 0 || n_heads <= 0 || head_dim <= 0 || v_head_dim <= 0 || q_rank < 0 || kv_rank <= 0 || window < 0)
            throw ConfigError("latent_attention: sizes must be positive");
        rot_head_dim = (int)s.get_int("rot_head_dim", 0);
        const std::string og = s.get_string("out_gate", "none");
        if (og != "none" && og != "head_sigmoid") throw ConfigError("latent_attention: out_gate '" + og + "' is not supported (none, head_sigmoid)");
        has_gate = og == "head_sigmoid";
        if (rot_head_dim < 0) throw ConfigError("latent_attention: rot_head_dim must not be negative");
        if (q_rank > 0 && (rot_head_dim > 0 || has_gate)) throw ConfigError("latent_attention: rotated channels and the head gate need q_rank 0 (queries straight from the input)");
        if (rot_head_dim > 0) {
            position = build_position(s.get_part("position"), rt);
            if (rt) position->prepare();
        }
        scale = s.has("scale") ? (float)s.get_double("scale") : (float)(1.0 / std::sqrt((double)head_dim));
        names = {{"q_down", "q_a_proj.weight"}, {"q_norm", "q_a_norm.weight"}, {"q_up", "q_b_proj.weight"}, {"kv_down", "kv_a_proj.weight"},
                 {"kv_norm", "kv_a_norm.weight"}, {"k_up", "k_b_proj.weight"}, {"v_up", "v_b_proj.weight"}, {"o", "o_proj.weight"},
                 {"q", "q_proj.weight"}, {"gate", "gate_proj.weight"}};
        if (s.has("names"))
            for (auto& m : s.params.at("names").members()) names[m.first] = m.second.as_string();
        if (rt && kv_rank + rot_head_dim > 1024)
            throw ConfigError("latent_attention: a latent of " + std::to_string(kv_rank + rot_head_dim) + " channels is beyond the kernels (up to 1024)");
    }
    bool direct() const { return q_rank == 0; }
    long long row() const { return (long long)kv_rank + rot_head_dim; }       // channels of a cache row
    bool graph_safe() const override { return true; }
    bool pad_safe() const override { return false; }
    CacheRequest cache_request() const override { return CacheRequest::paged_keys_only(1, (int)row(), window); }
    TensorDecls tensors() const override {
        const long long q = (long long)n_heads * head_dim, v = (long long)n_heads * v_head_dim;
        auto nm = [&](const char* role) { return names.at(role); };
        if (direct()) {
            TensorDecls d = {{nm("q"), TensorDecl{{(long long)n_heads * (head_dim + rot_head_dim), hidden}}}, {nm("kv_down"), TensorDecl{{row(), hidden}}},
                             {nm("kv_norm"), TensorDecl{{(long long)kv_rank}, "norm"}}, {nm("k_up"), TensorDecl{{q, (long long)kv_rank}}},
                             {nm("v_up"), TensorDecl{{v, (long long)kv_rank}}}};
            if (has_gate) d.push_back({nm("gate"), TensorDecl{{(long long)n_heads, hidden}}});
            d.push_back({nm("o"), TensorDecl{{hidden, v}}});
            return d;
        }
        return {{nm("q_down"), TensorDecl{{(long long)q_rank, hidden}}}, {nm("q_norm"), TensorDecl{{(long long)q_rank}, "norm"}},
                {nm("q_up"), TensorDecl{{q, (long long)q_rank}}}, {nm("kv_down"), TensorDecl{{(long long)kv_rank, hidden}}},
                {nm("kv_norm"), TensorDecl{{(long long)kv_rank}, "norm"}}, {nm("k_up"), TensorDecl{{q, (long long)kv_rank}}},
                {nm("v_up"), TensorDecl{{v, (long long)kv_rank}}}, {nm("o"), TensorDecl{{hidden, v}}}};
    }
    // rows of the packed matrix of the direct path: the queries, then latent and raw key part, then the gate
    long long dq_rows() const { return (long long)n_heads * (head_dim + rot_head_dim); }
    void load(TensorSource& src) override {
        const size_t es = dtype_size(rt->dtype);
        if (direct()) {
            const long long all = dq_rows() + row() + (has_gate ? n_heads : 0);
            w_buf = DeviceBuffer(rt->dev, (size_t)all * hidden * es, "the packed projections of a latent-attention layer");
            w_down = Mat{w_buf.get(), all, hidden, rt->dtype, all};
            src.fetch_into(names.at("q"), w_down.p, rt->dtype);
            src.fetch_into(names.at("kv_down"), (char*)w_down.p + (size_t)dq_rows() * hidden * es, rt->dtype);
            if (has_gate) src.fetch_into(names.at("gate"), (char*)w_down.p + (size_t)(dq_rows() + row()) * hidden * es, rt->dtype);
            w_uk = fetch_owned(rt, src, names.at("k_up"), rt->dtype, "the key up-projection");
            w_uv = fetch_owned(rt, src, names.at("v_up"), rt->dtype, "the value up-projection");
            w_o = fetch_owned(rt, src, names.at("o"), rt->dtype, "the output matrix of an attention layer");
            n_kv = fetch_owned(rt, src, names.at("kv_norm"), DType::F32, "a latent norm's weight");
            return;
        }
        const long long all = (long long)q_rank + kv_rank;
        w_buf = DeviceBuffer(rt->dev, (size_t)all * hidden * es, "the packed latent projections");
        w_down = Mat{w_buf.get(), all, hidden, rt->dtype, all};
        src.fetch_into(names.at("q_down"), w_down.p, rt->dtype);
        src.fetch_into(names.at("kv_down"), (char*)w_down.p + (size_t)q_rank * hidden * es, rt->dtype);
        w_uq = fetch_owned(rt, src, names.at("q_up"), rt->dtype, "the query up-projection");
        w_uk = fetch_owned(rt, src, names.at("k_up"), rt->dtype, "the key up-projection");
        w_uv = fetch_owned(rt, src, names.at("v_up"), rt->dtype, "the value up-projection");
        w_o = fetch_owned(rt, src, names.at("o"), rt->dtype, "the output matrix of an attention layer");
        n_q = fetch_owned(rt, src, names.at("q_norm"), DType::F32, "a latent norm's weight");
        n_kv = fetch_owned(rt, src, names.at("kv_norm"), DType::F32, "a latent norm's weight");
    }

    MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool may_defer) override {
        if (cache.kind != CacheView::KV) throw EngineError("latent_attention: the layer's cache entry holds no keys");
        Device& dev = *rt->dev;
        KVView kv = cache.kv;
        kv.writes = writes;
        if (kv.n_kv_heads != 1 || kv.head_dim != row()) throw EngineError("latent_attention: the cache entry does not hold this layer's latent");
        if (direct()) return forward_direct(h, ctx, kv, may_defer);
        Mat x = ops::linear(dev, rt->gemm, h, w_down, DType::F32, false).m;
        Mat cq = ops::latent_prep(dev, x, q_rank, kv_rank, (const float*)n_q.m.p, (const float*)n_kv.m.p, norm_eps, ctx, kv, rt->dtype);
        // a prompt's queries are rounded to the activation dtype for the library's batched product; single tokens stay float32
        Mat q = ops::linear(dev, rt->gemm, cq, w_uq.m, ctx.is_decode ? DType::F32 : rt->dtype, false).m;
        Mat qa = ops::head_linear(dev, q, w_uk.m, n_heads, true, rt->dtype);          // U_k,h^T q_h
        const ops::Geometry g{n_heads, 1, kv_rank};
        ops::AttentionExtras ex;
        ex.wide_weights = true;       // the softmax weights are not to be rounded to eight bits
        // a latent whose width the framework's attention kernels do not take (not a multiple of 8, beyond 256) has a plain kernel
        Mat o = (kv_rank % 8 || kv_rank > ops::kMaxHeadDimGeneric) ? ops::latent_attention_any(dev, qa, kv, ctx, n_heads, scale)
                                                                  : ops::attention_ex(dev, qa, kv, ctx, g, scale, ex);
        Mat ov = ops::head_linear(dev, o, w_uv.m, n_heads, false, rt->dtype);         // U_v,h (sum p c)
        return ops::linear(dev, rt->gemm, ov, w_o.m, out_f32 ? DType::F32 : rt->dtype, may_defer);
    }

    // queries straight from the input, optionally rotated channels beside the latent and a gate per head
    MatOrPartials forward_direct(const Mat& h, const StepContext& ctx, const KVView& kv, bool may_defer) {
        Device& dev = *rt->dev;
        Mat x = ops::linear(dev, rt->gemm, h, w_down, DType::F32, false).m;
        ops::LatentRope p;
        p.q_off = 0;
        p.c_off = (int)dq_rows();
        p.n_heads = n_heads;
        p.head_dim = head_dim;
        p.rot_head_dim = rot_head_dim;
        p.kv_rank = kv_rank;
        p.w_kv = (const float*)n_kv.m.p;
        p.eps = norm_eps;
        if (rot_head_dim > 0) {
            const float* table = nullptr;
            int rot = 0;
            long long n_pos = 0;
            bool pairs = false;
            if (!position->table_rotation(&table, &rot, &n_pos, &pairs)) throw EngineError("latent_attention: the position encoding must be a table rotation");
            if (rot > rot_head_dim) throw EngineError("latent_attention: the rotation is wider than the rotated channels");
            p.cos_sin = table;
            p.rot_dim = rot;
            p.pairs = pairs;
            p.n_pos = n_pos;
        }
        Mat qa;
        Mat qn = ops::latent_rope_prep(dev, x, p, ctx, kv, rt->dtype, &qa);
        ops::HeadPieces into;
        into.into = &qa;
        into.y_head_stride = row();
        ops::head_linear_pieces(dev, qn, w_uk.m, n_heads, true, rt->dtype, into);        // U_k,h^T q_h into the head's first kv_rank channels
        const ops::Geometry g{n_heads, 1, (int)row()};
        ops::AttentionExtras ex;
        ex.wide_weights = true;       // the softmax weights are not to be rounded to eight bits
        if (has_gate) {
            ex.gate = (const float*)x.p + (dq_rows() + row());
            ex.gate_stride = (int)x.cols;
        }
        // a row whose width the framework's attention kernels do not take (not a multiple of 8, beyond 256) has a plain kernel
        Mat o = (row() % 8 || row() > ops::kMaxHeadDimGeneric) ? ops::latent_attention_any(dev, qa, kv, ctx, n_heads, scale, ex.gate, ex.gate_stride)
                                                               : ops::attention_ex(dev, qa, kv, ctx, g, scale, ex);
        ops::HeadPieces from;
        from.x_head_stride = row();
        Mat ov = ops::head_linear_pieces(dev, o, w_uv.m, n_heads, false, rt->dtype, from);      // U_v,h on the first kv_rank channels of sum p [c, kr]
        return ops::linear(dev, rt->gemm, ov, w_o.m, out_f32 ? DType::F32 : rt->dtype, may_defer);
    }
};

}  // namespace

void register_latent_parts(std::map<std::string, PartFactory<Mixer>>& mixers) {
    mixers["latent_attention"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new LatentAttention(s, rt)); };
}

}  // namespace illm
