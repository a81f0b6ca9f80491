// Two mixers whose per-sequence state is a matrix per head that every token decays by one number and adds an outer
// product to, S_t = a_t S_(t-1) + b_t k_t v_t^T, o_t = S_t^T q_t (ops::gated_scan); they differ in where a_t, b_t, q, k
// and v come from and in what follows the read-out.  Everything between the float32 projection and the normed, gated
// row is float32 in both modes; the state is float32 and zero when a sequence starts.
//
// "mlstm": the matrix memory with exponential gating.
//     q = W_q h * d^(-1/2), k = W_k h  [heads x d];  v = W_v h  [heads x dv]
//     i = cap tanh((W_i h + b_i) / cap),  f = logsigmoid(cap tanh((W_f h + b_f) / cap))        per head
//     m_t = max(f + m_(t-1), i)  (m starts at 0);  a_t = exp(f + m_(t-1) - m_t);  b_t = exp(i - m_t)
//     n_t = a_t n_(t-1) + b_t k_t;   o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
//     y = W_o ( o / rms(o) per head * w_norm * sigmoid(W_g h) )
//   Cache entry: S [heads, dv, d], n [heads, d], m [heads].
//
// "mamba2": the selective state space with a scalar decay per head.
//     W_in h = [z: inner | x: inner | B: groups N | C: groups N | dt: heads],  inner = heads dv
//     x, B, C <- silu(conv(x, B, C) + bias)   (one causal filter per channel, `conv` taps)
//     dt <- softplus(dt + dt_bias);  a_t = exp(-exp(A_log) dt);  b_t = dt;  k = B, q = C of the head's group, v = x
//     y = W_o ( rms-norm in norm_groups parts of ((o + D x) * silu(z)) * w_norm )
//   Cache entry: S [heads, dv, N] and the last conv - 1 rows of (x, B, C) before the convolution.
#include <cmath>

#include "parts/parts.h"

namespace illm {

namespace {

long long round4(long long n) { return (n + 3) / 4 * 4; }

std::map<std::string, std::string> names_of(const PartSpec& s, std::map<std::string, std::string> names) {
    if (s.has("names"))
        for (auto& m : s.params.at("names").members()) names[m.first] = m.second.as_string();
    return names;
}

// rows of several tensors stacked into one matrix in the compute dtype; rows beyond the last tensor (up to a
// multiple of four) are zero
struct Packed {
    DeviceBuffer buf;
    Mat m;
    void make(Runtime* rt, TensorSource& src, const std::vector<std::pair<std::string, long long>>& parts, long long cols, const char* what) {
        long long rows = 0;
        for (auto& p : parts) rows += p.second;
        const long long held = round4(rows);
        const size_t es = dtype_size(rt->dtype);
        buf = DeviceBuffer(rt->dev, (size_t)held * cols * es, what);
        m = Mat{buf.get(), held, cols, rt->dtype, held};
        check_cuda(cudaMemsetAsync(buf.get(), 0, (size_t)held * cols * es, rt->dev->stream()), "clearing a packed matrix");
        long long at = 0;
        for (auto& p : parts) {
            src.fetch_into(p.first, (char*)buf.get() + (size_t)at * cols * es, rt->dtype);
            at += p.second;
        }
    }
};

struct MatrixMemory : Mixer {
    long long hidden;
    int n_heads, head_dim, v_head_dim;
    float cap, norm_eps;
    bool out_f32;
    std::map<std::string, std::string> names;
    Packed w_in;
    OwnedMat w_o, norm_w, i_bias, f_bias;

    MatrixMemory(const PartSpec& s, Runtime* rt)
            : Mixer(s, rt), hidden(s.get_int("hidden_size")), n_heads((int)s.get_int("n_heads")), head_dim((int)s.get_int("head_dim")),
              v_head_dim((int)s.get_int("v_head_dim", s.get_int("head_dim"))), cap((float)s.get_double("gate_cap")),
              norm_eps((float)s.get_double("norm_eps", 1e-6)), out_f32(s.get_string("output_dtype", "compute") == "float32") {
        if (hidden <= 0 || n_heads <= 0 || head_dim <= 0 || v_head_dim <= 0) throw ConfigError("mlstm: sizes must be positive");
        if (!(cap > 0)) throw ConfigError("mlstm: gate_cap must be positive");
        names = names_of(s, {{"q", "q_proj.weight"}, {"k", "k_proj.weight"}, {"v", "v_proj.weight"}, {"gate", "g_proj.weight"}, {"o", "o_proj.weight"},
                             {"norm", "norm.weight"}, {"i", "i_proj.weight"}, {"i_bias", "i_proj.bias"}, {"f", "f_proj.weight"}, {"f_bias", "f_proj.bias"}});
        if (rt && !ops::decay_scan_supported(head_dim, v_head_dim)) throw ConfigError("mlstm: heads of more than 1024 channels are beyond the kernel");
    }
    bool graph_safe() const override { return true; }
    bool pad_safe() const override { return false; }
    long long qk() const { return (long long)n_heads * head_dim; }
    long long vv() const { return (long long)n_heads * v_head_dim; }
    long long s_elems() const { return round4(qk() * v_head_dim); }
    long long n_off() const { return s_elems(); }
    long long m_off() const { return s_elems() + qk(); }
    CacheRequest cache_request() const override { return CacheRequest::state({round4(m_off() + n_heads)}, DType::F32); }
    TensorDecls tensors() const override {
        auto nm = [&](const char* r) { return names.at(r); };
        const long long H = n_heads;
        return {{nm("q"), TensorDecl{{qk(), hidden}}}, {nm("k"), TensorDecl{{qk(), hidden}}}, {nm("v"), TensorDecl{{vv(), hidden}}},
                {nm("gate"), TensorDecl{{vv(), hidden}}}, {nm("o"), TensorDecl{{hidden, vv()}}}, {nm("norm"), TensorDecl{{vv()}, "norm"}},
                {nm("i"), TensorDecl{{H, hidden}}}, {nm("i_bias"), TensorDecl{{H}}}, {nm("f"), TensorDecl{{H, hidden}}}, {nm("f_bias"), TensorDecl{{H}}}};
    }
    void load(TensorSource& src) override {
        w_in.make(rt, src, {{names.at("q"), qk()}, {names.at("k"), qk()}, {names.at("v"), vv()}, {names.at("gate"), vv()}, {names.at("i"), n_heads},
                            {names.at("f"), n_heads}},
                  hidden, "the packed projections of a matrix-memory layer");
        w_o = fetch_owned(rt, src, names.at("o"), rt->dtype, "the output matrix of a matrix-memory layer");
        norm_w = fetch_owned(rt, src, names.at("norm"), DType::F32, "a matrix-memory layer's norm weight");
        i_bias = fetch_owned(rt, src, names.at("i_bias"), DType::F32, "an input gate's bias");
        f_bias = fetch_owned(rt, src, names.at("f_bias"), DType::F32, "a forget gate's bias");
    }
    MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool may_defer) override {
        if (cache.kind != CacheView::State) throw EngineError("mlstm: the layer's cache entry holds no state");
        if (!writes) throw EngineError("mlstm: the state belongs to one layer");
        Device& dev = *rt->dev;
        Mat x = ops::linear(dev, rt->gemm, h, w_in.m, DType::F32, false).m;
        const size_t n = (size_t)x.rows * n_heads;
        float *ga = dev.alloc_n<float>(n), *gb = dev.alloc_n<float>(n), *sc = dev.alloc_n<float>(n);
        ops::MlstmGates gp;
        gp.q_off = 0;
        gp.k_off = (int)qk();
        gp.i_off = (int)(2 * qk() + 2 * vv());
        gp.f_off = gp.i_off + n_heads;
        gp.i_bias = (const float*)i_bias.m.p;
        gp.f_bias = (const float*)f_bias.m.p;
        gp.cap = cap;
        gp.q_scale = (float)(1.0 / std::sqrt((double)head_dim));
        gp.n_heads = n_heads;
        gp.head_dim = head_dim;
        gp.n_off = n_off();
        gp.m_off = m_off();
        ops::mlstm_gates(dev, x, gp, ctx, cache.st, ga, gb, sc);
        ops::GatedScan sp;
        sp.q_off = 0;
        sp.k_off = (int)qk();
        sp.v_off = (int)(2 * qk());
        sp.n_heads = sp.n_qk_heads = n_heads;
        sp.head_dim = head_dim;
        sp.v_head_dim = v_head_dim;
        sp.ga = ga;
        sp.gb = gb;
        sp.in_order = rt->is_f32();     // the float32 mode gives the same bits however a prompt is cut
        Mat o = ops::gated_scan(dev, x, sp, ctx, cache.st);
        ops::NormGateExtras ex;
        ex.row_scale = sc;
        ex.head = v_head_dim;
        const float* gate = (const float*)x.p + (2 * qk() + vv());
        Mat y = ops::group_norm_gate_ex(dev, o, v_head_dim, (const float*)norm_w.m.p, (int)vv(), norm_eps, gate, (int)x.cols, 2, rt->dtype, ex);
        return ops::linear(dev, rt->gemm, y, w_o.m, out_f32 ? DType::F32 : rt->dtype, may_defer);
    }
};

struct ScalarDecaySSM : Mixer {
    long long hidden;
    int n_heads, v_head_dim, n_state, groups, norm_groups, taps;
    float norm_eps;
    bool out_f32;
    std::map<std::string, std::string> names;
    Packed w_in;
    OwnedMat w_o, conv_w, conv_b, dt_bias, a_log, skip, norm_w;

    ScalarDecaySSM(const PartSpec& s, Runtime* rt)
            : Mixer(s, rt), hidden(s.get_int("hidden_size")), n_heads((int)s.get_int("n_heads")), v_head_dim((int)s.get_int("v_head_dim")),
              n_state((int)s.get_int("state")), groups((int)s.get_int("groups", 1)), norm_groups((int)s.get_int("norm_groups", 1)),
              taps((int)s.get_int("conv", 1)), norm_eps((float)s.get_double("norm_eps", 1e-6)),
              out_f32(s.get_string("output_dtype", "compute") == "float32") {
        if (hidden <= 0 || n_heads <= 0 || v_head_dim <= 0 || n_state <= 0 || groups <= 0 || norm_groups <= 0 || taps < 1)
            throw ConfigError("mamba2: sizes must be positive");
        if (n_heads % groups) throw ConfigError("mamba2: heads must be a multiple of groups");
        if (inner() % norm_groups) throw ConfigError("mamba2: heads x vdim must be a multiple of norm_groups");
        names = names_of(s, {{"in", "in_proj.weight"}, {"conv", "conv1d.weight"}, {"conv_bias", "conv1d.bias"}, {"dt_bias", "dt_bias"},
                             {"a_log", "A_log"}, {"skip", "D"}, {"norm", "norm.weight"}, {"o", "out_proj.weight"}});
        if (rt && !ops::decay_scan_supported(n_state, v_head_dim)) throw ConfigError("mamba2: a state of more than 1024 rows per head is beyond the kernel");
    }
    bool graph_safe() const override { return true; }
    bool pad_safe() const override { return false; }
    long long inner() const { return (long long)n_heads * v_head_dim; }
    long long gn() const { return (long long)groups * n_state; }
    long long conv_ch() const { return inner() + 2 * gn(); }
    long long in_rows() const { return 2 * inner() + 2 * gn() + n_heads; }
    long long s_elems() const { return round4(inner() * n_state); }
    CacheRequest cache_request() const override { return CacheRequest::state({round4(s_elems() + (long long)(taps - 1) * conv_ch())}, DType::F32); }
    TensorDecls tensors() const override {
        auto nm = [&](const char* r) { return names.at(r); };
        const long long H = n_heads;
        return {{nm("in"), TensorDecl{{in_rows(), hidden}}}, {nm("conv"), TensorDecl{{conv_ch(), (long long)taps}}}, {nm("conv_bias"), TensorDecl{{conv_ch()}}},
                {nm("dt_bias"), TensorDecl{{H}}}, {nm("a_log"), TensorDecl{{H}}}, {nm("skip"), TensorDecl{{H}}},
                {nm("norm"), TensorDecl{{inner()}, "norm"}}, {nm("o"), TensorDecl{{hidden, inner()}}}};
    }
    void load(TensorSource& src) override {
        w_in.make(rt, src, {{names.at("in"), in_rows()}}, hidden, "the input matrix of a state-space layer");
        w_o = fetch_owned(rt, src, names.at("o"), rt->dtype, "the output matrix of a state-space layer");
        conv_w = fetch_owned(rt, src, names.at("conv"), DType::F32, "a convolution's taps");
        conv_b = fetch_owned(rt, src, names.at("conv_bias"), DType::F32, "a convolution's bias");
        dt_bias = fetch_owned(rt, src, names.at("dt_bias"), DType::F32, "a state-space layer's step bias");
        a_log = fetch_owned(rt, src, names.at("a_log"), DType::F32, "a state-space layer's decay rates");
        skip = fetch_owned(rt, src, names.at("skip"), DType::F32, "a state-space layer's skip weights");
        norm_w = fetch_owned(rt, src, names.at("norm"), DType::F32, "a state-space layer's norm weight");
    }
    MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool may_defer) override {
        if (cache.kind != CacheView::State) throw EngineError("mamba2: the layer's cache entry holds no state");
        if (!writes) throw EngineError("mamba2: the state belongs to one layer");
        Device& dev = *rt->dev;
        Mat p = ops::linear(dev, rt->gemm, h, w_in.m, DType::F32, false).m;
        Mat xbc = ops::new_mat(dev, p.rows, conv_ch(), DType::F32);
        ops::ShortConv cp;
        cp.x_off = (int)inner();
        cp.C = (int)conv_ch();
        cp.taps = taps;
        cp.w = (const float*)conv_w.m.p;
        cp.bias = (const float*)conv_b.m.p;
        cp.act = 1;
        cp.state_off = s_elems();
        ops::short_conv(dev, p, cp, ctx, cache.st, xbc, 0);
        const size_t n = (size_t)p.rows * n_heads;
        float *ga = dev.alloc_n<float>(n), *gb = dev.alloc_n<float>(n);
        ops::ssm_gates(dev, p, (int)(2 * inner() + 2 * gn()), (const float*)dt_bias.m.p, (const float*)a_log.m.p, n_heads, ga, gb);
        ops::GatedScan sp;
        sp.v_off = 0;
        sp.k_off = (int)inner();
        sp.q_off = (int)(inner() + gn());
        sp.n_heads = n_heads;
        sp.n_qk_heads = groups;
        sp.head_dim = n_state;
        sp.v_head_dim = v_head_dim;
        sp.ga = ga;
        sp.gb = gb;
        sp.in_order = rt->is_f32();     // the float32 mode gives the same bits however a prompt is cut
        Mat o = ops::gated_scan(dev, xbc, sp, ctx, cache.st);
        ops::NormGateExtras ex;
        ex.head = v_head_dim;
        ex.skip_w = (const float*)skip.m.p;
        ex.skip_x = (const float*)xbc.p;
        ex.skip_ld = (int)xbc.cols;
        ex.gate_first = true;
        Mat y = ops::group_norm_gate_ex(dev, o, (int)(inner() / norm_groups), (const float*)norm_w.m.p, (int)inner(), norm_eps, (const float*)p.p,
                                        (int)p.cols, 1, rt->dtype, ex);
        return ops::linear(dev, rt->gemm, y, w_o.m, out_f32 ? DType::F32 : rt->dtype, may_defer);
    }
};

}  // namespace

void register_gated_state_parts(std::map<std::string, PartFactory<Mixer>>& mixers) {
    mixers["mlstm"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new MatrixMemory(s, rt)); };
    mixers["mamba2"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new ScalarDecaySSM(s, rt)); };
}

}  // namespace illm
