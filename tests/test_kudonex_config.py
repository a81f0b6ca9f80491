"""The Kudonex configuration class and the plain implementation's own pieces, on the CPU.

What config.json says must arrive in the ModelSpec unchanged (sizes, constants, layer order), the tensors the model
declares must be the file's names and shapes, and a configuration that cannot be built is refused in words.  The plain
implementation's mechanisms are checked against second, independent formulations of the same equations.
"""
import math

import numpy as np
import pytest
import plain_kudonex as pk

from inferllm_b200 import ConfigError, KudonexConfig, config_from_dict
from inferllm_b200.weights import tensor_decls

M, S, A = "mlstm", "mamba2", "attention"


def f64(w):
    return {k: np.asarray(v, np.float64) for k, v in w.items()}


def test_spec_carries_every_size_and_constant():
    cfg = pk.random_config((S, A, M, A), width=56, vocab=77, taps=4, emb_scale=1.7, eps=3e-5, heads=3, dim=12, vdim=20, gate_cap=7.5, ssm_heads=6,
                           ssm_vdim=10, state=14, groups=3, norm_groups=5, conv=2, att_heads=6, kv_heads=3, att_dim=10, window=33, scale=0.37,
                           experts=8, top=3, group_count=4, group_keep=2, expert_ff=22, shared_ff=30, mlps=[True, None, "bare", True])
    spec = config_from_dict(cfg).model_spec()
    assert (spec.hidden_size, spec.vocab_size) == (56, 77)
    assert [(e.layer, e.cache, e.writes, e.reenter) for e in spec.schedule] == [(i, i, True, False) for i in range(4)]
    assert [l.block for l in spec.layers] == ["sandwich", "sandwich_mixer", "sandwich", "sandwich"]
    assert [list(l.norms) for l in spec.layers][:2] == [["norm1", "norm1b", "norm2", "norm2b"], ["norm1", "norm1b"]]
    for l in spec.layers:
        assert l.mixer.kind == "input_conv" and (l.mixer["taps"], l.mixer["width"]) == (4, 56)
        assert all(n.kind == "layernorm" and n["eps"] == 3e-5 for n in l.norms.values())
    s, a, m = (spec.layers[i].mixer["inner"] for i in (0, 1, 2))
    assert (s.kind, a.kind, m.kind) == ("mamba2", "attention", "mlstm")
    assert (s["n_heads"], s["v_head_dim"], s["state"], s["groups"], s["norm_groups"], s["conv"], s["norm_eps"]) == (6, 10, 14, 3, 5, 2, 3e-5)
    assert (a["n_heads"], a["n_kv_heads"], a["head_dim"], a["window"], a["scale"], a["values"]) == (6, 3, 10, 33, 0.37, "keys")
    assert (m["n_heads"], m["head_dim"], m["v_head_dim"], m["gate_cap"], m["norm_eps"]) == (3, 12, 20, 7.5, 3e-5)
    full, bare = spec.layers[0].ffn, spec.layers[2].ffn
    assert full.kind == "routed_mlp" and spec.layers[1].ffn.kind == ""
    assert (full["experts"], full["top"], full["intermediate_size"], full["scoring"], full["renormalize"]) == (8, 3, 22, "softmax_all", False)
    assert full["groups"] == {"count": 4, "keep": 2} and full["shared"]["intermediate_size"] == 30
    assert "groups" not in bare.params and "shared" not in bare.params
    e = spec.embedding
    assert e.kind == "embedding" and e["scale"] == 1.7 and e["sinusoid_base"] == 10000.0
    assert spec.head["tied"] is True and spec.final_norm.kind == "layernorm"


def test_without_the_input_convolution_or_a_window_nothing_of_them_exists():
    cfg = pk.random_config((A, M), taps=0, window=0)
    spec = config_from_dict(cfg).model_spec()
    assert [l.mixer.kind for l in spec.layers] == ["attention", "mlstm"]
    assert spec.layers[0].mixer["window"] == 0
    assert not any(n.endswith("canon1") for n in tensor_decls(config_from_dict(cfg)))


def test_the_python_face_is_typed_and_round_trips():
    cfg = pk.random_config((M, S), width=40)
    c = config_from_dict(cfg)
    assert isinstance(c, KudonexConfig) and c.architecture == "Kudonex"
    assert KudonexConfig.from_dict(c.to_dict()) == c and c.to_dict()["width"] == 40


def test_declared_tensors_are_the_files_names_and_shapes():
    cfg = pk.random_config((M, S, A, S), mlps=[True, "bare", None, True], ssm_heads=6, groups=3, norm_groups=1, conv=4, taps=2)
    decls = {name: tuple(shape) for name, (shape, _) in tensor_decls(config_from_dict(cfg)).items()}
    assert decls == {k: tuple(v[0]) for k, v in pk.tensor_shapes(cfg).items()}


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "unknown type"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_heads", 3), "multiple of n_kv_heads"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 8), "values are the keys"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("groups", 3), "multiple of groups"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("norm_groups", 7), "norm_groups"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("gate_cap", 0.0), "gate_cap"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("keep", 1), "groups"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "kind"),
    (lambda c: c["canon"].__setitem__("taps", 0), "taps"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_what_cannot_be_built_is_refused_in_words(edit, word):
    cfg = pk.random_config((M, S, A), experts=6, top=3, group_count=3, group_keep=2)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        c = config_from_dict(cfg)
        from inferllm_b200.weights import tensor_decls as decls
        decls(c)            # what the configuration reader leaves to the parts is said when they are built
    assert word in str(e.value)


# ---------------------------------------------------------------- the plain implementation against second formulations


def test_matrix_memory_against_its_unstabilised_sum():
    """Without the running maximum: C_t = sum_s exp(i_s + sum_(r in s+1..t) f_r) k_s v_s^T, n_t likewise, and
    o_t = C_t^T q / max(|n_t . q|, 1) in the true (unscaled) numbers, as long as m stays where exp() is harmless; the
    small constant is added in the stabilised numbers."""
    rng = np.random.default_rng(0)
    cfg = pk.random_config((M,), heads=2, dim=8, vdim=6, gate_cap=3.0)
    w, m = f64(pk.random_weights(cfg, 3)), cfg["layers"][0]["mixer"]
    h = rng.standard_normal((25, cfg["width"]))
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w["l0.mix.q"].T).reshape(-1, H, d) / math.sqrt(d)
    k = (h @ w["l0.mix.k"].T).reshape(-1, H, d)
    v = (h @ w["l0.mix.v"].T).reshape(-1, H, dv)
    ig = cap * np.tanh((h @ w["l0.mix.i"].T + w["l0.mix.i.b"]) / cap)
    fg = -np.log1p(np.exp(-cap * np.tanh((h @ w["l0.mix.f"].T + w["l0.mix.f.b"]) / cap)))
    o = np.zeros((25, H, dv))
    for a in range(H):
        for t in range(25):
            wt = np.array([math.exp(ig[s, a] + fg[s + 1:t + 1, a].sum()) for s in range(t + 1)])
            C = np.einsum("s,sd,se->de", wt, k[:t + 1, a], v[:t + 1, a])
            n = wt @ k[:t + 1, a]
            mt = max(max(ig[s, a] + fg[s + 1:t + 1, a].sum() for s in range(t + 1)), fg[:t + 1, a].sum())     # m starts at 0
            o[t, a] = (C.T @ q[t, a]) / (max(abs(n @ q[t, a]), 1.0) + 1e-6 * math.exp(mt))
    y = o / np.sqrt((o * o).mean(-1, keepdims=True) + 1e-5)
    y = y.reshape(25, -1) * w["l0.mix.norm"] * pk.sigmoid(h @ w["l0.mix.g"].T)
    assert np.allclose(pk.mlstm_mixer(h, w, "l0.mix.", m, 1e-5), y @ w["l0.mix.o"].T, rtol=1e-9, atol=1e-11)


def test_state_space_against_its_attention_form():
    """The dual form: y_t = sum_(s<=t) (C_t . B_s) exp(sum_(r in s+1..t) log a_r) dt_s x_s + D x_t."""
    rng = np.random.default_rng(1)
    cfg = pk.random_config((S,), ssm_heads=4, ssm_vdim=5, state=7, groups=2, norm_groups=1, conv=3)
    w, m = f64(pk.random_weights(cfg, 4)), cfg["layers"][0]["mixer"]
    h = rng.standard_normal((20, cfg["width"]))
    H, dv, N, G = 4, 5, 7, 2
    inner = H * dv
    p = h @ w["l0.mix.in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    pad = np.concatenate([np.zeros((2, xbc.shape[1])), xbc])
    conv = sum(pad[j:j + 20] * w["l0.mix.conv"][:, j] for j in range(3)) + w["l0.mix.conv.b"]
    xbc = conv / (1 + np.exp(-conv))
    x, B, C = xbc[:, :inner].reshape(20, H, dv), xbc[:, inner:inner + G * N].reshape(20, G, N), xbc[:, inner + G * N:].reshape(20, G, N)
    dt = np.log1p(np.exp(dt + w["l0.mix.dt_bias"]))
    la = -np.exp(w["l0.mix.A_log"]) * dt
    y = np.zeros((20, H, dv))
    for a in range(H):
        g = a // 2
        for t in range(20):
            for s in range(t + 1):
                y[t, a] += (C[t, g] @ B[s, g]) * math.exp(la[s + 1:t + 1, a].sum()) * dt[s, a] * x[s, a]
            y[t, a] += w["l0.mix.D"][a] * x[t, a]
    y = y.reshape(20, inner) * (z / (1 + np.exp(-z)))
    y = y / np.sqrt((y * y).mean(-1, keepdims=True) + 1e-5) * w["l0.mix.norm"]
    assert np.allclose(pk.mamba2_mixer(h, w, "l0.mix.", m, 1e-5), y @ w["l0.mix.o"].T, rtol=1e-9, atol=1e-11)


def test_attention_against_a_masked_matrix():
    rng = np.random.default_rng(2)
    cfg = pk.random_config((A,), att_heads=4, kv_heads=2, att_dim=8, window=6, scale=0.8)
    w, m = f64(pk.random_weights(cfg, 5)), cfg["layers"][0]["mixer"]
    n = 19
    h = rng.standard_normal((n, cfg["width"]))
    q = (h @ w["l0.mix.q"].T).reshape(n, 4, 8)
    k = np.repeat((h @ w["l0.mix.k"].T).reshape(n, 2, 8), 2, axis=1)
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    dist = np.maximum(i - j, 0)
    s = np.einsum("ihd,jhd->hij", q, k) * 0.8 - w["l0.mix.r1"][:, None, None] * np.log(1 + w["l0.mix.r2"][:, None, None] * dist)
    s = np.einsum("hg,gij->hij", w["l0.mix.talk"], s)
    s = np.where((j <= i) & (i - j < 6), s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    o = np.einsum("hij,jhd->ihd", p, k).reshape(n, 32) * pk.sigmoid(h @ w["l0.mix.g"].T)
    assert np.allclose(pk.attention_mixer(h, w, "l0.mix.", m), o @ w["l0.mix.o"].T, rtol=1e-9, atol=1e-11)


def test_routing_against_a_mask_over_all_experts():
    """Groups, correction and weights restated with masks: the choice uses corrected scores inside the kept groups, a
    negative corrected score still beats an expert outside them, and the weights are the plain scores."""
    rng = np.random.default_rng(3)
    cfg = pk.random_config((A,), experts=8, top=3, group_count=4, group_keep=2)
    w, mlp = f64(pk.random_weights(cfg, 6)), cfg["layers"][0]["mlp"]
    w["l0.mlp.correction"] = w["l0.mlp.correction"] - 0.5           # all corrected scores negative for most tokens
    h = rng.standard_normal((40, cfg["width"]))
    z = h @ w["l0.mlp.router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    c = s + w["l0.mlp.correction"]
    assert (c < 0).all(-1).any()
    gs = c.reshape(40, 4, 2).max(-1)
    kept = np.argsort(-gs, axis=-1, kind="stable")[:, :2]
    mask = np.full((40, 8), -np.inf)
    for t in range(40):
        for g in kept[t]:
            mask[t, 2 * g:2 * g + 2] = 0.0
    pick = np.argsort(-(c + mask), axis=-1, kind="stable")[:, :3]
    chosen, weights = pk.route(h, w, "l0.mlp.", mlp["router"])
    assert [sorted(x) for x in chosen] == [sorted(x) for x in pick.tolist()]
    for t in range(40):
        assert np.allclose(weights[t], s[t, chosen[t]])
    dense = np.zeros((40, cfg["width"]))
    for e in range(8):
        on = np.array([e in chosen[t] for t in range(40)])
        dense += (on * s[:, e])[:, None] * pk.expert(h, w, "l0.mlp.e%d." % e)
    dense += pk.expert(h, w, "l0.mlp.shared.")
    assert np.allclose(pk.moe(h, w, "l0.mlp.", mlp), dense, rtol=1e-9, atol=1e-11)


def test_convolution_and_norm_restated():
    rng = np.random.default_rng(4)
    h, taps = rng.standard_normal((9, 5)), rng.standard_normal((5, 4))
    pad = np.concatenate([np.zeros((3, 5)), h])
    assert np.allclose(pk.causal_conv(h, taps), sum(pad[j:j + 9] * taps[:, j] for j in range(4)))
    x, g = rng.standard_normal((3, 11)), rng.standard_normal(11)
    assert np.allclose(pk.layer_norm(x, g, 1e-3), (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-3) * g)
    e = pk.embed([2, 0], np.arange(12.0).reshape(3, 4), 0.5, first_pos=3)
    assert np.allclose(e[1], np.array([0, 1, 2, 3]) * 0.5 + [math.sin(4), math.cos(4), math.sin(4 * 0.01), math.cos(4 * 0.01)])
