"""The Tukulorn configuration class and the plain implementation's own pieces, on the CPU.

What config.json says must arrive in the ModelSpec unchanged (sizes, constants, layer order), the tensors the model
declares must be the file's names and shapes, and a configuration that cannot be built is refused in words.  The plain
implementation's mechanisms are checked against second, independent formulations of the same equations.
"""
import cmath
import math

import numpy as np
import pytest
import plain_tukulorn as pt

from inferllm_b200 import ConfigError, TukulornConfig, config_from_dict
from inferllm_b200.weights import tensor_decls

D, L = "attention", "latent_attention"


def f64(w):
    return {k: np.asarray(v, np.float64) for k, v in w.items()}


def sample_config():
    return pt.make_config([(D, pt.diff_mixer(heads=6, kv_heads=3, dim=10, vdim=14, diff=0.35, scale=0.37, coef=0.4, every=33), pt.dense(52)),
                           (L, pt.latent_mixer(heads=5, dim=12, rot_dim=6, vdim=9, kv_rank=22, window=31, scale=0.21, base=777.0),
                            pt.routed(experts=8, top=3, count=4, keep=2, ff=22, limit=1.75, scale=2.25)),
                           (D, pt.diff_mixer(every=0), None),
                           (L, pt.latent_mixer(window=0), pt.routed(count=0))], width=56, vocab=77, eps=3e-5, loop=(1, 3, 3))


def test_spec_carries_every_size_and_constant():
    spec = config_from_dict(sample_config()).model_spec()
    assert (spec.hidden_size, spec.vocab_size) == (56, 77)
    # the loop unrolls: layers 1 and 2 three times, a cache entry per run, every pass but the first re-enters
    assert [(e.layer, e.cache, e.writes, e.reenter) for e in spec.schedule] == \
        [(0, 0, True, False), (1, 1, True, False), (2, 2, True, False), (1, 3, True, True), (2, 4, True, False), (1, 5, True, True),
         (2, 6, True, False), (3, 7, True, False)]
    assert spec.reentry.kind == "add_embedding"
    assert [l.block for l in spec.layers] == ["prenorm_scaled", "prenorm_scaled", "prenorm_scaled_mixer", "prenorm_scaled"]
    assert sorted(spec.layers[0].norms) == ["ls1", "ls2", "norm1", "norm2"] and sorted(spec.layers[2].norms) == ["ls1", "norm1"]
    for l in spec.layers:
        assert l.norms["norm1"].kind == "rmsnorm" and l.norms["norm1"]["eps"] == 3e-5 and l.norms["norm1"]["weight_offset"] == 1.0
        assert l.norms["ls1"].kind == "layer_scale" and l.norms["ls1"]["size"] == 56
    a, b = spec.layers[0].mixer, spec.layers[1].mixer
    assert (a.kind, b.kind) == ("attention", "latent_attention")
    assert (a["n_heads"], a["n_kv_heads"], a["head_dim"], a["v_head_dim"], a["score_maps"], a["diff"], a["scale"]) == (6, 3, 10, 14, 2, 0.35, 0.37)
    assert a["q_temperature"] == {"coef": 0.4, "every": 33} and a["qkv_bias"] is True and a["o_bias"] is True and a["norm_eps"] == 3e-5
    assert "q_temperature" not in spec.layers[2].mixer.params
    assert (b["n_heads"], b["head_dim"], b["rot_head_dim"], b["v_head_dim"], b["kv_rank"], b["q_rank"], b["window"], b["scale"]) == (5, 12, 6, 9, 22, 0, 31, 0.21)
    pos = b["position"]
    assert pos.kind == "rope_pairs" and (pos["theta"], pos["rot_dim"], pos["head_dim"]) == (777.0, 6, 6)
    assert b["out_gate"] == "head_sigmoid" and spec.layers[3].mixer["window"] == 0
    dense, moe, bare = spec.layers[0].ffn, spec.layers[1].ffn, spec.layers[3].ffn
    assert dense.kind == "gated_mlp" and (dense["intermediate_size"], dense["activation"]) == (52, "silu") and spec.layers[2].ffn.kind == ""
    assert (moe["experts"], moe["top"], moe["intermediate_size"], moe["scoring"], moe["group_score_top"]) == (8, 3, 22, "sigmoid", 2)
    assert (moe["weight_scale"], moe["activation"], moe["activation_limit"], moe["sum_eps"]) == (2.25, "swish_clamped", 1.75, 1e-20)
    assert moe["groups"] == {"count": 4, "keep": 2} and "groups" not in bare.params
    assert spec.head["tied"] is False and spec.final_norm["weight_offset"] == 1.0 and spec.embedding.kind == "embedding"


def test_without_a_loop_nothing_of_it_exists():
    cfg = pt.make_config([(D, pt.diff_mixer(), None), (L, pt.latent_mixer(), pt.dense())])
    spec = config_from_dict(cfg).model_spec()
    assert [(e.layer, e.cache, e.reenter) for e in spec.schedule] == [(0, 0, False), (1, 1, False)]
    assert spec.reentry is None or spec.reentry.kind == ""
    once = pt.make_config([(D, pt.diff_mixer(), None), (L, pt.latent_mixer(), pt.dense())], loop=(0, 2, 1))
    assert not any(e.reenter for e in config_from_dict(once).model_spec().schedule)


def test_the_python_face_is_typed_and_round_trips():
    c = config_from_dict(sample_config())
    assert isinstance(c, TukulornConfig) and c.architecture == "Tukulorn"
    assert TukulornConfig.from_dict(c.to_dict()) == c and c.to_dict()["width"] == 56


def test_declared_tensors_are_the_files_names_and_shapes():
    cfg = sample_config()
    decls = {name: tuple(shape) for name, (shape, _) in tensor_decls(config_from_dict(cfg)).items()}
    assert decls == {k: tuple(v[0]) for k, v in pt.tensor_shapes(cfg).items()}


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 4), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].__setitem__("every", 0), "every"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 5), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_rank", 0), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 3), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("keep", 1), "groups"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c["loop"].__setitem__("times", 0), "loop"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_what_cannot_be_built_is_refused_in_words(edit, word):
    cfg = sample_config()
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        tensor_decls(config_from_dict(cfg))      # what the configuration reader leaves to the parts is said when they are built
    assert word in str(e.value)


# ---------------------------------------------------------------- the plain implementation against second formulations


def test_differential_attention_against_its_matrix_form():
    """Both maps as masked matrix softmaxes over the key heads repeated per query head."""
    rng = np.random.default_rng(0)
    m = pt.diff_mixer(heads=4, kv_heads=2, dim=6, vdim=10, diff=0.3, scale=0.7, coef=0.5, every=3)
    cfg = pt.make_config([(D, m, None)])
    w = f64(pt.random_weights(cfg, 3))
    n = 17
    h = rng.standard_normal((n, cfg["width"]))
    q = (h @ w["l0.mix.q"].T + w["l0.mix.q.b"]).reshape(n, 4, 2, 6)
    q = q * np.array([1 + 0.5 * math.log((p + 1) // 3 + 1) for p in range(n)])[:, None, None, None]
    k = np.repeat((h @ w["l0.mix.k"].T + w["l0.mix.k.b"]).reshape(n, 2, 2, 6), 2, axis=1)
    v = np.repeat((h @ w["l0.mix.v"].T + w["l0.mix.v.b"]).reshape(n, 2, 10), 2, axis=1)
    s = np.einsum("ihcd,jhcd->hcij", q, k) * 0.7
    s = np.where(np.tril(np.ones((n, n), bool)), s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    a = np.einsum("hcij,jhe->cihe", p, v)
    lam = math.exp(w["l0.mix.lq1"] @ w["l0.mix.lk1"]) - math.exp(w["l0.mix.lq2"] @ w["l0.mix.lk2"]) + 0.3
    o = a[0] - lam * a[1]
    o = o / np.sqrt((o * o).mean(-1, keepdims=True) + 1e-5) * 0.7
    want = o.reshape(n, -1) @ w["l0.mix.o"].T + w["l0.mix.o.b"]
    assert np.allclose(pt.differential_attention(h, w, "l0.mix.", m, 1e-5), want, rtol=1e-9, atol=1e-11)


def test_pair_rotation_against_complex_numbers():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 12))
    for p in (0, 1, 37):
        z = (x[:, 0:8:2] + 1j * x[:, 1:8:2]) * np.array([cmath.exp(1j * p * 50.0 ** (-2.0 * i / 8)) for i in range(4)])
        y = pt.rotate_pairs(x, p, 50.0, 8)
        assert np.allclose(y[:, 0:8:2], z.real) and np.allclose(y[:, 1:8:2], z.imag) and np.array_equal(y[:, 8:], x[:, 8:])


def test_latent_attention_against_its_absorbed_form():
    """score = (U_k^T q) . c + rot(q_r) . rot(k_r) and o = U_v (sum p c): nothing but the latent and the shared part is
    needed per key; the rotated product depends on the distance alone."""
    rng = np.random.default_rng(2)
    m = pt.latent_mixer(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=14, window=5, scale=0.4, base=20.0)
    cfg = pt.make_config([(L, m, None)])
    w = f64(pt.random_weights(cfg, 5))
    n = 19
    h = rng.standard_normal((n, cfg["width"]))
    q = (h @ w["l0.mix.q"].T).reshape(n, 3, 12)
    down = h @ w["l0.mix.dkv"].T
    c = down[:, :14] / np.sqrt((down[:, :14] ** 2).mean(-1, keepdims=True) + 1e-5) * w["l0.mix.dkv.norm"]
    uk, uv = w["l0.mix.uk"].reshape(3, 8, 14), w["l0.mix.uv"].reshape(3, 6, 14)
    gate = 1 / (1 + np.exp(-(h @ w["l0.mix.g"].T)))
    out = np.zeros((n, 3, 6))
    for i in range(n):
        for a in range(3):
            qa = uk[a].T @ q[i, a, :8]
            sc = []
            for j in range(max(0, i - 4), i + 1):
                # the rotated parts as complex numbers: conj(q_r e^(i p)) (k_r e^(i j)) depends on j - i
                zq = q[i, a, 8::2] + 1j * q[i, a, 9::2]
                zk = down[j, 14::2] + 1j * down[j, 15::2]
                turn = np.array([cmath.exp(1j * (j - i) * 20.0 ** (-2.0 * t / 4)) for t in range(2)])
                sc.append((qa @ c[j] + (np.conj(zq) * zk * turn).real.sum()) * 0.4)
            p = np.exp(np.array(sc) - max(sc))
            p /= p.sum()
            out[i, a] = uv[a] @ (p @ c[max(0, i - 4):i + 1]) * gate[i, a]
    assert np.allclose(pt.latent_attention(h, w, "l0.mix.", m, 1e-5), out.reshape(n, -1) @ w["l0.mix.o"].T, rtol=1e-9, atol=1e-11)


def test_routing_rules():
    """Hand-made scores: the best expert alone does not save its group; the weights sum to router.scale."""
    r = {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}
    z = np.log(np.array([[0.9, 0.05, 0.6, 0.5, 0.1, 0.1]]) / (1 - np.array([[0.9, 0.05, 0.6, 0.5, 0.1, 0.1]])))     # sigmoid(z) = those scores
    W = {"r.router": np.eye(6)}
    chosen, weights = pt.route(z, W, "r.", r)
    assert chosen == [[2, 3]]                                # group 1 (0.6 + 0.5) beats group 0 (0.9 + 0.05)
    assert np.allclose(weights[0], [3.0 * 0.6 / 1.1, 3.0 * 0.5 / 1.1])
    r["groups"] = {"count": 1, "keep": 1}
    chosen, weights = pt.route(z, W, "r.", r)
    assert chosen == [[0, 2]] and math.isclose(sum(weights[0]), 3.0)


def test_expert_limits():
    """The gate is cut from above only, the up projection on both sides."""
    W = {"e.gate": np.array([[1.0]]), "e.up": np.array([[1.0]]), "e.down": np.array([[1.0]])}
    def f(x): return float(pt.expert(np.array([[x]]), W, "e.", 2.0)[0, 0])
    assert math.isclose(f(5.0), 2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0)
    assert math.isclose(f(-5.0), -5.0 / (1 + math.exp(1.702 * 5.0)) * (-2.0 + 1.0))
    assert math.isclose(f(0.5), 0.5 / (1 + math.exp(-1.702 * 0.5)) * 1.5)


def test_loop_adds_the_embedding_before_every_pass_but_the_first():
    cfg = pt.make_config([(D, pt.diff_mixer(), pt.dense()), (L, pt.latent_mixer(), None)], loop=(1, 2, 3))
    assert pt.layer_order(cfg) == [(0, False), (1, False), (1, True), (1, True)]
    w = f64(pt.random_weights(cfg, 1))
    ids = [3, 9, 27, 81, 5]
    layers = []
    pt.forward(cfg, w, ids, layers)
    x0 = w["embed"][ids]
    h = pt.zero_centred_norm(layers[1] + x0, w["l1.norm1"], cfg["norm"]["eps"])
    want = layers[1] + x0 + pt.latent_attention(h, w, "l1.mix.", cfg["layers"][1]["mixer"], cfg["norm"]["eps"]) * w["l1.ls1"]
    assert np.allclose(layers[2], want)
