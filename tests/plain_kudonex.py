"""A plain, slow implementation of the Kudonex decoder in float64 numpy: one function per mechanism, every
recurrence and every attention row a literal loop.  It shares nothing with the library; the GPU tests compare the
engine with it.

A model is (cfg, W): cfg the config.json object, W a dict name -> float64 array.  Everything runs on one
sequence: x is [n, width], the first token has position 0.
"""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis, var the mean squared deviation; no bias."""
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def causal_conv(h, w, bias=None):
    """y_t[c] = sum_j w[c, j] * h_(t - taps + 1 + j)[c] (+ bias[c]); rows before the sequence are zero."""
    n, taps = h.shape[0], w.shape[1]
    y = np.zeros_like(h)
    for t in range(n):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * h[s]
    if bias is not None:
        y += bias
    return y


def embed(tokens, table, scale, first_pos=0):
    """table[token] * scale plus the sinusoid vector: entry 2i sin(p * 10000^(-2i / width)), entry 2i + 1 its cosine."""
    width = table.shape[1]
    x = table[np.asarray(tokens)] * scale
    for r in range(len(tokens)):
        p = first_pos + r
        for c in range(width):
            ang = p * 10000.0 ** (-(2 * (c // 2)) / width)
            x[r, c] += math.sin(ang) if c % 2 == 0 else math.cos(ang)
    return x


def mlstm_mixer(h, W, pre, m, eps):
    """The matrix memory with exponential gating and a running maximum that starts at 0."""
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    n = h.shape[0]
    q = (h @ W[pre + "q"].T).reshape(n, H, d) * d ** -0.5
    k = (h @ W[pre + "k"].T).reshape(n, H, d)
    v = (h @ W[pre + "v"].T).reshape(n, H, dv)
    ig = cap * np.tanh((h @ W[pre + "i"].T + W[pre + "i.b"]) / cap)
    fg = log_sigmoid(cap * np.tanh((h @ W[pre + "f"].T + W[pre + "f.b"]) / cap))
    out = np.zeros((n, H, dv))
    for a in range(H):
        S, nv, mx = np.zeros((d, dv)), np.zeros(d), 0.0
        for t in range(n):
            new = max(fg[t, a] + mx, ig[t, a])
            keep, put = math.exp(fg[t, a] + mx - new), math.exp(ig[t, a] - new)
            S = keep * S + put * np.outer(k[t, a], v[t, a])
            nv = keep * nv + put * k[t, a]
            mx = new
            out[t, a] = (S.T @ q[t, a]) / (max(abs(nv @ q[t, a]), math.exp(-mx)) + 1e-6)
    y = rms_unit(out, eps).reshape(n, H * dv) * W[pre + "norm"] * sigmoid(h @ W[pre + "g"].T)
    return y @ W[pre + "o"].T


def mamba2_mixer(h, W, pre, m, eps):
    """The selective state space in its scalar-decay (duality) form."""
    H, dv, N, G, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    n, inner = h.shape[0], m["heads"] * m["vdim"]
    p = h @ W[pre + "in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[pre + "conv"], W[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(n, H, dv)
    Bm = xbc[:, inner:inner + G * N].reshape(n, G, N)
    Cm = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + W[pre + "dt_bias"])
    y = np.zeros((n, H, dv))
    for a in range(H):
        g = a // (H // G)
        S = np.zeros((N, dv))
        for t in range(n):
            S = math.exp(-math.exp(W[pre + "A_log"][a]) * dt[t, a]) * S + dt[t, a] * np.outer(Bm[t, g], x[t, a])
            y[t, a] = S.T @ Cm[t, g] + W[pre + "D"][a] * x[t, a]
    y = y.reshape(n, inner) * silu(z)
    y = rms_unit(y.reshape(n, parts, inner // parts), eps).reshape(n, inner) * W[pre + "norm"]
    return y @ W[pre + "o"].T


def attention_mixer(h, W, pre, m):
    """Softmax attention over a sliding window whose values are the keys, with a logarithmic distance penalty and the
    heads' scores mixed by a matrix before the softmax; an element-wise sigmoid gate on the way out."""
    H, G, d, window, scale = m["heads"], m["kv_heads"], m["dim"], m["mask"]["size"] if m.get("mask") else 0, m["scale"]
    n = h.shape[0]
    q = (h @ W[pre + "q"].T).reshape(n, H, d)
    k = (h @ W[pre + "k"].T).reshape(n, G, d)
    out = np.zeros((n, H, d))
    for i in range(n):
        lo = max(0, i - window + 1) if window else 0
        js = np.arange(lo, i + 1)
        s = np.zeros((H, len(js)))
        for a in range(H):
            s[a] = (k[js, a // (H // G)] @ q[i, a]) * scale - W[pre + "r1"][a] * np.log1p(W[pre + "r2"][a] * (i - js))
        s = W[pre + "talk"] @ s
        for a in range(H):
            e = np.exp(s[a] - s[a].max())
            out[i, a] = (e / e.sum()) @ k[js, a // (H // G)]
    y = out.reshape(n, H * d) * sigmoid(h @ W[pre + "g"].T)
    return y @ W[pre + "o"].T


def expert(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def route(h, W, pre, r, margins=None):
    """Per token: the chosen experts and their weights.  Softmax over all experts; the choice adds a correction and is
    confined to the best groups (a group's score: its largest corrected score); the weights are the plain scores.
    `margins` (a list) receives per token how far the choice is from another one: the smaller of the gap between the
    last kept and the first dropped group and the gap between the last chosen and the first unchosen allowed expert."""
    E, top = r["experts"], r["top"]
    count, keep = (r["groups"]["count"], r["groups"]["keep"]) if r.get("groups") else (1, 1)
    z = h @ W[pre + "router"].T
    chosen, weights = [], []
    for t in range(h.shape[0]):
        e = np.exp(z[t] - z[t].max())
        s = e / e.sum()
        c = s + W[pre + "correction"] if pre + "correction" in W else s.copy()
        per = E // count
        gscore = [c[g * per:(g + 1) * per].max() for g in range(count)]
        kept = sorted(range(count), key=lambda g: (-gscore[g], g))[:keep]
        allowed = [x for x in range(E) if x // per in kept]
        ranked = sorted(allowed, key=lambda x: (-c[x], x))
        pick = ranked[:top]
        chosen.append(pick)
        weights.append([s[x] for x in pick])
        if margins is not None:
            by_group = sorted(gscore, reverse=True)
            gap_g = by_group[keep - 1] - by_group[keep] if keep < count else math.inf
            gap_e = c[ranked[top - 1]] - c[ranked[top]] if top < len(ranked) else math.inf
            margins.append(min(gap_g, gap_e))
    return chosen, weights


def moe(h, W, pre, mlp, margins=None):
    chosen, weights = route(h, W, pre, mlp["router"], margins)
    y = np.zeros((h.shape[0], W[pre + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for x, w in zip(chosen[t], weights[t]):
            y[t] += w * expert(h[t:t + 1], W, pre + "e%d." % x)[0]
    if mlp.get("shared"):
        y += expert(h, W, pre + "shared.")
    return y


def forward(cfg, W, tokens, layers_out=None, margins_out=None):
    """Logits [n, vocab] of one sequence from its first token; layers_out (a list) receives the stream after every layer,
    margins_out (a list) one list per routed feed-forward with every token's distance from another choice of experts."""
    eps = cfg["norm"]["eps"]
    x = embed(tokens, W["embed"], cfg["embedding"]["scale"])
    for i, L in enumerate(cfg["layers"]):
        pre = "l%d." % i
        h = layer_norm(x, W[pre + "norm1"], eps)
        if cfg.get("canon"):
            h = h + causal_conv(h, W[pre + "canon1"])
        if L["type"] == "mlstm":
            y = mlstm_mixer(h, W, pre + "mix.", L["mixer"], eps)
        elif L["type"] == "mamba2":
            y = mamba2_mixer(h, W, pre + "mix.", L["mixer"], eps)
        elif L["type"] == "attention":
            y = attention_mixer(h, W, pre + "mix.", L["mixer"])
        else:
            raise ValueError(L["type"])
        x = x + layer_norm(y, W[pre + "norm1b"], eps)
        if L.get("mlp"):
            if margins_out is not None:
                margins_out.append([])
            y = moe(layer_norm(x, W[pre + "norm2"], eps), W, pre + "mlp.", L["mlp"], margins_out[-1] if margins_out is not None else None)
            x = x + layer_norm(y, W[pre + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return layer_norm(x, W["final.norm"], eps) @ W["embed"].T


def choice_margin(cfg, W, tokens):
    """Per position the smallest distance of any of its routers from another choice of experts (infinite without one)."""
    m = []
    forward(cfg, W, tokens, None, m)
    return np.min(np.asarray(m, np.float64), 0) if m else np.full(len(tokens), math.inf)


def amplification(cfg, W, tokens, rel=1e-7):
    """By how much the model enlarges a small relative change of its embedding table on the way to the logits, per
    position (1: not at all).  A unit norm or a layer norm over a vector that happens to be tiny (the matrix memory's
    read-out at a first token whose query and key are nearly orthogonal, say) enlarges every rounding before it."""
    ref = forward(cfg, W, tokens)
    W2 = dict(W)
    W2["embed"] = W["embed"] * (1.0 + rel * np.random.default_rng(0).standard_normal(W["embed"].shape))
    return np.abs(forward(cfg, W2, tokens) - ref).max(-1) / np.abs(ref).max() / rel


def greedy_generate(cfg, W, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(np.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]


# ---------------------------------------------------------------- test infrastructure: configurations and weights


def random_config(types, width=48, vocab=97, taps=3, emb_scale=2.0, eps=1e-5, heads=2, dim=16, vdim=24, gate_cap=10.0, ssm_heads=4, ssm_vdim=12,
                  state=16, groups=2, norm_groups=2, conv=3, att_heads=4, kv_heads=2, att_dim=16, window=20, scale=0.5, experts=6, top=2,
                  group_count=3, group_keep=2, expert_ff=24, shared_ff=40, mlps=None, max_positions=2048):
    """A small configuration: `types` names the mixers, `mlps` says per layer whether it has a feed-forward (True,
    "bare": one without groups and without a shared expert, or None); all if not given."""
    layers = []
    for i, t in enumerate(types):
        if t == "mlstm":
            m = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}
        elif t == "mamba2":
            m = {"heads": ssm_heads, "vdim": ssm_vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}
        else:
            m = {"heads": att_heads, "kv_heads": kv_heads, "dim": att_dim, "vdim": att_dim, "scale": scale}
            if window:
                m["mask"] = {"size": window}
        kind = mlps[i] if mlps is not None else True
        mlp = None
        if kind:
            mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}}
            if kind != "bare":
                mlp["router"]["groups"] = {"count": group_count, "keep": group_keep}
                mlp["shared"] = {"ff": shared_ff}
        layers.append({"type": t, "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Kudonex", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": emb_scale}, "layers": layers,
           "max_positions": max_positions}
    if taps:
        cfg["canon"] = {"taps": taps}
    return cfg


def tensor_shapes(cfg):
    """name -> (shape, kind); kind says how random_weights draws the tensor."""
    width, out = cfg["width"], {"embed": ((cfg["vocab"], cfg["width"]), "embed"), "final.norm": ((cfg["width"],), "norm")}
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L.get("mlp") else ()):
            out[p + n] = ((width,), "norm")
        if cfg.get("canon"):
            out[p + "canon1"] = ((width, cfg["canon"]["taps"]), "taps")
        x = p + "mix."
        if L["type"] == "mlstm":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out.update({x + "q": ((H * d, width), "mat"), x + "k": ((H * d, width), "mat"), x + "v": ((H * dv, width), "mat"),
                        x + "g": ((H * dv, width), "mat"), x + "o": ((width, H * dv), "mat"), x + "norm": ((H * dv,), "norm"),
                        x + "i": ((H, width), "mat"), x + "i.b": ((H,), "bias"), x + "f": ((H, width), "mat"), x + "f.b": ((H,), "fbias")})
        elif L["type"] == "mamba2":
            H, dv, N, G, c = m["heads"], m["vdim"], m["state"], m["groups"], m.get("conv", 1)
            inner, ch = H * dv, H * dv + 2 * G * N
            out.update({x + "in": ((2 * inner + 2 * G * N + H, width), "mat"), x + "conv": ((ch, c), "taps"), x + "conv.b": ((ch,), "bias"),
                        x + "dt_bias": ((H,), "bias"), x + "A_log": ((H,), "alog"), x + "D": ((H,), "norm"), x + "norm": ((inner,), "norm"),
                        x + "o": ((width, inner), "mat")})
        else:
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            out.update({x + "q": ((H * d, width), "mat"), x + "k": ((G * d, width), "mat"), x + "g": ((H * d, width), "mat"),
                        x + "o": ((width, H * d), "mat"), x + "r1": ((H,), "r1"), x + "r2": ((H,), "r2"), x + "talk": ((H, H), "talk")})
        if L.get("mlp"):
            f, r = p + "mlp.", L["mlp"]["router"]
            out[f + "router"] = ((r["experts"], width), "router")
            out[f + "correction"] = ((r["experts"],), "correction")
            blocks = [(f + "e%d." % e, L["mlp"]["expert"]["ff"]) for e in range(r["experts"])]
            if L["mlp"].get("shared"):
                blocks.append((f + "shared.", L["mlp"]["shared"]["ff"]))
            for b, ff in blocks:
                out.update({b + "gate": ((ff, width), "mat"), b + "up": ((ff, width), "mat"), b + "down": ((width, ff), "mat")})
    return out


def bf16_round(a):
    """float32 array rounded to the nearest bfloat16 value (ties to even), still float32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def random_weights(cfg, seed, gain=1.0):
    """Random weights, rounded to bfloat16 values.  Drawn so that faults show: router logits are spread (a wrong expert
    changes the row), corrections have both signs and are large enough to change the choice, decay rates run from slow
    to fast, the distance factors and the head mix are far from 0 and the identity."""
    rng, w = np.random.default_rng(seed), {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        n_in = shape[-1]
        if kind == "mat":
            a = rng.standard_normal(shape) * gain / math.sqrt(n_in)
        elif kind == "embed":
            a = rng.standard_normal(shape)
        elif kind == "norm":
            a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif kind == "taps":
            a = 0.5 * rng.standard_normal(shape)
        elif kind == "bias":
            a = 0.5 * rng.standard_normal(shape)
        elif kind == "fbias":
            a = 2.0 + rng.standard_normal(shape)
        elif kind == "alog":
            a = np.linspace(-4.0, 0.5, shape[0])
        elif kind == "r1":
            a = 0.3 + rng.random(shape)
        elif kind == "r2":
            a = 0.2 + 2.0 * rng.random(shape)
        elif kind == "talk":
            a = np.eye(shape[0]) + 0.4 * rng.standard_normal(shape)
        elif kind == "router":
            a = rng.standard_normal(shape) * 6.0 / math.sqrt(n_in)
        elif kind == "correction":
            a = 0.15 * rng.standard_normal(shape)
        else:
            raise ValueError(kind)
        w[name] = bf16_round(a.astype(np.float32))
    return w


def write_model(folder, cfg, w):
    """config.json and model.safetensors (bfloat16) of (cfg, w) in `folder`."""
    import json
    import os
    import struct
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, a in w.items():
        blob = (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [off, off + len(blob)]}
        blobs.append(blob)
        off += len(blob)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
