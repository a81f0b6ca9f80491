"""A plain, slow implementation of the Tukulorn decoder in float64 numpy: one function per mechanism, every attention
row a literal loop over its keys.  It shares nothing with the library; the GPU tests compare the engine with it.

A model is (cfg, W): cfg the config.json object, W a dict name -> float64 array.  Everything runs on one
sequence: x is [n, width], the first token has position 0.
"""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def zero_centred_norm(x, w, eps):
    """x / rms(x) * (1 + w): the weight is stored around zero."""
    return rms_unit(x, eps) * (1.0 + w)


def softmax_row(s):
    e = np.exp(s - s.max())
    return e / e.sum()


def query_temperature(p, t):
    """The factor on a query at position p: it grows by steps, one every `every` positions."""
    return 1.0 + t["coef"] * math.log((p + 1) // t["every"] + 1)


def differential_lambda(W, pre, diff):
    return math.exp(float(W[pre + "lq1"] @ W[pre + "lk1"])) - math.exp(float(W[pre + "lq2"] @ W[pre + "lk2"])) + diff


def differential_attention(h, W, pre, m, eps, first_pos=0):
    """Causal attention with two score maps per head over the same values: o = a1 - lambda a2, then a unit norm per head
    and the factor 1 - diff.  Biases on q, k, v and the output map; no rotation, but a temperature on the queries."""
    H, G, d, dv, diff, scale = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"], m["scale"]
    n = h.shape[0]
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).reshape(n, H, 2, d)
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).reshape(n, G, 2, d)
    v = (h @ W[pre + "v"].T + W[pre + "v.b"]).reshape(n, G, dv)
    if m.get("q_temp"):
        for i in range(n):
            q[i] *= query_temperature(first_pos + i, m["q_temp"])
    lam = differential_lambda(W, pre, diff)
    out = np.zeros((n, H, dv))
    for i in range(n):
        for a in range(H):
            g = a // (H // G)
            maps = []
            for c in range(2):
                s = np.array([q[i, a, c] @ k[j, g, c] for j in range(i + 1)]) * scale
                maps.append(softmax_row(s) @ v[:i + 1, g])
            out[i, a] = rms_unit(maps[0] - lam * maps[1], eps) * (1.0 - diff)
    return out.reshape(n, H * dv) @ W[pre + "o"].T + W[pre + "o.b"]


def rotate_pairs(x, p, base, dims):
    """Channels (2i, 2i + 1) of the first `dims` channels of x turned by the angle p * base^(-2i / dims)."""
    y = np.array(x, np.float64)
    for i in range(dims // 2):
        a = p * base ** (-2.0 * i / dims)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        y[..., 2 * i] = u * math.cos(a) - v * math.sin(a)
        y[..., 2 * i + 1] = v * math.cos(a) + u * math.sin(a)
    return y


def latent_attention(h, W, pre, m, eps, first_pos=0):
    """Attention whose keys and values are maps of one normed latent per token, beside one rotated key part that all
    heads share; a sliding window; a sigmoid gate per head on the way out."""
    H, d, dr, dv, rank, scale = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"]
    window = m["mask"]["size"] if m.get("mask") else 0
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    n = h.shape[0]
    q = (h @ W[pre + "q"].T).reshape(n, H, d + dr)
    down = h @ W[pre + "dkv"].T
    c = rms_unit(down[:, :rank], eps) * W[pre + "dkv.norm"]
    kr = np.stack([rotate_pairs(down[t, rank:], first_pos + t, base, dims) for t in range(n)])
    k = (c @ W[pre + "uk"].T).reshape(n, H, d)
    v = (c @ W[pre + "uv"].T).reshape(n, H, dv)
    gate = sigmoid(h @ W[pre + "g"].T)
    out = np.zeros((n, H, dv))
    for i in range(n):
        lo = max(0, i - window + 1) if window else 0
        for a in range(H):
            qr = rotate_pairs(q[i, a, d:], first_pos + i, base, dims)
            s = np.array([q[i, a, :d] @ k[j, a] + qr @ kr[j] for j in range(lo, i + 1)]) * scale
            out[i, a] = (softmax_row(s) @ v[lo:i + 1, a]) * gate[i, a]
    return out.reshape(n, H * dv) @ W[pre + "o"].T


def dense_mlp(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def expert(h, W, pre, limit):
    g = np.minimum(h @ W[pre + "gate"].T, limit)
    u = np.clip(h @ W[pre + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[pre + "down"].T


def route(h, W, pre, r, margins=None):
    """Per token: the chosen experts and their weights.  Scores are sigmoids of the router's logits; a group's score is
    the sum of its two largest scores, only experts of the best groups can be chosen; the weights are the chosen scores
    over their sum, times router.scale.  `margins` (a list) receives per token how far the choice is from another."""
    E, top = r["experts"], r["top"]
    count, keep = (r["groups"]["count"], r["groups"]["keep"]) if r.get("groups") else (1, 1)
    z = h @ W[pre + "router"].T
    chosen, weights = [], []
    for t in range(h.shape[0]):
        s = sigmoid(z[t])
        per = E // count
        gscore = [float(np.sort(s[g * per:(g + 1) * per])[-2:].sum()) for g in range(count)]
        kept = sorted(range(count), key=lambda g: (-gscore[g], g))[:keep]
        allowed = [x for x in range(E) if x // per in kept]
        ranked = sorted(allowed, key=lambda x: (-s[x], x))
        pick = ranked[:top]
        total = sum(s[x] for x in pick) + 1e-20
        chosen.append(pick)
        weights.append([s[x] / total * r.get("scale", 1.0) for x in pick])
        if margins is not None:
            by_group = sorted(gscore, reverse=True)
            gap_g = by_group[keep - 1] - by_group[keep] if keep < count else math.inf
            gap_e = s[ranked[top - 1]] - s[ranked[top]] if top < len(ranked) else math.inf
            margins.append(min(gap_g, gap_e))
    return chosen, weights


def moe(h, W, pre, mlp, margins=None):
    chosen, weights = route(h, W, pre, mlp["router"], margins)
    y = np.zeros((h.shape[0], W[pre + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for x, w in zip(chosen[t], weights[t]):
            y[t] += w * expert(h[t:t + 1], W, pre + "e%d." % x, mlp["expert"]["limit"])[0]
    return y


def layer_order(cfg):
    """(layer index, whether a pass of the loop starts here that is not the first)."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(lp["start"])]
    for p in range(lp["times"]):
        order += [(i, p > 0 and i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return order + [(i, False) for i in range(lp["stop"], n)]


def forward(cfg, W, tokens, layers_out=None, margins_out=None):
    """Logits [n, vocab] of one sequence from its first token; layers_out (a list) receives the stream after every layer
    run, margins_out (a list) one list per routed feed-forward run with every token's distance from another choice."""
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][np.asarray(tokens)]
    x = x0.copy()
    for i, again in layer_order(cfg):
        L, pre = cfg["layers"][i], "l%d." % i
        if again:
            x = x + x0
        h = zero_centred_norm(x, W[pre + "norm1"], eps)
        if L["type"] == "attention":
            y = differential_attention(h, W, pre + "mix.", L["mixer"], eps)
        elif L["type"] == "latent_attention":
            y = latent_attention(h, W, pre + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + y * W[pre + "ls1"]
        if L.get("mlp"):
            h = zero_centred_norm(x, W[pre + "norm2"], eps)
            if L["mlp"]["kind"] == "dense":
                y = dense_mlp(h, W, pre + "mlp.")
            else:
                if margins_out is not None:
                    margins_out.append([])
                y = moe(h, W, pre + "mlp.", L["mlp"], margins_out[-1] if margins_out is not None else None)
            x = x + y * W[pre + "ls2"]
        if layers_out is not None:
            layers_out.append(x.copy())
    return zero_centred_norm(x, W["final.norm"], eps) @ W["head"].T


def choice_margin(cfg, W, tokens):
    """Per position the smallest distance of any of its routers from another choice of experts (infinite without one)."""
    m = []
    forward(cfg, W, tokens, None, m)
    return np.min(np.asarray(m, np.float64), 0) if m else np.full(len(tokens), math.inf)


def greedy_generate(cfg, W, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(np.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]


# ---------------------------------------------------------------- test infrastructure: configurations and weights


def diff_mixer(heads=4, kv_heads=2, dim=16, vdim=24, diff=0.4, scale=0.3, coef=0.25, every=16):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale}
    if every:
        m["q_temp"] = {"coef": coef, "every": every}
    return m


def latent_mixer(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, window=20, scale=0.25, base=100.0):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if window:
        m["mask"] = {"size": window}
    return m


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def routed(experts=6, top=2, count=3, keep=2, ff=24, limit=1.25, scale=1.5):
    r = {"experts": experts, "top": top, "scale": scale}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}


def make_config(layers, width=48, vocab=97, eps=1e-5, loop=None, max_positions=2048):
    """layers: a list of (type, mixer, mlp or None)."""
    cfg = {"architecture": "Tukulorn", "width": width, "vocab": vocab, "norm": {"eps": eps},
           "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers], "max_positions": max_positions}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def tensor_shapes(cfg):
    """name -> (shape, kind); kind says how random_weights draws the tensor."""
    width = cfg["width"]
    out = {"embed": ((cfg["vocab"], width), "embed"), "final.norm": ((width,), "norm"), "head": ((cfg["vocab"], width), "mat")}
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        out[p + "norm1"] = ((width,), "norm")
        out[p + "ls1"] = ((width,), "ls")
        x = p + "mix."
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({x + "q": ((H * 2 * d, width), "mat"), x + "q.b": ((H * 2 * d,), "bias"), x + "k": ((G * 2 * d, width), "mat"),
                        x + "k.b": ((G * 2 * d,), "bias"), x + "v": ((G * dv, width), "mat"), x + "v.b": ((G * dv,), "bias"),
                        x + "lq1": ((d,), "lam"), x + "lk1": ((d,), "lam"), x + "lq2": ((d,), "lam"), x + "lk2": ((d,), "lam"),
                        x + "o": ((width, H * dv), "mat"), x + "o.b": ((width,), "bias")})
        else:
            H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({x + "q": ((H * (d + dr), width), "mat"), x + "dkv": ((rank + dr, width), "mat"), x + "dkv.norm": ((rank,), "plain_norm"),
                        x + "uk": ((H * d, rank), "mat"), x + "uv": ((H * dv, rank), "mat"), x + "g": ((H, width), "mat"),
                        x + "o": ((width, H * dv), "mat")})
        if L.get("mlp"):
            f = p + "mlp."
            out[p + "norm2"] = ((width,), "norm")
            out[p + "ls2"] = ((width,), "ls")
            if L["mlp"]["kind"] == "dense":
                ff = L["mlp"]["ff"]
                out.update({f + "gate": ((ff, width), "mat"), f + "up": ((ff, width), "mat"), f + "down": ((width, ff), "mat")})
            else:
                r, ff = L["mlp"]["router"], L["mlp"]["expert"]["ff"]
                out[f + "router"] = ((r["experts"], width), "router")
                for e in range(r["experts"]):
                    b = f + "e%d." % e
                    out.update({b + "gate": ((ff, width), "gate"), b + "up": ((ff, width), "gate"), b + "down": ((width, ff), "mat")})
    return out


def bf16_round(a):
    """float32 array rounded to the nearest bfloat16 value (ties to even), still float32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def random_weights(cfg, seed, gain=1.0):
    """Random weights, rounded to bfloat16 values.  Drawn so that faults show: router logits are spread (a wrong expert
    changes the row), the experts' gate and up maps are large enough to reach the limits, norm weights and layer scales
    are far from 0 and 1, the lambda vectors make the two exponentials differ."""
    rng, w = np.random.default_rng(seed), {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        n_in = shape[-1]
        if kind == "mat":
            a = rng.standard_normal(shape) * gain / math.sqrt(n_in)
        elif kind == "gate":
            a = rng.standard_normal(shape) * 1.5 * gain / math.sqrt(n_in)
        elif kind == "embed":
            a = rng.standard_normal(shape)
        elif kind == "norm":
            a = 0.3 * rng.standard_normal(shape)
        elif kind == "plain_norm":
            a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif kind == "ls":
            a = 0.6 + 0.3 * rng.standard_normal(shape)
        elif kind == "bias":
            a = 0.3 * rng.standard_normal(shape)
        elif kind == "lam":
            a = 0.3 * rng.standard_normal(shape)
        elif kind == "router":
            a = rng.standard_normal(shape) * 4.0 / math.sqrt(n_in)
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
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
