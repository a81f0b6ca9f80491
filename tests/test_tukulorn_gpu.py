"""The Tukulorn decoder in the engine against the plain implementation (tests/plain_tukulorn.py), GPU.

Every test makes its own small configuration and its own weights (numpy, rounded to bfloat16 so that the float32
mode, the bfloat16 mode and the plain implementation see the same numbers).  Weights are drawn so that faults show:
router logits are spread, the experts reach their limits, norm weights and layer scales are far from 0 and 1, and
where one key has to decide (a far key among hundreds, a window's edge) the weights are edited so that it does.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import plain_tukulorn as pt
from util import BF16_TOL, assert_close, rel_err

from inferllm_b200 import Engine, EngineOptions, Model, ModelConfig, StepItem

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
D, L = "attention", "latent_attention"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def f64(w):
    return {k: np.asarray(v, np.float64) for k, v in w.items()}


def write_model(folder, cfg, seed, edit=None, gain=0.5):
    w = pt.random_weights(cfg, seed, gain)
    if edit:
        edit(w)
        w = {k: pt.bf16_round(np.asarray(v, np.float32)) for k, v in w.items()}
    pt.write_model(folder, cfg, w)
    return f64(w)


def engine(folder, dtype, max_tokens=2048, page_size=64, max_seq_len=1024, poison=False, max_batch=None):
    return Engine.from_folder(folder, EngineOptions(dtype=dtype, max_tokens=max_tokens, page_size=page_size, max_seq_len=max_seq_len,
                                                    poison_freed_pages=poison, max_batch=max_batch))


def whole(eng, ids):
    s = eng.new_sequence()
    lg = eng.step([StepItem(s, list(ids), list(range(len(ids))))]).cpu().numpy()
    eng.end_sequence(s)
    return lg


def in_portions(eng, ids, sizes):
    """The sequence in steps of the given sizes (the last size repeats)."""
    s, at, out, k = eng.new_sequence(), 0, [], 0
    while at < len(ids):
        n = min(sizes[min(k, len(sizes) - 1)], len(ids) - at)
        out.append(eng.step([StepItem(s, list(ids[at:at + n]), list(range(n)))]).cpu().numpy())
        at += n
        k += 1
    eng.end_sequence(s)
    return np.concatenate(out)


def close(got, ref, dtype, what):
    """float32: every position within the bound.  bfloat16: a router whose choice hangs on two scores closer together
    than the rounding of its input may choose the other expert, which changes that token's row by more than rounding:
    at most one position in fifty (or one) may exceed the bound, none five times the bound."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    if dtype == "float32" or got.ndim < 2:
        return assert_close(got, ref, dtype, what)
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    err = np.abs(got - ref).max(-1) / max(np.abs(ref).max(), 1e-30)
    over = err > BF16_TOL
    assert over.sum() <= max(1, len(err) // 50), f"{what}: {int(over.sum())} of {len(err)} positions exceed {BF16_TOL:.1e} (worst {err.max():.3e})"
    assert err.max() <= 5 * BF16_TOL, f"{what}: a position is off by {err.max():.3e}"
    if (~over).any():
        assert_close(got[~over], ref[~over], dtype, what)


def same_or_close(a, b, dtype, what):
    """float32: every kernel fixes the order of its sums per row, so two ways of cutting the same tokens give the
    same bits; bfloat16: the library's products choose kernels by shape."""
    if dtype == "float32":
        assert np.array_equal(a, b), f"{what}: float32 logits differ between two cuttings (max {np.abs(a - b).max():.3e})"
    else:
        close(a, b, dtype, what)


def prompt(cfg, n, seed, w=None, dtype="float32"):
    """Random tokens.  With the weights given, tokens are drawn again until no router's choice hangs on two scores
    that rounding could swap (in bfloat16 with a wide margin where one expert is all a token gets; with several, `close`
    allows the rare swap)."""
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, cfg["vocab"], n).tolist()
    if w is None:
        return ids
    one_expert = any(layer.get("mlp") and layer["mlp"]["kind"] == "moe" and layer["mlp"]["router"]["top"] == 1 for layer in cfg["layers"])
    least = 1e-4 if dtype != "bfloat16" else 2e-2 if one_expert else 3e-3
    for _ in range(60):
        bad = pt.choice_margin(cfg, w, ids) < least
        if not bad.any():
            return ids
        for p in np.nonzero(bad)[0]:
            ids[p] = int(rng.integers(0, cfg["vocab"]))
    raise AssertionError("no well-conditioned prompt found")


CONFIGS = {
    # both mixers, a dense and routed feed-forwards, a loop over the middle layers, a window shorter than a page
    "mixed": pt.make_config([(D, pt.diff_mixer(), pt.dense()), (D, pt.diff_mixer(), pt.routed()), (L, pt.latent_mixer(), pt.routed()),
                             (L, pt.latent_mixer(), pt.dense())], loop=(1, 3, 2)),
    # no loop, no window, no temperature, no groups, a layer without a feed-forward, one key head per query head, one
    # expert per token, value heads as wide as the maps, odd sizes
    "other": pt.make_config([(L, pt.latent_mixer(heads=2, dim=12, rot_dim=4, vdim=12, kv_rank=20, window=0, scale=0.4, base=50.0), None),
                             (D, pt.diff_mixer(heads=3, kv_heads=3, dim=12, vdim=12, diff=0.7, scale=0.5, every=0), pt.routed(experts=3, top=1, count=0)),
                             (D, pt.diff_mixer(heads=2, kv_heads=1, dim=8, vdim=40, diff=0.2, every=1), pt.dense(24))], width=40, vocab=61, eps=1e-6),
    # a cache row of 128 channels (the tensor-core attention kernels), a window across pages, a loop of one layer three
    # times at the model's end, every expert chosen
    "wide": pt.make_config([(D, pt.diff_mixer(heads=4, kv_heads=1, dim=32, vdim=64, scale=0.18, every=50), pt.routed(experts=2, top=2, count=2, keep=2)),
                            (L, pt.latent_mixer(heads=4, dim=32, rot_dim=32, vdim=32, kv_rank=96, window=70, scale=0.15),
                             pt.routed(experts=8, top=3, count=4, keep=2, ff=32))], width=64, vocab=128, loop=(1, 2, 3)),
    # an odd width and an odd vocabulary, a cache row that is no multiple of 8, a loop that starts at the first layer
    "odd": pt.make_config([(L, pt.latent_mixer(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=27, window=11, scale=0.3), pt.routed(experts=4, top=4, count=2, keep=2, ff=10)),
                           (D, pt.diff_mixer(heads=3, kv_heads=1, dim=6, vdim=10, every=7), None)], width=45, vocab=71, loop=(0, 2, 2)),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("tk_" + name))
        out[name] = (d, cfg, write_model(d, cfg, 7 + i))
    return out


# ------------------------------------------------------------------ each mechanism alone

ALONE = {
    "diff": pt.make_config([(D, pt.diff_mixer(), None)]),
    "diff_one_kv_head": pt.make_config([(D, pt.diff_mixer(heads=6, kv_heads=1, dim=10, vdim=16), None)]),
    "diff_head_per_kv_head_no_temperature": pt.make_config([(D, pt.diff_mixer(heads=2, kv_heads=2, dim=24, vdim=8, diff=0.8, every=0), None)]),
    "diff_one_head_temperature_every_token": pt.make_config([(D, pt.diff_mixer(heads=1, kv_heads=1, dim=16, vdim=16, coef=0.6, every=1), None)]),
    "diff_wide_values": pt.make_config([(D, pt.diff_mixer(heads=2, kv_heads=1, dim=64, vdim=128, scale=0.12, every=9), None)], width=64),
    "latent": pt.make_config([(L, pt.latent_mixer(), None)]),
    "latent_no_window": pt.make_config([(L, pt.latent_mixer(window=0), None)]),
    "latent_window_of_one": pt.make_config([(L, pt.latent_mixer(window=1), None)]),
    "latent_one_head": pt.make_config([(L, pt.latent_mixer(heads=1, dim=24, rot_dim=2, vdim=8, kv_rank=30, window=9), None)]),
    "latent_row_of_128": pt.make_config([(L, pt.latent_mixer(heads=5, dim=16, rot_dim=32, vdim=16, kv_rank=96, window=33, scale=0.2), None)]),
    "latent_row_of_64_many_heads": pt.make_config([(L, pt.latent_mixer(heads=18, dim=8, rot_dim=16, vdim=8, kv_rank=48, window=0, scale=0.3), None)]),
    "latent_row_of_128_window_of_one": pt.make_config([(L, pt.latent_mixer(heads=2, dim=16, rot_dim=32, vdim=16, kv_rank=96, window=1, scale=0.2), None)]),
    "latent_row_of_64_window_of_two": pt.make_config([(L, pt.latent_mixer(heads=3, dim=16, rot_dim=16, vdim=16, kv_rank=48, window=2, scale=0.2), None)]),
    "latent_row_of_128_window_of_a_page": pt.make_config([(L, pt.latent_mixer(heads=2, dim=16, rot_dim=64, vdim=16, kv_rank=64, window=64, scale=0.2), None)]),
    "latent_odd_row": pt.make_config([(L, pt.latent_mixer(heads=2, dim=12, rot_dim=6, vdim=10, kv_rank=21, window=13), None)]),
    "dense": pt.make_config([(D, pt.diff_mixer(), pt.dense())]),
    "moe_groups": pt.make_config([(D, pt.diff_mixer(), pt.routed(experts=8, top=3, count=4, keep=2))]),
    "moe_one_group_kept": pt.make_config([(L, pt.latent_mixer(), pt.routed(experts=6, top=3, count=2, keep=1))]),
    "moe_no_groups_one_expert": pt.make_config([(D, pt.diff_mixer(), pt.routed(experts=5, top=1, count=0, scale=1.0))]),
    "moe_groups_of_one": pt.make_config([(L, pt.latent_mixer(), pt.routed(experts=4, top=2, count=4, keep=3, limit=0.5, scale=3.0))]),
    "moe_all_chosen": pt.make_config([(D, pt.diff_mixer(), pt.routed(experts=4, top=4, count=1, keep=1))]),
    "loop_of_everything": pt.make_config([(D, pt.diff_mixer(), pt.dense()), (L, pt.latent_mixer(), None)], loop=(0, 2, 3)),
    "loop_once": pt.make_config([(D, pt.diff_mixer(), pt.dense()), (L, pt.latent_mixer(), None)], loop=(1, 2, 1)),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALONE))
def test_mechanism_alone(tmp_path, name, dtype):
    cfg = ALONE[name]
    w = write_model(str(tmp_path), cfg, 3)
    ids = prompt(cfg, 141 if "window_of" in name else 41, 5, w, dtype)
    layers = []
    ref = pt.forward(cfg, w, ids, layers)
    eng = engine(str(tmp_path), dtype)
    close(whole(eng, ids), ref, dtype, name)
    # and token by token through the cache
    close(in_portions(eng, ids, [1]), ref, dtype, name + " token by token")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompt_through_the_tile_kernels(tmp_path, dtype):
    """A prompt long enough for the experts' products on row tiles of 128, for the prompt attention kernels' tiles of
    queries and keys, and for several steps of the query temperature."""
    cfg = pt.make_config([(D, pt.diff_mixer(heads=4, kv_heads=2, dim=32, vdim=64, scale=0.2, every=128), pt.routed(experts=4, top=2, count=2, keep=2, ff=64)),
                          (L, pt.latent_mixer(heads=4, dim=32, rot_dim=32, vdim=32, kv_rank=96, window=150, scale=0.15), pt.dense(128))], width=64)
    w = write_model(str(tmp_path), cfg, 21)
    ids = prompt(cfg, 600, 8, w, dtype)
    ref = pt.forward(cfg, w, ids)
    eng = engine(str(tmp_path), dtype, max_tokens=2048)
    got = whole(eng, ids)
    close(got, ref, dtype, "600 tokens in one step")
    same_or_close(in_portions(eng, ids, [520, 1]), got, dtype, "the same, its last tokens one by one")
    close(in_portions(eng, ids, [250, 200, 150]), ref, dtype, "three long portions")


OTHER_SIZES = {
    # query heads per key/value head that fill the single-token kernel's groups of heads exactly, partly and twice over
    "diff_group_of_8": pt.make_config([(D, pt.diff_mixer(heads=8, kv_heads=1, dim=16, vdim=32, scale=0.3, every=20), None)], width=64),
    "diff_group_of_3": pt.make_config([(D, pt.diff_mixer(heads=6, kv_heads=2, dim=8, vdim=16, scale=0.4, every=11), None)]),
    "diff_group_of_7": pt.make_config([(D, pt.diff_mixer(heads=7, kv_heads=1, dim=24, vdim=8, scale=0.3, every=0), None)], width=56),
    "diff_group_of_16": pt.make_config([(D, pt.diff_mixer(heads=16, kv_heads=1, dim=8, vdim=24, scale=0.5), None)], width=64),
    "diff_group_of_5_many_kv_heads": pt.make_config([(D, pt.diff_mixer(heads=20, kv_heads=4, dim=16, vdim=16, scale=0.3), None)], width=80),
    # maps and values wider than the tensor-core kernel takes, and values that are no multiple of 16
    "diff_maps_of_208": pt.make_config([(D, pt.diff_mixer(heads=2, kv_heads=1, dim=208, vdim=32, scale=0.07), None)], width=64),
    "diff_values_of_256": pt.make_config([(D, pt.diff_mixer(heads=2, kv_heads=2, dim=32, vdim=256, scale=0.2), None)], width=64),
    "diff_values_of_72": pt.make_config([(D, pt.diff_mixer(heads=4, kv_heads=2, dim=48, vdim=72, scale=0.15), None)], width=64),
    # a latent far wider than a head, cache rows of 192, 264 and 576 channels, more heads than one block of the ring kernel holds
    "latent_row_of_192": pt.make_config([(L, pt.latent_mixer(heads=4, dim=24, rot_dim=64, vdim=40, kv_rank=128, window=50, scale=0.1), None)], width=64),
    "latent_row_of_264": pt.make_config([(L, pt.latent_mixer(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=256, window=0, scale=0.1), None)], width=64),
    "latent_row_of_576": pt.make_config([(L, pt.latent_mixer(heads=3, dim=32, rot_dim=64, vdim=32, kv_rank=512, window=45, scale=0.06), None)], width=64),
    "latent_40_heads_row_of_128": pt.make_config([(L, pt.latent_mixer(heads=40, dim=8, rot_dim=16, vdim=8, kv_rank=112, window=37, scale=0.2), None)], width=64),
    # many experts in many groups, and more experts per token than a group holds
    "moe_64_experts": pt.make_config([(D, pt.diff_mixer(), pt.routed(experts=64, top=6, count=16, keep=5, ff=8, limit=2.0, scale=0.5))]),
    "moe_32_groups": pt.make_config([(L, pt.latent_mixer(), pt.routed(experts=32, top=4, count=32, keep=7, ff=8))]),
    # a wider model, a long loop
    "wider": pt.make_config([(D, pt.diff_mixer(heads=8, kv_heads=4, dim=32, vdim=32, scale=0.2), pt.dense(300)),
                             (L, pt.latent_mixer(heads=8, dim=24, rot_dim=16, vdim=24, kv_rank=48, window=30, scale=0.2), pt.routed(ff=40))],
                            width=192, vocab=301, loop=(0, 2, 4)),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(OTHER_SIZES))
def test_other_sizes(tmp_path, name, dtype):
    cfg = OTHER_SIZES[name]

    def edit(w):       # with dozens of experts the best scores crowd at 1 unless the router's logits are small
        for k in w:
            if k.endswith("mlp.router") and w[k].shape[0] >= 32:
                w[k] = 0.25 * np.asarray(w[k])

    w = write_model(str(tmp_path), cfg, 13, edit)
    ids = prompt(cfg, 90, 7, w, dtype)
    ref = pt.forward(cfg, w, ids)
    eng = engine(str(tmp_path), dtype)
    close(whole(eng, ids), ref, dtype, name)
    close(in_portions(eng, ids, [70, 1]), ref, dtype, name + ", its last tokens one by one")
    a, b = ids[:55], ids[20:90]
    sa, sb = eng.new_sequence(), eng.new_sequence()
    eng.step([StepItem(sa, a[:40], []), StepItem(sb, b[:66], [])])
    got = [eng.step([StepItem(sa, [a[40 + i]], [0]), StepItem(sb, [b[66 + i]], [0])]).cpu().numpy() for i in range(4)]
    eng.end_sequence(sa)
    eng.end_sequence(sb)
    ra, rb = pt.forward(cfg, w, a), pt.forward(cfg, w, b)
    close(np.stack([g[0] for g in got]), ra[40:44], dtype, name + ", two sequences decoded together, the first")
    close(np.stack([g[1] for g in got]), rb[66:70], dtype, name + ", two sequences decoded together, the second")


# ------------------------------------------------------------------ whole models


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt(models, name, dtype):
    d, cfg, w = models[name]
    ids = prompt(cfg, 150, 11, w, dtype)
    layers = []
    ref = pt.forward(cfg, w, ids, layers)
    assert len(layers) == len(pt.layer_order(cfg))
    close(whole(engine(d, dtype), ids), ref, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_first_tokens_and_one_token(models, name, dtype):
    d, cfg, w = models[name]
    eng = engine(d, dtype)
    for n in (1, 2, 3):
        ids = prompt(cfg, n, 20 + n, w, dtype)
        close(whole(eng, ids), pt.forward(cfg, w, ids), dtype, f"{name} {n} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_and_decoding(models, name, dtype):
    """Prefill against token-by-token decoding and portions of several sizes, down to two tokens, across page borders
    and window edges."""
    d, cfg, w = models[name]
    ids = prompt(cfg, 200, 13, w, dtype)
    ref = pt.forward(cfg, w, ids)
    eng = engine(d, dtype)
    base = whole(eng, ids)
    close(base, ref, dtype, name)
    for sizes in ([1], [2], [63, 2, 64, 7], [128, 1], [5, 64, 3], [1, 1, 2, 3, 50]):
        got = in_portions(eng, ids, sizes)
        close(got, ref, dtype, f"{name} portions {sizes}")
        same_or_close(got, base, dtype, f"{name} portions {sizes}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_unequal_batches(models, name, dtype):
    """Requests of different lengths in one batch, then decoded together while the shorter ones end, against each alone."""
    d, cfg, w = models[name]
    eng = engine(d, dtype, max_tokens=4096)
    lens, extra = [1, 37, 150, 66], [9, 30, 12, 5]
    seqs = [prompt(cfg, n + e, 40 + i, w, dtype) for i, (n, e) in enumerate(zip(lens, extra))]
    refs = [pt.forward(cfg, w, s) for s in seqs]
    alone = [whole(eng, s) for s in seqs]
    slots = [eng.new_sequence() for _ in seqs]
    lg = eng.step([StepItem(slots[i], seqs[i][:lens[i]], list(range(lens[i]))) for i in range(len(seqs))]).cpu().numpy()
    at, got = 0, []
    for i, n in enumerate(lens):
        got.append([lg[at:at + n]])
        at += n
    pos = list(lens)
    live = list(range(len(seqs)))
    while live:
        lg = eng.step([StepItem(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            got[i].append(lg[r:r + 1])
            pos[i] += 1
        for i in list(live):
            if pos[i] == len(seqs[i]):
                eng.end_sequence(slots[i])
                live.remove(i)
    for i in range(len(seqs)):
        g = np.concatenate(got[i])
        close(g, refs[i], dtype, f"{name} batch, sequence {i}")
        same_or_close(g, alone[i], dtype, f"{name} batch, sequence {i} against itself alone")


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(models, dtype):
    """A small cache whose slots and pages go round several times, freed pages poisoned with NaN: a sequence must never
    read a page that it does not hold, and pages that left a window are given back while their sequence goes on."""
    d, cfg, w = models["mixed"]
    eng = engine(d, dtype, max_tokens=320, max_batch=3, max_seq_len=256, poison=True)
    for rnd in range(4):
        seqs = [prompt(cfg, n, 70 + 10 * rnd + i, w, dtype) for i, n in enumerate((90 + rnd, 33, 70))]
        slots = [eng.new_sequence() for _ in seqs]
        cut = [len(s) // 2 + rnd for s in seqs]
        eng.step([StepItem(slots[i], seqs[i][:cut[i]], []) for i in range(3)])
        eng.end_sequence(slots[1])                        # its slot and pages go to the next sequence at once
        late = prompt(cfg, 40, 90 + rnd, w, dtype)
        s_late = eng.new_sequence()
        got_late = eng.step([StepItem(s_late, late, list(range(40)))]).cpu().numpy()
        close(got_late, pt.forward(cfg, w, late), dtype, f"round {rnd}: a sequence in a slot used before")
        for i in (0, 2):
            rest = seqs[i][cut[i]:]
            got = eng.step([StepItem(slots[i], rest, list(range(len(rest))))]).cpu().numpy()
            close(got, pt.forward(cfg, w, seqs[i])[cut[i]:], dtype, f"round {rnd}: sequence {i} continued")
            eng.end_sequence(slots[i])
        eng.end_sequence(s_late)


# ------------------------------------------------------------------ crafted cases

FAR = 63            # the last row of the first page of 64


def crafted_ids(cfg, n, seed):
    """Random tokens in which token 7 stands at position FAR and nowhere else."""
    ids = [t if t != 7 else 8 for t in prompt(cfg, n, seed)]
    ids[FAR] = 7
    return ids


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page", [64, 16])
def test_one_far_key_decides_a_differential_head(tmp_path, page, dtype):
    """The key of one position is made to stand out in the FIRST score map of every later query: its token appears
    once, its embedding is a spike in one channel, the first map's keys read that channel and the first map's queries
    carry a constant through their bias.  The second map does not see it, so the difference of the maps hangs on that
    one key, hundreds of positions back, at a page border, in a prompt and in decoding."""
    m = pt.diff_mixer(heads=2, kv_heads=1, dim=8, vdim=12, diff=0.3, scale=1.0, coef=0.2, every=100)
    cfg = pt.make_config([(D, m, None)], vocab=50)
    ids = crafted_ids(cfg, 300, 3)

    def edit(w):
        w["embed"][7] = 0.0
        w["embed"][7, 5] = 6.0
        for head in range(2):                             # channel 0 of map 1 of both query heads: a constant
            w["l0.mix.q"][head * 16] = 0.0
            w["l0.mix.q.b"][head * 16] = 3.0
        w["l0.mix.k"][0] = 0.0                            # channel 0 of map 1 of the key head reads the spike
        w["l0.mix.k"][0, 5] = 1.0
        w["l0.mix.k.b"][0] = 0.0
        w["l0.norm1"][5] = 0.0
        w["l0.mix.o"] = 4.0 * np.asarray(w["l0.mix.o"])          # the mixer's share of the logits

    w = write_model(str(tmp_path), cfg, 9, edit)
    ref = pt.forward(cfg, w, ids)
    alt = pt.forward(cfg, w, ids[:FAR] + [8] + ids[FAR + 1:])
    assert rel_err(alt[200:], ref[200:]) > 0.05, "the crafted key does not decide"
    eng = engine(str(tmp_path), dtype, page_size=page)
    assert_close(whole(eng, ids), ref, dtype, "prompt")
    assert_close(in_portions(eng, ids, [60, 1]), ref, dtype, "decoding past the key")
    assert_close(in_portions(eng, ids, [FAR + 1, 2]), ref, dtype, "portions from the key on")
    assert_close(in_portions(eng, ids, [FAR, 1, 130, 7]), ref, dtype, "the key alone in a step")


def with_window(cfg, size):
    c = json.loads(json.dumps(cfg))
    for layer in c["layers"]:
        if layer["type"] == L:
            layer["mixer"]["mask"] = {"size": size}
    return c


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,page,rank", [(0, 64, 24), (64, 64, 24), (65, 64, 24), (63, 64, 24), (7, 16, 24), (33, 16, 21), (2, 64, 24),
                                              (64, 64, 120), (65, 64, 120), (130, 64, 120)])
def test_one_key_decides_at_the_windows_edge(tmp_path, window, page, rank, dtype):
    """The same through the rotated key part that all heads of a latent-attention layer share: with a huge base all
    pairs but the first hardly turn, so a spike in the second pair of one position's key part, against queries that
    carry a constant there, stands out whatever the distance.  Whether exactly that key is seen decides the output:
    just inside and just outside the window, at a page border, among hundreds of keys, in a prompt and in decoding.
    The plain implementation with a window one longer or shorter must disagree, or the test would show nothing.
    (rank 120 makes cache rows of 128 channels: the tensor-core kernels in bfloat16; 21 a row that is no multiple of 8.)"""
    m = pt.latent_mixer(heads=2, dim=8, rot_dim=8, vdim=12, kv_rank=rank, window=window, scale=1.0, base=1e30)
    cfg = pt.make_config([(L, m, None)], vocab=50)
    ids = crafted_ids(cfg, 300 if window == 0 else 64 + window + 60, 3)

    def edit(w):
        w["embed"][:, 6] = 2.0                            # a constant channel, read by the queries
        w["embed"][7] = 0.0
        w["embed"][7, 5] = 6.0
        w["embed"][7, 6] = 2.0
        w["l0.norm1"][5] = w["l0.norm1"][6] = 0.0
        for head in range(2):                             # channel 2 of the rotated part of both heads
            w["l0.mix.q"][head * 16 + 8 + 2] = 0.0
            w["l0.mix.q"][head * 16 + 8 + 2, 6] = 2.0
        w["l0.mix.dkv"][rank + 2] = 0.0                   # channel 2 of the shared key part reads the spike
        w["l0.mix.dkv"][rank + 2, 5] = 1.0
        w["l0.mix.g"][:] = 0.3 * np.asarray(w["l0.mix.g"])
        w["l0.mix.o"] = 4.0 * np.asarray(w["l0.mix.o"])          # the mixer's share of the logits

    w = write_model(str(tmp_path), cfg, 9, edit)
    ref = pt.forward(cfg, w, ids)
    if window:
        edge = FAR + window                               # the first query that no longer sees the key
        for other in (window - 1, window + 1):
            alt = pt.forward(with_window(cfg, other), w, ids)
            assert rel_err(alt[edge - 1:edge + 1], ref[edge - 1:edge + 1]) > 0.05, "the crafted key does not decide"
    else:
        alt = pt.forward(cfg, w, ids[:FAR] + [8] + ids[FAR + 1:])
        assert rel_err(alt[200:], ref[200:]) > 0.05, "the crafted key does not decide"
    eng = engine(str(tmp_path), dtype, page_size=page)
    assert_close(whole(eng, ids), ref, dtype, f"window {window}, prompt")
    assert_close(in_portions(eng, ids, [60, 1]), ref, dtype, f"window {window}, decoding past the key")
    assert_close(in_portions(eng, ids, [FAR + 1, 2]), ref, dtype, f"window {window}, portions from the key on")
    if window:
        assert_close(in_portions(eng, ids, [FAR + window - 1, 1, 1, 1, 40]), ref, dtype, f"window {window}, steps at the edge")


@pytest.mark.parametrize("dtype", DTYPES)
def test_rotation_sees_the_distance_only(tmp_path, dtype):
    """Sharp attention through the rotated parts alone: the latent's keys are switched off, so a score depends on the
    rotated pairs, whose product is a function of the distance.  The same tokens must give the same rows wherever a
    step cuts them, far from position 0, and the plain implementation rotated in the other direction must disagree."""
    m = pt.latent_mixer(heads=2, dim=8, rot_dim=16, vdim=12, kv_rank=24, window=40, scale=2.0, base=30.0)
    cfg = pt.make_config([(L, m, None)])

    def edit(w):
        w["l0.mix.uk"][:] = 0.0

    w = write_model(str(tmp_path), cfg, 12, edit, gain=1.0)
    ids = prompt(cfg, 230, 4)
    ref = pt.forward(cfg, w, ids)
    back = json.loads(json.dumps(cfg))
    back["layers"][0]["mixer"]["rot"]["base"] = 31.0
    assert rel_err(pt.forward(back, w, ids)[50:], ref[50:]) > 0.01
    eng = engine(str(tmp_path), dtype)
    assert_close(whole(eng, ids), ref, dtype, "prompt")
    assert_close(in_portions(eng, ids, [190, 1]), ref, dtype, "decoding")
    assert_close(in_portions(eng, ids, [39, 2, 41, 64, 3]), ref, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_experts_at_their_limits_and_groups_that_exclude(tmp_path, dtype):
    """Gate and up projections far beyond the limit on both sides (the gate is cut from above only, the up projection on
    both sides), and a router whose best expert lies in a group that loses: the group's score is the sum of its two
    largest, so one expert far ahead does not save a group whose others are far behind."""
    mlp = pt.routed(experts=6, top=2, count=3, keep=1, ff=16, limit=0.75, scale=2.5)
    cfg = pt.make_config([(D, pt.diff_mixer(), mlp)])

    def edit(w):
        for e in range(6):
            w["l0.mlp.e%d.gate" % e] = 6.0 * np.asarray(w["l0.mlp.e%d.gate" % e])
            w["l0.mlp.e%d.up" % e] = 6.0 * np.asarray(w["l0.mlp.e%d.up" % e])
        r = np.asarray(w["l0.mlp.router"]).copy()
        r[0] = 4.0 * r[0]                  # expert 0 is often the best of all, its neighbour 1 is pushed down
        r[1] = -np.abs(r[1])
        w["l0.mlp.router"] = r

    w = write_model(str(tmp_path), cfg, 31, edit)
    ids = prompt(cfg, 120, 6, w, dtype)
    ref = pt.forward(cfg, w, ids)
    # the plain implementation itself depends on the group rule and on the limit
    one = json.loads(json.dumps(cfg))
    one["layers"][0]["mlp"]["router"]["groups"] = {"count": 1, "keep": 1}
    assert rel_err(pt.forward(one, w, ids), ref) > 0.02
    wide = json.loads(json.dumps(cfg))
    wide["layers"][0]["mlp"]["expert"]["limit"] = 50.0
    assert rel_err(pt.forward(wide, w, ids), ref) > 0.02
    eng = engine(str(tmp_path), dtype)
    close(whole(eng, ids), ref, dtype, "prompt")
    close(in_portions(eng, ids, [100, 1]), ref, dtype, "decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(models, dtype):
    """Three hundred tokens one by one behind a short prompt: past several pages, windows, steps of the temperature."""
    d, cfg, w = models["mixed"]
    ids = prompt(cfg, 330, 17, w, dtype)
    close(in_portions(engine(d, dtype), ids, [30, 1]), pt.forward(cfg, w, ids), dtype, "long decoding")


# ------------------------------------------------------------------ the library's own entry points


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_model_api(models, dtype):
    """Model.generate: the scheduler batches the requests, decodes them together and ends each by itself."""
    d, cfg, w = models["mixed"]
    prompts = [prompt(cfg, n, 50 + n, w, dtype) for n in (3, 17, 70, 1)]
    m = Model(ModelConfig(compt_type=dtype, nr_ctx=256, max_tokens=1024))
    m.load(d)
    m.init(top_k=0, top_p=1.0, temp=0.0, repeat_penalty=1.0, repeat_last_n=0, seed=0, end_token=-1)
    got = m.generate(prompts, max_new_tokens=12, stop_ids=[]).tokens
    want = [pt.greedy_generate(cfg, w, p, 12) for p in prompts]
    if dtype == "float32":
        assert got == want
        return
    # bfloat16 may turn a near-tie: every token the engine chose must be (within rounding) the best continuation of what
    # it had generated so far, by the plain implementation's logits for that very sequence
    for p, g in zip(prompts, got):
        assert len(g) == 12
        lg = pt.forward(cfg, w, p + g)[len(p) - 1:-1]
        gap = lg.max(-1) - lg[np.arange(12), g]
        assert (gap <= BF16_TOL * np.abs(lg).max()).all(), (g, gap)


def test_command_line(models):
    """bin/llama on a Tukulorn folder: greedy tokens of two requests, float32."""
    d, cfg, w = models["mixed"]
    prompts = [prompt(cfg, n, 90 + n, w) for n in (7, 12)]
    want = [pt.greedy_generate(cfg, w, p, 6) for p in prompts]
    args = [os.path.join(ROOT, "bin", "llama"), "-m", d, "-d", "float32", "-c", "128", "-n", "6", "--temp", "0", "--top_k", "0",
            "--top_p", "1", "--repeat_penalty", "1", "-s", "1"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    r = subprocess.run(args, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = [[int(t) for t in ln.split(": ")[1].split(",")] for ln in r.stdout.splitlines() if ln.startswith("[")]
    assert got == want


def test_trace_replay_program(models, tmp_path):
    d, cfg, w = models["other"]
    a, b = prompt(cfg, 40, 1, w), prompt(cfg, 9, 2, w)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[33:34], "want": [0]}, {"id": "b", "tokens": b[8:], "want": []}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[34:35], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[35:], "want": [4]}], "end": ["a"]}]
    out = str(tmp_path / "out")
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out, "--max-tokens", "128"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done %d" % i for i in range(4)]
    ra, rb = pt.forward(cfg, w, a), pt.forward(cfg, w, b)
    V = cfg["vocab"]
    got0 = np.fromfile(os.path.join(out, "0.f32"), "<f4").reshape(-1, V)
    assert_close(got0, np.stack([ra[0], ra[32], rb[7]]), "float32", "step 0")
    assert_close(np.fromfile(os.path.join(out, "1.f32"), "<f4").reshape(-1, V), ra[33:34], "float32", "step 1")
    assert_close(np.fromfile(os.path.join(out, "2.f32"), "<f4").reshape(-1, V), ra[34:35], "float32", "step 2")
    assert_close(np.fromfile(os.path.join(out, "3.f32"), "<f4").reshape(-1, V), ra[39:40], "float32", "step 3")
