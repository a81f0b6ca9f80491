"""The Kudonex decoder in the engine against the plain implementation (tests/plain_kudonex.py), GPU.

Every test makes its own small configuration and its own weights (numpy, rounded to bfloat16 so that the float32
mode, the bfloat16 mode and the plain implementation see the same numbers).  Weights are drawn so that faults show:
router logits are spread and the corrections change the choice, decay rates run from slow to fast, the distance
factors and the matrix that mixes the heads' scores are far from 0 and from the identity.
"""
import json
import os

import numpy as np
import pytest
import plain_kudonex as pk
from util import BF16_TOL, assert_close, rel_err

from inferllm_b200 import Engine, EngineOptions, Model, ModelConfig, StepItem

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
M, S, A = "mlstm", "mamba2", "attention"


def f64(w):
    return {k: np.asarray(v, np.float64) for k, v in w.items()}


def write_model(folder, cfg, seed, edit=None, gain=0.5):
    """config.json + model.safetensors (bfloat16) with random weights; returns them as float64.  `gain` scales the
    matrices: with larger ones a stack of layers amplifies rounding until bfloat16 decides the result."""
    w = pk.random_weights(cfg, seed, gain)
    if edit:
        edit(w)
        w = {k: pk.bf16_round(np.asarray(v, np.float32)) for k, v in w.items()}
    pk.write_model(folder, cfg, w)
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
    than the rounding of its input may choose the other expert, which changes that token's row (and, less, the rows
    after it) by more than rounding: at most one position in fifty (or one) may exceed the bound, none five times the
    bound, and the others are held to it."""
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


CONFIGS = {
    # all three mixers, groups of experts with two kept, a window shorter than a page
    "mixed": pk.random_config((M, S, A, M)),
    # no input convolution, no window, one key head per query head, one state-space group, one tap, one expert per
    # token, a feed-forward without groups and without a shared expert, a layer without a feed-forward, odd sizes
    "other": pk.random_config((A, S, M), width=40, vocab=61, taps=0, heads=3, dim=24, vdim=10, ssm_heads=6, ssm_vdim=8, state=20, groups=1,
                              norm_groups=3, conv=1, att_heads=5, kv_heads=5, att_dim=8, window=0, scale=0.6, experts=3, top=1, group_count=1,
                              group_keep=1, expert_ff=20, shared_ff=12, mlps=["bare", None, True], eps=1e-6, emb_scale=1.0, gate_cap=4.0),
    # heads of 64 channels, one matrix-memory head, a window across pages, three query heads per key head, four taps in
    # the state space and two in the input convolution, the norm over the whole row
    "wide": pk.random_config((S, A, M), width=64, vocab=128, taps=2, heads=1, dim=64, vdim=40, ssm_heads=2, ssm_vdim=64, state=64, groups=2,
                             norm_groups=1, conv=4, att_heads=6, kv_heads=2, att_dim=32, window=70, scale=0.3, experts=8, top=3, group_count=4,
                             group_keep=2, expert_ff=32, shared_ff=96),
    # heads of 128 channels, one key head for eight query heads, a window across three pages, every expert chosen
    "wide128": pk.random_config((M, A, S), width=96, vocab=150, taps=5, heads=2, dim=128, vdim=16, ssm_heads=4, ssm_vdim=16, state=128, groups=1,
                                norm_groups=4, conv=2, att_heads=8, kv_heads=1, att_dim=128, window=130, scale=0.1, experts=2, top=2,
                                group_count=2, group_keep=2, expert_ff=48, shared_ff=16),
    # an odd width and an odd vocabulary, head sizes that are multiples of nothing much, a group per state-space head
    "odd_width": pk.random_config((A, M, S, A), width=45, vocab=71, taps=3, heads=3, dim=10, vdim=6, ssm_heads=3, ssm_vdim=5, state=7, groups=3,
                                  norm_groups=5, conv=3, att_heads=3, kv_heads=1, att_dim=6, window=11, scale=0.9, experts=4, top=4,
                                  group_count=2, group_keep=2, expert_ff=10, shared_ff=30, mlps=[True, "bare", None, True]),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("kx_" + name))
        out[name] = (d, cfg, write_model(d, cfg, 7 + i))
    return out


def prompt(cfg, n, seed, w=None, dtype="float32"):
    """Random tokens.  With the weights given, tokens are drawn again until the prompt is a fair test of arithmetic:
    no router's choice hangs on two scores that rounding could swap (in bfloat16 only where one expert is all a token
    gets: with several, `close` allows the rare swap), and no position enlarges rounding more than tenfold (a unit norm
    over a read-out that happens to be tiny would)."""
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, cfg["vocab"], n).tolist()
    if w is None:
        return ids
    one_expert = any(L.get("mlp") and L["mlp"]["router"]["top"] == 1 for L in cfg["layers"])
    least = 2e-2 if dtype == "bfloat16" and one_expert else 1e-4
    for _ in range(60):
        bad = (pk.choice_margin(cfg, w, ids) < least) | (pk.amplification(cfg, w, ids) > 10.0)
        if not bad.any():
            return ids
        for p in np.nonzero(bad)[0]:
            ids[p] = int(rng.integers(0, cfg["vocab"]))
    raise AssertionError("no well-conditioned prompt found")


# ------------------------------------------------------------------ each mechanism alone

ALONE = {
    "mlstm": pk.random_config((M,), mlps=[None], taps=0),
    "mlstm_one_head_small_cap": pk.random_config((M,), mlps=[None], taps=0, heads=1, dim=12, vdim=12, gate_cap=1.5),
    "mlstm_many_heads": pk.random_config((M,), mlps=[None], taps=0, heads=5, dim=8, vdim=20, gate_cap=30.0),
    "mamba2": pk.random_config((S,), mlps=[None], taps=0),
    "mamba2_one_group_one_tap": pk.random_config((S,), mlps=[None], taps=0, groups=1, norm_groups=1, conv=1),
    "mamba2_group_per_head": pk.random_config((S,), mlps=[None], taps=0, ssm_heads=3, ssm_vdim=10, state=9, groups=3, norm_groups=6, conv=5),
    "attention": pk.random_config((A,), mlps=[None], taps=0, window=0, scale=1.5),
    "attention_window": pk.random_config((A,), mlps=[None], taps=0, window=5, scale=1.5),
    "attention_window_of_one": pk.random_config((A,), mlps=[None], taps=0, window=1, scale=1.5),
    "attention_one_kv_head": pk.random_config((A,), mlps=[None], taps=0, window=9, att_heads=6, kv_heads=1, att_dim=10, scale=0.8),
    "attention_one_head": pk.random_config((A,), mlps=[None], taps=0, window=0, att_heads=1, kv_heads=1, att_dim=24, scale=0.4),
    "input_conv": pk.random_config((A,), mlps=[None], taps=4, window=0),
    "input_conv_one_tap": pk.random_config((M,), mlps=[None], taps=1),
    "moe_groups": pk.random_config((A,), taps=0, experts=8, top=3, group_count=4, group_keep=2),
    "moe_one_group_kept": pk.random_config((A,), taps=0, experts=6, top=3, group_count=2, group_keep=1),
    "moe_bare": pk.random_config((A,), taps=0, mlps=["bare"], experts=5, top=2),
    "moe_all_chosen": pk.random_config((A,), taps=0, experts=4, top=4, group_count=1, group_keep=1),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALONE))
def test_mechanism_alone(tmp_path, name, dtype):
    cfg = ALONE[name]
    w = write_model(str(tmp_path), cfg, 3)
    ids = prompt(cfg, 41, 5)
    layers = []
    ref = pk.forward(cfg, w, ids, layers)
    eng = engine(str(tmp_path), dtype)
    close(whole(eng, ids), ref, dtype, name)
    # and token by token through the cache and the state
    close(in_portions(eng, ids, [1]), ref, dtype, name + " token by token")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompt_through_the_fused_products(tmp_path, dtype):
    """A prompt long enough for the experts' products on row tiles of 128 and for the scan over many blocks of tokens."""
    cfg = pk.random_config((M, A, S), width=64, expert_ff=64, shared_ff=128, experts=4, top=2, group_count=2, group_keep=2, window=50,
                           att_heads=2, kv_heads=1, att_dim=16)
    w = write_model(str(tmp_path), cfg, 21)
    ids = prompt(cfg, 600, 8)
    ref = pk.forward(cfg, w, ids)
    eng = engine(str(tmp_path), dtype, max_tokens=2048)
    got = whole(eng, ids)
    close(got, ref, dtype, "600 tokens in one step")
    same_or_close(in_portions(eng, ids, [520, 1]), got, dtype, "the same, its last tokens one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv,dim,window", [(12, 4, 128, 37), (4, 4, 64, 0), (3, 1, 32, 16), (20, 2, 16, 17), (2, 1, 48, 90)])
def test_prompt_attention_in_token_tiles(tmp_path, heads, kv, dim, window, dtype):
    """Prompts and portions long enough for the kernel that takes 16 tokens of a sequence per block (bfloat16): head
    counts that one block holds and that take several, windows that end inside a tile of tokens and of keys, tiles
    that two sequences of a batch share a step with, a last tile of one token, and each alone for comparison."""
    cfg = pk.random_config((A,), mlps=[None], taps=0, att_heads=heads, kv_heads=kv, att_dim=dim, window=window, scale=dim ** -0.5 * 2, width=64)
    w = write_model(str(tmp_path), cfg, 17)
    a, b = prompt(cfg, 161, 4), prompt(cfg, 83, 5)
    ra, rb = pk.forward(cfg, w, a), pk.forward(cfg, w, b)
    eng = engine(str(tmp_path), dtype)
    close(whole(eng, a), ra, dtype, "one prompt")
    close(in_portions(eng, a, [70, 91]), ra, dtype, "two long portions")
    close(in_portions(eng, a, [97, 1, 3, 60]), ra, dtype, "portions long and short")
    sa, sb = eng.new_sequence(), eng.new_sequence()
    lg = eng.step([StepItem(sa, a, list(range(len(a)))), StepItem(sb, b, list(range(len(b))))]).cpu().numpy()
    eng.end_sequence(sa)
    eng.end_sequence(sb)
    close(lg[:len(a)], ra, dtype, "first of two prompts in a step")
    close(lg[len(a):], rb, dtype, "second of two prompts in a step")


# ------------------------------------------------------------------ whole models


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt(models, name, dtype):
    d, cfg, w = models[name]
    ids = prompt(cfg, 150, 11, w, dtype)
    close(whole(engine(d, dtype), ids), pk.forward(cfg, w, ids), dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_first_tokens_and_one_token(models, name, dtype):
    d, cfg, w = models[name]
    eng = engine(d, dtype)
    for n in (1, 2, 3):
        ids = prompt(cfg, n, 20 + n, w, dtype)
        close(whole(eng, ids), pk.forward(cfg, w, ids), dtype, f"{name} {n} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_and_decoding(models, name, dtype):
    """Prefill against token-by-token decoding and portions of several sizes, down to two tokens, across page borders,
    window edges and the rows that the convolutions keep."""
    d, cfg, w = models[name]
    ids = prompt(cfg, 200, 13)
    ref = pk.forward(cfg, w, ids)
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
    seqs = [prompt(cfg, n + e, 40 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    refs = [pk.forward(cfg, w, s) for s in seqs]
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
    """A small cache whose slots, pages and state rows go round several times, freed pages poisoned with NaN: a new
    sequence must find a zero state and zero convolution rows, whatever the slot's last owner left."""
    d, cfg, w = models["mixed"]
    eng = engine(d, dtype, max_tokens=320, max_batch=3, max_seq_len=256, poison=True)
    for rnd in range(4):
        seqs = [prompt(cfg, n, 70 + 10 * rnd + i) for i, n in enumerate((90 + rnd, 33, 70))]
        slots = [eng.new_sequence() for _ in seqs]
        cut = [len(s) // 2 + rnd for s in seqs]
        eng.step([StepItem(slots[i], seqs[i][:cut[i]], []) for i in range(3)])
        eng.end_sequence(slots[1])                        # its slot and pages go to the next sequence at once
        late = prompt(cfg, 40, 90 + rnd)
        s_late = eng.new_sequence()
        got_late = eng.step([StepItem(s_late, late, list(range(40)))]).cpu().numpy()
        close(got_late, pk.forward(cfg, w, late), dtype, f"round {rnd}: a sequence in a slot used before")
        for i in (0, 2):
            rest = seqs[i][cut[i]:]
            got = eng.step([StepItem(slots[i], rest, list(range(len(rest))))]).cpu().numpy()
            close(got, pk.forward(cfg, w, seqs[i])[cut[i]:], dtype, f"round {rnd}: sequence {i} continued")
            eng.end_sequence(slots[i])
        eng.end_sequence(s_late)


# ------------------------------------------------------------------ crafted cases


def with_window(cfg, size):
    c = json.loads(json.dumps(cfg))
    for L in c["layers"]:
        if L["type"] == A:
            L["mixer"]["mask"] = {"size": size}
    return c


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,page", [(0, 64), (64, 64), (65, 64), (63, 64), (7, 16), (33, 16), (2, 64)])
def test_one_key_decides(tmp_path, window, page, dtype):
    """One position's key is made to stand out in the scores of the queries after it: its token appears once, its
    embedding is a spike in one channel, and the key matrix reads that channel strongly.  Whether exactly that key is
    seen then decides the output: just inside and just outside the window, at a page border, among hundreds of keys,
    in a prompt and in decoding.  The plain implementation with a window one longer or shorter must disagree, or the
    test would show nothing."""
    cfg = pk.random_config((A,), mlps=[None], taps=0, window=window, scale=1.5, vocab=50, emb_scale=4.0)
    far = 63                                             # the last row of the first page of 64
    ids = prompt(cfg, 300 if window == 0 else 140, 3)
    ids = [t if t != 7 else 8 for t in ids]
    ids[far] = 7                                         # token 7 appears once

    def edit(w):
        w["embed"][7] = 0.0
        w["embed"][7, 5] = 8.0
        w["l0.mix.k"][:, 5] = 1.0
        w["l0.mix.talk"] = np.eye(4) + 0.1 * np.asarray(w["l0.mix.talk"] - np.eye(4))

    w = write_model(str(tmp_path), cfg, 9, edit)
    ref = pk.forward(cfg, w, ids)
    if window:
        edge = far + window                              # the first query that no longer sees the key
        for other in (window - 1, window + 1):
            alt = pk.forward(with_window(cfg, other), w, ids)
            assert rel_err(alt[edge - 1:edge + 1], ref[edge - 1:edge + 1]) > 0.05, "the crafted key does not decide"
    else:
        alt = pk.forward(cfg, w, ids[:far] + [8] + ids[far + 1:])
        assert rel_err(alt[200:], ref[200:]) > 0.05, "the crafted key does not decide"
    eng = engine(str(tmp_path), dtype, page_size=page)
    assert_close(whole(eng, ids), ref, dtype, f"window {window}, prompt")
    assert_close(in_portions(eng, ids, [60, 1]), ref, dtype, f"window {window}, decoding past the key")
    assert_close(in_portions(eng, ids, [far + 1, 2]), ref, dtype, f"window {window}, portions from the key on")
    if window:
        assert_close(in_portions(eng, ids, [far + window - 1, 1, 1, 1, 40]), ref, dtype, f"window {window}, steps at the edge")


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_preferred(tmp_path, dtype):
    """Negative distance factors turn the distance term into a bonus for far keys, so every query looks mostly at the
    oldest keys it may see: every position tests the window's far edge, across several pages."""
    cfg = pk.random_config((A,), mlps=[None], taps=0, window=37, scale=0.5, att_heads=3, kv_heads=3, att_dim=8)

    def edit(w):
        w["l0.mix.r1"] = np.full(3, -6.0, np.float32)
        w["l0.mix.r2"] = np.asarray([0.5, 1.0, 3.0], np.float32)
        w["l0.mix.talk"] = np.eye(3, dtype=np.float32)

    w = write_model(str(tmp_path), cfg, 5, edit)
    ids = prompt(cfg, 180, 2)
    ref = pk.forward(cfg, w, ids)
    assert rel_err(pk.forward(with_window(cfg, 36), w, ids)[40:], ref[40:]) > 0.02
    eng = engine(str(tmp_path), dtype, page_size=16)
    assert_close(whole(eng, ids), ref, dtype, "prompt")
    assert_close(in_portions(eng, ids, [30, 1]), ref, dtype, "decoding")
    assert_close(in_portions(eng, ids, [17, 2, 36, 37, 38]), ref, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", [M, S])
def test_state_far_back(tmp_path, kind, dtype):
    """Gates that forget almost nothing: what the first tokens wrote is still in the state hundreds of tokens later,
    through a prompt and through long decoding."""
    cfg = pk.random_config((kind, kind), mlps=[None, "bare"], taps=2)

    def edit(w):
        for name in w:
            if name.endswith("A_log"):
                w[name] = np.full(w[name].shape, -9.0, np.float32)
            if name.endswith("mix.f.b"):
                w[name] = np.full(w[name].shape, 9.0, np.float32)
            if name.endswith("mix.i.b"):
                w[name] = np.full(w[name].shape, -1.0, np.float32)

    w = write_model(str(tmp_path), cfg, 4, edit)
    ids = prompt(cfg, 420, 6)
    ref = pk.forward(cfg, w, ids)
    # the oracle itself depends on the first tokens at the end: the test would not see a lost state otherwise
    other = pk.forward(cfg, w, prompt(cfg, 20, 99) + ids[20:])
    assert rel_err(other[-1], ref[-1]) > 1e-3
    eng = engine(str(tmp_path), dtype)
    close(whole(eng, ids), ref, dtype, "prompt")
    close(in_portions(eng, ids, [100, 1]), ref, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_running_maximum_starts_at_zero(tmp_path, dtype):
    """Input gates far below zero: the stabiliser of the matrix memory stays at its starting value 0 for the first
    tokens, and the read-out's lower bound exp(-m) = 1 decides the output.  A stabiliser that started at minus
    infinity would give another result, so the plain implementation is checked to depend on it."""
    cfg = pk.random_config((M,), mlps=[None], taps=0, gate_cap=8.0)

    def edit(w):
        w["l0.mix.i.b"] = np.full(w["l0.mix.i.b"].shape, -6.0, np.float32)
        w["l0.mix.i"] = 0.1 * np.asarray(w["l0.mix.i"], np.float32)

    w = write_model(str(tmp_path), cfg, 14, edit)
    ids = prompt(cfg, 60, 3)
    ref = pk.forward(cfg, w, ids)
    eng = engine(str(tmp_path), dtype)
    close(whole(eng, ids), ref, dtype, "prompt")
    close(in_portions(eng, ids, [1]), ref, dtype, "token by token")
    close(in_portions(eng, ids, [7, 2]), ref, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_choice_scores_below_zero(tmp_path, dtype):
    """Corrections so far below zero that every choice score is negative: an implementation that zeroed the experts
    outside the kept groups instead of excluding them would let them beat every allowed one.  The weights stay the
    plain scores."""
    cfg = pk.random_config((A,), taps=0, experts=8, top=2, group_count=4, group_keep=1)

    def edit(w):
        w["l0.mlp.correction"] = np.asarray(-2.0 - 0.5 * np.arange(8) % 3, np.float32)

    w = write_model(str(tmp_path), cfg, 31, edit)
    ids = prompt(cfg, 80, 12, w, dtype)
    ref = pk.forward(cfg, w, ids)
    eng = engine(str(tmp_path), dtype)
    close(whole(eng, ids), ref, dtype, "prompt")
    close(in_portions(eng, ids, [1]), ref, dtype, "token by token")


# ------------------------------------------------------------------ generation


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation(models, dtype):
    """Greedy tokens through Model.generate (the scheduler, batches, the sampler) against the plain implementation."""
    d, cfg, w = models["mixed"]
    prompts = [prompt(cfg, n, 50 + n) for n in (3, 17, 70, 1)]
    m = Model(ModelConfig(compt_type=dtype, nr_ctx=256, max_tokens=1024))
    m.load(d)
    m.init(top_k=0, top_p=1.0, temp=0.0, repeat_penalty=1.0, repeat_last_n=0, seed=0, end_token=-1)
    got = m.generate(prompts, max_new_tokens=12, stop_ids=[]).tokens
    want = [pk.greedy_generate(cfg, w, p, 12) for p in prompts]
    if dtype == "float32":
        assert got == want
        return
    # bfloat16 may turn a near-tie: every token the engine chose must be (within rounding) the best continuation of what
    # it had generated so far, by the plain implementation's logits for that very sequence
    for p, g in zip(prompts, got):
        assert len(g) == 12
        lg = pk.forward(cfg, w, p + g)[len(p) - 1:-1]
        gap = lg.max(-1) - lg[np.arange(12), g]
        assert (gap <= BF16_TOL * np.abs(lg).max()).all(), (g, gap)


def test_trace_replay_program(models, tmp_path):
    """bin/trace_run on a Kudonex folder: portions, a batch, ends, and the logits files."""
    import subprocess
    d, cfg, w = models["other"]
    a, b = prompt(cfg, 9, 1), prompt(cfg, 5, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:6], "want": [0, 5]}, {"id": "b", "tokens": b[:4], "want": [3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[6:7], "want": [0]}, {"id": "b", "tokens": b[4:5], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[7:], "want": [1]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "out")
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    ra, rb = pk.forward(cfg, w, a), pk.forward(cfg, w, b)
    want = [np.stack([ra[0], ra[5], rb[3]]), np.stack([ra[6], rb[4]]), np.stack([ra[8]])]
    for n, ref in enumerate(want):
        got = np.fromfile(os.path.join(out, f"{n}.f32"), "<f4").reshape(ref.shape)
        assert_close(got, ref, "float32", f"step {n}")


def test_command_line(models):
    """bin/llama on a Kudonex folder: greedy tokens of two requests, float32."""
    import subprocess
    d, cfg, w = models["mixed"]
    prompts = [prompt(cfg, n, 90 + n) for n in (7, 12)]
    want = [pk.greedy_generate(cfg, w, p, 6) for p in prompts]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = [os.path.join(root, "bin", "llama"), "-m", d, "-d", "float32", "-c", "128", "-n", "6", "--temp", "0", "--top_k", "0",
            "--top_p", "1", "--repeat_penalty", "1", "-s", "1"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    r = subprocess.run(args, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = [[int(t) for t in ln.split(": ")[1].split(",")] for ln in r.stdout.splitlines() if ln.startswith("[")]
    assert got == want
