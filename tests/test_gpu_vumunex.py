"""Vumunex on the layered runtime against the plain restatement in tests/vumunex_oracle.py: every mechanism alone, prefill against
token-by-token decoding, portions of several sizes, interleaved requests, pages and slots used again, keys far away, at page borders
and on both sides of a window's edge, the sink term, the first tokens of a sequence, long decoding, sizes that defeat every vector
width, values that happen to be equal or 1, and greedy generation through the engine's own entry points.  Small random models, each
written to a temporary folder and loaded by the engine like any model folder."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from nano_b200 import engine as E, modeldir as md

import vumunex_oracle as O

pytestmark = pytest.mark.gpu

WIN = {"heads": 3, "dim": 20, "vdim": 12, "kv_rank": 40, "scale": 0.28, "mask": {"size": 21}}
ROT = {"heads": 5, "dim": 12, "rot_dim": 8, "vdim": 20, "kv_rank": 24, "scale": 0.35, "rot": {"dims": 8, "base": 300.0}}
DENSE = {"kind": "dense", "ff": 56}
MOE = {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 24, "limit": 1.2}, "shared": {"ff": 40, "limit": 0.8}}


def win(**kw):
    m = copy.deepcopy(WIN)
    m.update(kw)
    return {k: v for k, v in m.items() if v is not None}


def rot(**kw):
    m = copy.deepcopy(ROT)
    m.update(kw)
    return {k: v for k, v in m.items() if v is not None}


def build(tmp_path, cfg, seed=0, f32=True, max_tokens=512, keep=False, chunk=None, name="m", tweak=None, layer_scale=True):
    w = md.vumunex_random(cfg, seed, layer_scale=layer_scale)
    if tweak:
        tweak(w)
        w = {k: md.bf16_round(v) for k, v in w.items()}          # the file holds bfloat16: the oracle reads the same numbers
    path = md.write_model_dir(str(tmp_path / name), cfg, w)
    os.environ.pop("NB200_KEEP_RESIDUALS", None); os.environ.pop("NB200_CHUNK", None)
    if keep: os.environ["NB200_KEEP_RESIDUALS"] = "1"
    if chunk: os.environ["NB200_CHUNK"] = str(chunk)
    try:
        eng = E.Engine(path, max_tokens, flags=E.FLAG_F32 if f32 else 0)
    finally:
        os.environ.pop("NB200_KEEP_RESIDUALS", None); os.environ.pop("NB200_CHUNK", None)
    return eng, w


def toks(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).astype(np.uint32)


def rows(got, want):
    """rms of the difference over the rms of the reference, per row (mean taken off: logits are shift-invariant)"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1) + 1e-30)


def rel(got, want):
    return float(rows(got, want).max())


F32_TOL, BF16_TOL = 3e-5, 4e-2


def close_bf16(got, want):
    """bfloat16 products may turn a router's close call the other way, which moves that token's row alone: nearly every row stays
    within the tolerance, the typical row far within it, and no row is far off"""
    r = rows(got, want)
    return np.median(r) < BF16_TOL / 3 and np.mean(r > BF16_TOL) <= 0.03 and r.max() < 8 * BF16_TOL


def whole(eng, t, want=None):
    s = eng.seq_open()
    out = eng.step(s, t, range(len(t)) if want is None else want)
    eng.seq_close(s)
    return out


def in_cuts(eng, t, cuts):
    s = eng.seq_open()
    out, at = [], 0
    for c in cuts:
        part = t[at:at + c]
        if len(part):
            out.append(eng.step(s, part, range(len(part))))
        at += c
    eng.seq_close(s)
    assert at >= len(t)
    return np.concatenate(out)


def check_alone(tmp_path, cfg, n=75, tweak=None, layer_scale=True):
    eng, w = build(tmp_path, cfg, keep=True, tweak=tweak, layer_scale=layer_scale)
    t = toks(cfg, n)
    trace = []
    ref = O.forward(cfg, w, t, trace)
    got = whole(eng, t)
    res = eng.read_residual(0, len(t))
    assert np.abs(res - trace[0]).max() <= 3e-5 * np.abs(trace[0]).max()
    assert rel(got, ref) < F32_TOL
    for cuts in ([1] * n, [2, 3, 4] * (n // 9 + 1), [5, 1, 30, 2, n]):
        assert rel(in_cuts(eng, t, cuts), ref) < F32_TOL, cuts[:3]
    eng.close()


MIXERS = [
    ("latent_attention", WIN),
    ("latent_attention", win(heads=1, dim=8, vdim=8, kv_rank=8, mask={"size": 1})),                       # every query sees itself alone (and the sink)
    ("latent_attention", win(heads=9, dim=7, vdim=5, kv_rank=33, mask={"size": 32})),                    # two blocks of heads; sizes no vector width divides; a page-wide window
    ("latent_attention", win(heads=4, dim=64, vdim=64, kv_rank=64, scale=0.125, mask={"size": 33})),     # the exact-rank instance
    ("latent_attention", win(heads=2, dim=16, vdim=24, kv_rank=128, mask={"size": 1000})),               # a window wider than the prompt
    ("latent_attention", win(heads=2, dim=40, vdim=8, kv_rank=260, scale=0.1, mask={"size": 50})),       # the widest register tile
    ("latent_attention_2", ROT),
    ("latent_attention_2", rot(heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=16, rot={"dims": 16, "base": 10000.0})),       # sizes all equal
    ("latent_attention_2", rot(heads=3, dim=5, rot_dim=6, vdim=9, kv_rank=30, rot={"dims": 2, "base": 7.0})),               # one pair turns, the rest of the part passes
    ("latent_attention_2", rot(heads=8, dim=32, rot_dim=32, vdim=32, kv_rank=128, scale=0.11, rot={"dims": 32, "base": 2e5})),
    ("latent_attention_2", rot(heads=2, dim=24, rot_dim=4, vdim=16, kv_rank=256, scale=0.2, rot={"dims": 4, "base": 50.0})),
    ("latent_attention_2", rot(heads=10, dim=3, rot_dim=2, vdim=4, kv_rank=13, rot={"dims": 2, "base": 2.0})),
]


# ---- each mechanism alone: one layer, no feed-forward, residual after the layer and logits; whole, token by token, short portions ----
@pytest.mark.parametrize("kind,mixer", MIXERS)
def test_mixer_alone(tmp_path, kind, mixer):
    check_alone(tmp_path, md.vumunex_config(61, 72, [(kind, mixer, None)], streams=2, scale=3.0))


@pytest.mark.parametrize("mlp", [
    DENSE, {"kind": "dense", "ff": 7}, {"kind": "dense", "ff": 129}, MOE,
    {"kind": "moe", "router": {"experts": 4, "top": 1}, "expert": {"ff": 9, "limit": 0.5}, "shared": {"ff": 17, "limit": 3.0}},
    {"kind": "moe", "router": {"experts": 3, "top": 3}, "expert": {"ff": 16, "limit": 2.0}},                  # every expert chosen, no shared expert
    {"kind": "moe", "router": {"experts": 40, "top": 4}, "expert": {"ff": 8, "limit": 1.0}, "shared": {"ff": 8, "limit": 1.0}},
])
def test_feed_forward(tmp_path, mlp):
    check_alone(tmp_path, md.vumunex_config(50, 40, [("latent_attention_2", rot(heads=2), mlp)], streams=3, scale=2.0), n=40)


def test_clamps_and_score_weights_show(tmp_path):
    """Large gate and up products: the clamps bite on most coordinates, and the oracle itself tells the limits and the renormalised
    weights apart from their absence."""
    mlp = {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 12, "limit": 0.7}, "shared": {"ff": 10, "limit": 0.4}}
    cfg = md.vumunex_config(40, 32, [("latent_attention", win(heads=2), mlp)], streams=1, residual_mult=1.0)

    def big(w):
        for k in w:
            if k.endswith(".gate") or k.endswith(".up"):
                w[k] *= 4.0
    eng, w = build(tmp_path, cfg, tweak=big)
    t = toks(cfg, 50)
    ref = O.forward(cfg, w, t)
    loose = copy.deepcopy(cfg); loose["layers"][0]["mlp"]["expert"]["limit"] = 50.0
    assert rel(O.forward(loose, w, t), ref) > 100 * F32_TOL
    loose = copy.deepcopy(cfg); loose["layers"][0]["mlp"]["shared"]["limit"] = 50.0
    assert rel(O.forward(loose, w, t), ref) > 100 * F32_TOL
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [3, 1, 2, 44]), ref) < F32_TOL
    eng.close()


@pytest.mark.parametrize("width,vocab", [(50, 61), (37, 33), (130, 7)])
def test_ragged_widths(tmp_path, width, vocab):
    """widths and vocabularies that no vector width divides, through every product of a layer"""
    cfg = md.vumunex_config(vocab, width, [("latent_attention_2", rot(heads=3), MOE), ("latent_attention", win(heads=2, kv_rank=18), DENSE)], streams=3, scale=2.0)
    eng, w = build(tmp_path, cfg)
    t = toks(cfg, 45)
    ref = O.forward(cfg, w, t)
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [3, 1, 2, 4, 35]), ref) < F32_TOL
    eng.close()
    eng, w = build(tmp_path, cfg, f32=False, name="b")
    assert close_bf16(whole(eng, t), ref) and close_bf16(in_cuts(eng, t, [40, 1, 1, 3]), ref)
    eng.close()


@pytest.mark.parametrize("streams,ls", [(None, False), (1, True), (2, False), (5, True), (8, True)])
def test_streams_and_layer_scale(tmp_path, streams, ls):
    """no connection tensors at all (plain residual), one stream with weights, several streams; with and without the layer scale"""
    cfg = md.vumunex_config(40, 48, [("latent_attention", win(heads=2), DENSE), ("latent_attention_2", rot(heads=2), None), ("latent_attention_2", rot(heads=2), MOE)],
                            streams=streams, residual_mult=0.7, scale=1.5)
    eng, w = build(tmp_path, cfg, keep=True, layer_scale=ls)
    assert ("l0.hc1.in" in w) == (streams is not None) and ("l0.ls1" in w) == ls
    t = toks(cfg, 45)
    trace = []
    ref = O.forward(cfg, w, t, trace)
    assert rel(whole(eng, t), ref) < F32_TOL
    for i, x in enumerate(trace):
        assert np.abs(eng.read_residual(i, len(t)) - x).max() <= 3e-5 * np.abs(x).max(), i
    assert rel(in_cuts(eng, t, [1] * 45), ref) < F32_TOL
    eng.close()


def mixed_cfg(vocab=67, streams=3):
    layers = [("latent_attention_2", ROT, DENSE), ("latent_attention", WIN, MOE), ("latent_attention_2", rot(heads=2, rot_dim=4, rot={"dims": 4, "base": 40.0}), None),
              ("latent_attention", win(heads=2, mask={"size": 40}), DENSE), ("latent_attention_2", ROT, MOE)]
    return md.vumunex_config(vocab, 56, layers, streams=streams, residual_mult=0.4, scale=4.0, loop=(1, 4, 2))


@pytest.mark.parametrize("loop", [None, (0, 2, 1), (0, 3, 3), (1, 1, 4), (2, 3, 2), (0, 1, 2)])
def test_layer_order_and_loops(tmp_path, loop):
    """the residual after every layer run: no loop, a span that runs once, the whole stack several times, an empty span, spans at either end"""
    layers = [("latent_attention", WIN, DENSE), ("latent_attention_2", ROT, None), ("latent_attention_2", rot(heads=2), MOE)]
    cfg = md.vumunex_config(40, 48, layers, streams=2, loop=loop)
    eng, w = build(tmp_path, cfg, keep=True)
    t = toks(cfg, 50)
    trace = []
    ref = O.forward(cfg, w, t, trace)
    assert len(trace) == len(O.run_order(cfg))
    assert rel(whole(eng, t), ref) < F32_TOL
    for i, x in enumerate(trace):
        assert np.abs(eng.read_residual(i, len(t)) - x).max() <= 3e-5 * np.abs(x).max(), i
    assert rel(in_cuts(eng, t, [20] + [1] * 30), ref) < F32_TOL          # every pass has a cache of its own
    eng.close()


# ---- prefill against token-by-token decoding, portions down to two tokens, the engine's own chunking ----
@pytest.mark.parametrize("f32", [True, False])
def test_portions_and_decoding(tmp_path, f32):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, f32=f32)
    t = toks(cfg, 150)
    ref = O.forward(cfg, w, t)
    ok = (lambda a, b: rel(a, b) < F32_TOL) if f32 else close_bf16
    full = whole(eng, t)
    assert ok(full, ref)
    for cuts in ([1] * 150, [2] * 75, [3, 2, 64, 5, 1, 1, 33, 2, 39], [100] + [1] * 50, [31, 1, 32, 33, 53], [7] * 22):
        got = in_cuts(eng, t, cuts)
        assert ok(got, ref), cuts[:4]
        assert ok(got, full), cuts[:4]
    eng.close()
    eng, _ = build(tmp_path, cfg, f32=f32, chunk=16, name="c")       # chunks of 16 inside one step
    assert ok(whole(eng, t), ref)
    eng.close()


def test_batches_of_unequal_requests_and_reuse(tmp_path):
    """Requests interleaved step by step equal each alone; pages and slots that were freed hold other requests' numbers."""
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, max_tokens=400)
    ts = [toks(cfg, n, seed=10 + n) for n in (90, 33, 140, 5)]
    refs = [O.forward(cfg, w, t) for t in ts]
    free0 = eng.free_pages
    for rounds in range(2):                      # the second round runs in pages and slots of the first
        seqs = [eng.seq_open() for _ in ts]
        outs, at = [[] for _ in ts], [0] * len(ts)
        sizes = [[40, 1, 1, 48], [2, 31], [64, 64, 3, 1, 1, 1, 6], [5]]
        step = 0
        while any(a < len(t) for a, t in zip(at, ts)):
            for i, t in enumerate(ts):
                if at[i] >= len(t) or step >= len(sizes[i]):
                    continue
                n = sizes[i][step]
                outs[i].append(eng.step(seqs[i], t[at[i]:at[i] + n], range(n)))
                at[i] += n
                if at[i] == len(t):
                    eng.seq_close(seqs[i])
            step += 1
        for o, r in zip(outs, refs):
            assert rel(np.concatenate(o), r) < F32_TOL
        assert eng.free_pages == free0
    eng.close()


def stand_out(w, tok, heads, dim, rot_dim, key_gain=2.0, query=1.5):
    """Coordinate 0 of the mixer's input is positive for token `tok` alone; every head's key reads it and every query is constant, so a
    query's weight sits on token `tok` wherever it is in sight."""
    w["embed"][:, :] *= 0.2
    w["embed"][:, 0] = -3.0; w["embed"][tok, 0] = 3.0
    w["l0.norm1"][0] = 1.0
    w["l0.mix.dkv"][:] *= 0.05; w["l0.mix.dkv"][0, :] = 0.0; w["l0.mix.dkv"][0, 0] = 2.0
    w["l0.mix.dkv.norm"][0] = 1.0
    w["l0.mix.uk"][:] = 0.0
    w["l0.mix.q"][:] = 0.0
    for h in range(heads):
        w["l0.mix.uk"][h * dim, 0] = key_gain
        w["l0.mix.q"][h * (dim + rot_dim), 0] = -query          # the input's coordinate 0 is negative for the other tokens: a positive query there


# ---- a far key among hundreds, where random weights would hide it: one key made to stand out, at and around page borders ----
@pytest.mark.parametrize("where", [0, 31, 32, 33, 95, 200])
def test_far_key_shows(tmp_path, where):
    """Token `where` is the only one of its id and its key is made large: queries hundreds of positions later put their weight on it, so
    losing that key (or its latent, which is its value) would change the logits far beyond the tolerance."""
    mixer = rot(heads=2, dim=16, rot_dim=4, vdim=16, kv_rank=24, scale=1.0, rot={"dims": 4, "base": 100.0})
    cfg = md.vumunex_config(40, 48, [("latent_attention_2", mixer, None)], streams=2, scale=1.0)
    t = toks(cfg, 330, seed=3)
    t[t == 7] = 8
    t[where] = 7
    eng, w = build(tmp_path, cfg, max_tokens=400, tweak=lambda w: stand_out(w, 7, 2, 16, 4))
    ref = O.forward(cfg, w, t)
    t2 = t.copy(); t2[where] = 9
    assert rel(O.forward(cfg, w, t2)[-20:], ref[-20:]) > 100 * F32_TOL          # the key matters to the last queries
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [290] + [1] * 40), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [29, 2, 2, 31, 1, 1, 64, 130, 3, 4, 63]), ref) < F32_TOL
    eng.close()


# ---- the window's edge: a key that stands out is seen by exactly `size` queries, itself included ----
@pytest.mark.parametrize("size", [1, 5, 32, 33, 45, 64, 97])
def test_window_edges_show(tmp_path, size):
    """The oracle itself tells size from size - 1 and size + 1 here (the stand-out key enters or leaves one query's sight); the engine
    follows the right one in a prompt, token by token, in ragged portions, and when the edge falls on the first token of a portion."""
    mixer = win(heads=2, dim=16, vdim=16, kv_rank=24, scale=1.0, mask={"size": size})
    cfg = md.vumunex_config(40, 48, [("latent_attention", mixer, None)], streams=2, scale=1.0)
    n, where = 230, 70
    t = toks(cfg, n, seed=5)
    t[t == 7] = 8
    t[where] = 7; t[3] = 7

    def tweak(w):
        stand_out(w, 7, 2, 16, 0)
        w["l0.mix.sink"][:] = -4.0
    eng, w = build(tmp_path, cfg, max_tokens=300, tweak=tweak)
    ref = O.forward(cfg, w, t)
    for other in (size - 1, size + 1):
        if other < 1:
            continue
        c2 = copy.deepcopy(cfg); c2["layers"][0]["mixer"]["mask"]["size"] = other
        edge = where + min(size, other)          # the first query the two sizes disagree on
        assert rel(O.forward(c2, w, t)[edge:edge + 1], ref[edge:edge + 1]) > 100 * F32_TOL
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [60] + [1] * 170), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [where + size - 1, 2, 2, 1, 64, 3, n]), ref) < F32_TOL          # the last query that sees it ends a portion
    assert rel(in_cuts(eng, t, [where + size, 2, 31, 1, 2, n]), ref) < F32_TOL                  # the first that does not begins one
    assert rel(in_cuts(eng, t, [4, 2] * 20 + [37, 3] * 5 + [1] * 30), ref) < F32_TOL
    eng.close()


def test_sink_shows(tmp_path):
    """A large sink takes most of the weight (the output shrinks), a very negative one none; each head has its own; a sink far above
    every score must not overflow.  The oracle tells them apart; the engine follows, also through the key splits of a long decode."""
    mixer = win(heads=3, dim=16, vdim=16, kv_rank=24, scale=0.5, mask={"size": 300})
    cfg = md.vumunex_config(40, 48, [("latent_attention", mixer, None)], streams=1, scale=2.0)
    t = toks(cfg, 200, seed=9)
    refs = []
    for i, sink in enumerate(([6.0, -30.0, 0.5], [0.0, 0.0, 0.0], [120.0, 3.0, -120.0])):
        def tweak(w, sink=sink):
            w["l0.mix.sink"][:] = np.asarray(sink, np.float32)
        eng, w = build(tmp_path, cfg, tweak=tweak, name="s%d" % i)
        ref = O.forward(cfg, w, t)
        refs.append(ref)
        assert np.isfinite(ref).all()
        assert rel(whole(eng, t), ref) < F32_TOL
        assert rel(in_cuts(eng, t, [150] + [1] * 50), ref) < F32_TOL
        assert rel(in_cuts(eng, t, [2, 3] * 40), ref) < F32_TOL
        eng.close()
    assert rel(refs[0], refs[1]) > 100 * F32_TOL and rel(refs[2], refs[1]) > 100 * F32_TOL


def test_rotation_shows(tmp_path):
    """The oracle tells the interleaved pairing from a rotation that is left out; the engine follows the pairing, far into a sequence."""
    mixer = rot(heads=2, dim=8, rot_dim=16, vdim=16, kv_rank=16, scale=0.6, rot={"dims": 16, "base": 50.0})
    cfg = md.vumunex_config(40, 48, [("latent_attention_2", mixer, None)], streams=2, scale=2.0)

    def tweak(w):
        w["l0.mix.q"][:] *= 2.0
    eng, w = build(tmp_path, cfg, tweak=tweak)
    t = toks(cfg, 300, seed=3)
    ref = O.forward(cfg, w, t)
    still = copy.deepcopy(cfg); still["layers"][0]["mixer"]["rot"]["dims"] = 0
    assert rel(O.forward(still, w, t), ref) > 100 * F32_TOL
    u = np.random.default_rng(1).standard_normal((3, 2, 8))
    r = O.rotate_pairs(u, {"dims": 4, "base": 100.0}, np.array([0.0, 1.0, 5.0]))
    z = (u[2, 1, 2] + 1j * u[2, 1, 3]) * np.exp(1j * 5 * 100.0 ** (-2.0 / 4))
    assert np.allclose([r[2, 1, 2], r[2, 1, 3]], [z.real, z.imag]) and np.array_equal(r[..., 4:], u[..., 4:]) and np.allclose(r[0], u[0])
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [250] + [1] * 50), ref) < F32_TOL
    eng.close()


def test_long_prompt_splits_keys_in_decoding(tmp_path):
    """Short portions deal the key pages in sight out to several blocks and merge: same logits as the whole prompt, with and without a window."""
    cfg = md.vumunex_config(40, 48, [("latent_attention_2", rot(heads=3), DENSE), ("latent_attention", win(heads=3, mask={"size": 200}), None)], streams=2, scale=2.0)
    eng, w = build(tmp_path, cfg, max_tokens=400)
    t = toks(cfg, 330, seed=6)
    ref = O.forward(cfg, w, t)
    assert rel(in_cuts(eng, t, [300] + [1] * 20 + [2, 3, 4, 1]), ref) < F32_TOL
    eng.close()


def test_long_decoding(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, max_tokens=700)
    t = toks(cfg, 650, seed=8)
    ref = O.forward(cfg, w, t)
    got = in_cuts(eng, t, [3] + [1] * 647)
    assert rel(got, ref) < 2 * F32_TOL
    eng.close()


def test_first_tokens_and_single_token_requests(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg)
    for n in (1, 2, 3, 5):
        t = toks(cfg, n, seed=20 + n)
        ref = O.forward(cfg, w, t)
        assert rel(whole(eng, t), ref) < F32_TOL
        assert rel(in_cuts(eng, t, [1] * n), ref) < F32_TOL
    t = toks(cfg, 9, seed=30)
    ref = O.forward(cfg, w, t)
    for _ in range(3):          # the same slot and pages again
        assert rel(in_cuts(eng, t, [1, 3, 5]), ref) < F32_TOL
    eng.close()


def test_bf16_close_to_oracle(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, f32=False)
    t = toks(cfg, 120)
    ref = O.forward(cfg, w, t)
    assert close_bf16(whole(eng, t), ref)
    assert close_bf16(in_cuts(eng, t, [90] + [1] * 30), ref)
    eng.close()


# ---- generation through the engine's own entry points ----
def test_greedy_generation(tmp_path):
    cfg = mixed_cfg(vocab=53)
    eng, w = build(tmp_path, cfg)
    prompt = toks(cfg, 17, seed=4)
    total = 60
    ids = np.zeros(total + 1, np.uint32); ids[:17] = prompt
    eng.decode_greedy(ids, 17, total)
    # the oracle follows the engine's ids and must agree on every choice whose margin is not a rounding matter
    ref = O.forward(cfg, w, ids[:total - 1])
    for pos in range(16, total - 1):
        top = np.sort(ref[pos])[-2:]
        if top[1] - top[0] > 1e-3:
            assert int(np.argmax(ref[pos])) == int(ids[pos + 1]), pos
    ids2 = np.zeros(total + 1, np.uint32); ids2[:17] = prompt
    for pos in range(total - 1):
        nxt = eng.next_greedy(ids2, pos, 1 if pos < 16 else 0)
        if pos >= 16:
            ids2[pos + 1] = nxt
    assert np.array_equal(ids[:total], ids2[:total])
    eng.close()
    # the generation command on the same folder
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "nano_b200.generate", "--model", str(tmp_path / "m"), "--prompt-ids", ",".join(str(int(x)) for x in prompt),
                        "--max-new", str(total - 17), "--dtype", "float32"], cwd=root, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(x) for x in p.stdout.split()] == [int(x) for x in ids[:total]]


def test_sampled_generation_and_penalty(tmp_path):
    """The device sampler and the repetition penalty on the implicit sequence."""
    cfg = mixed_cfg(vocab=80)
    eng, w = build(tmp_path, cfg)
    prompt = [5, 17, 3, 44]
    ids = np.zeros(32, np.uint32); ids[:4] = prompt
    for pos in range(3):
        eng.next_greedy(ids, pos, 1)
    tok, top6 = eng.next_sampled(ids, 3, 1.0, 0.8, 0.95, 0.01)
    ref = O.forward(cfg, w, prompt)[-1]
    assert top6[0] == int(np.argmax(ref)) and tok == top6[0]          # a coin near 0 takes the most probable token
    eng.forward(5, 0); eng.forward(17, 1)                             # position 0 starts over
    assert rel(eng.logits()[None, :], O.forward(cfg, w, [5, 17])[-1:]) < F32_TOL
    pen = O.forward(cfg, w, [5, 17, 3])[-1].copy()
    for i in (5, 17):
        pen[i] = pen[i] / 50.0 if pen[i] > 0 else pen[i] * 50.0
    ids[:3] = [5, 17, 3]
    assert eng.next_greedy(ids, 2, 0, 50.0) == int(np.argmax(pen))
    eng.close()


def test_bad_folders_are_refused(tmp_path):
    cfg = md.vumunex_config(30, 32, [("latent_attention_2", rot(rot={"dims": 10, "base": 10.0}), None)])
    with pytest.raises(E.NB200Error):          # more turning coordinates than the rotated part has
        build(tmp_path, cfg, name="a")
    cfg = md.vumunex_config(30, 32, [("latent_attention", win(mask={"size": 0}), None)])
    with pytest.raises(E.NB200Error):          # an empty window
        build(tmp_path, cfg, name="b")
    cfg = md.vumunex_config(30, 32, [("latent_attention", WIN, None)], streams=3)
    w = md.vumunex_random(cfg)
    del w["l0.hc1.mix"]
    path = md.write_model_dir(str(tmp_path / "c"), cfg, w)
    with pytest.raises(E.NB200Error):          # several streams without their mixing matrix
        E.Engine(path, 64)
    cfg = md.vumunex_config(30, 32, [("latent_attention", WIN, None)], streams=9)
    with pytest.raises(E.NB200Error):          # more streams than the update kernel holds
        build(tmp_path, cfg, name="d")


def test_replay_command(tmp_path):
    """bin/trace_run on a Vumunex folder: portions, single tokens, a step that wants nothing, two requests one after the other."""
    cfg = mixed_cfg()
    w = md.vumunex_random(cfg, 2)
    path = md.write_model_dir(str(tmp_path / "m"), cfg, w)
    a, b = toks(cfg, 70, seed=1), toks(cfg, 9, seed=2)
    ra, rb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40].tolist(), "want": [39, 3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[40:42].tolist(), "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[42:43].tolist(), "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[43:70].tolist(), "want": [26]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": b.tolist(), "want": [8]}], "end": ["b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        out = tmp_path / ("out_" + dtype)
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.split("\n") if l.startswith("done")] == ["done %d" % i for i in range(5)]
        V = cfg["vocab"]
        g0 = np.fromfile(out / "0.f32", "<f4").reshape(-1, V)
        assert rel(g0, ra[[39, 3]]) < tol
        assert not (out / "1.f32").exists()
        assert rel(np.fromfile(out / "2.f32", "<f4").reshape(-1, V), ra[[42]]) < tol
        assert rel(np.fromfile(out / "3.f32", "<f4").reshape(-1, V), ra[[69]]) < tol
        assert rel(np.fromfile(out / "4.f32", "<f4").reshape(-1, V), rb[[8]]) < tol
