"""Gokinex on the layered runtime against the plain restatement in tests/gokinex_oracle.py: every mechanism alone, prefill against
token-by-token decoding, portions of several sizes, interleaved requests, pages and slots used again, far keys at page borders, far
tokens carried by slow states, the first tokens of a sequence, long decoding, sizes that defeat every vector width, values that
happen to be equal or 1, and greedy generation through the engine's own entry points.  Small random models, each written to a
temporary folder and loaded by the engine like any model folder."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from nano_b200 import engine as E, modeldir as md

import gokinex_oracle as O

pytestmark = pytest.mark.gpu

SCALING = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 64}
ATT = {"heads": 6, "kv_heads": 2, "dim": 20, "vdim": 24, "scale": 0.3, "diff": 0.35, "rot": {"dims": 12, "base": 500.0, "scaling": SCALING}}
SSD = {"heads": 4, "vdim": 12, "state": 10, "groups": 2, "conv": 3, "norm_groups": 2}
DENSE = {"kind": "dense", "ff": 56}
MOE = {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 24}, "shared": {"ff": 40}}
BIGRAM = {"buckets": 37, "mul_prev": 11, "mul_cur": 5}


def att(**kw):
    m = copy.deepcopy(ATT)
    m.update(kw)
    return {k: v for k, v in m.items() if v is not None}


def ssd(**kw):
    m = dict(SSD)
    m.update(kw)
    return m


def build(tmp_path, cfg, seed=0, f32=True, max_tokens=512, keep=False, chunk=None, name="m", tweak=None):
    w = md.gokinex_random(cfg, seed)
    if tweak:
        tweak(w)
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


def check_alone(tmp_path, cfg, n=75, tweak=None):
    eng, w = build(tmp_path, cfg, keep=True, tweak=tweak)
    t = toks(cfg, n)
    trace = []
    ref = O.forward(cfg, w, t, np.float64, trace)
    got = whole(eng, t)
    res = eng.read_residual(0, len(t))
    assert np.abs(res - trace[0]).max() <= 3e-5 * np.abs(trace[0]).max()
    assert rel(got, ref) < F32_TOL
    for cuts in ([1] * n, [2, 3, 4] * (n // 9 + 1), [5, 1, 30, 2, n]):
        assert rel(in_cuts(eng, t, cuts), ref) < F32_TOL, cuts[:3]
    eng.close()


MIXERS = [
    ("attention", ATT),
    ("attention", att(heads=4, kv_heads=4, dim=8, vdim=8, rot={"dims": 8, "base": 100.0})),                       # every coordinate turns, no scaling, one head per kv head
    ("attention", att(heads=3, kv_heads=1, dim=37, vdim=33, rot={"dims": 2, "base": 7.0, "scaling": SCALING})),   # one pair turns; odd sizes
    ("attention", att(heads=5, kv_heads=5, dim=12, vdim=70, rot=None, diff=0.0)),                                 # no rotation, diff 0
    ("attention", att(heads=16, kv_heads=2, dim=16, vdim=32, scale=0.25, diff=0.8)),                              # two blocks of heads
    ("attention", att(heads=12, kv_heads=4, dim=64, vdim=128, scale=0.125, rot={"dims": 64, "base": 1e4, "scaling": {"factor": 6.0, "low": 1.5, "high": 5.0, "original": 40}})),
    ("attention", att(heads=2, kv_heads=1, dim=132, vdim=200, scale=0.05)),
    ("mamba2", SSD),
    ("mamba2", ssd(heads=1, vdim=8, state=1, groups=1, conv=1, norm_groups=1)),
    ("mamba2", ssd(heads=6, vdim=7, state=33, groups=3, conv=2, norm_groups=3)),
    ("mamba2", ssd(heads=3, vdim=40, state=70, groups=1, conv=4, norm_groups=1)),
    ("mamba2", ssd(heads=8, vdim=64, state=128, groups=2, conv=4, norm_groups=4)),                                # four columns per warp
    ("mamba2", ssd(heads=2, vdim=16, state=130, groups=2, conv=5, norm_groups=2)),
]


# ---- each mechanism alone: one layer, no feed-forward, residual after the layer and logits; whole, token by token, short portions ----
@pytest.mark.parametrize("kind,mixer", MIXERS)
def test_mixer_alone(tmp_path, kind, mixer):
    check_alone(tmp_path, md.gokinex_config(61, 72, [(kind, mixer, None)], scale=3.0, bigram=BIGRAM))


def test_embedding_pairs(tmp_path):
    """no pair table; a table of one bucket; multipliers that overflow 32 bits when multiplied by a token id"""
    for bg in (None, {"buckets": 1, "mul_prev": 3, "mul_cur": 1}, {"buckets": 251, "mul_prev": 4000000007, "mul_cur": 3999999979}):
        check_alone(tmp_path, md.gokinex_config(300, 40, [("mamba2", SSD, None)], scale=0.5, bigram=bg), n=40)


@pytest.mark.parametrize("mlp", [DENSE, {"kind": "dense", "ff": 7}, {"kind": "dense", "ff": 129}, MOE,
                                 {"kind": "moe", "router": {"experts": 4, "top": 1}, "expert": {"ff": 9}, "shared": {"ff": 5}},
                                 {"kind": "moe", "router": {"experts": 3, "top": 3}, "expert": {"ff": 16}},                     # every expert, no shared expert
                                 {"kind": "moe", "router": {"experts": 40, "top": 4}, "expert": {"ff": 8}, "shared": {"ff": 64}}])
def test_feed_forward(tmp_path, mlp):
    cfg = md.gokinex_config(50, 64, [("mamba2", SSD, mlp)], scale=2.0, bigram=BIGRAM)
    eng, w = build(tmp_path, cfg, keep=True)
    t = toks(cfg, 80)
    trace = []
    ref = O.forward(cfg, w, t, np.float64, trace)
    assert rel(whole(eng, t), ref) < F32_TOL
    assert np.abs(eng.read_residual(0, len(t)) - trace[0]).max() <= 3e-5 * np.abs(trace[0]).max()
    assert rel(in_cuts(eng, t[:30], [1] * 20 + [3, 2, 4, 1]), ref[:30]) < F32_TOL
    eng.close()


def test_score_weights_the_experts_input(tmp_path):
    """silu is not homogeneous: with large gate products, weighting the output instead of the input is a different number"""
    mlp = {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 16}}

    def big(w):
        for k in w:
            if k.endswith(".gate") and ".e" in k:
                w[k] = md.bf16_round(w[k] * 6.0)
    cfg = md.gokinex_config(50, 48, [("mamba2", SSD, mlp)], scale=2.0)
    eng, w = build(tmp_path, cfg, tweak=big)
    t = toks(cfg, 40)
    ref = O.forward(cfg, w, t, np.float64)
    tt = {k: v.astype(np.float64) for k, v in w.items()}
    h = np.random.default_rng(0).standard_normal((8, 48))
    s = O.sigmoid(h @ tt["l0.mlp.router"].T)
    wrong = sum(s[:, e:e + 1] * O.gated(tt, "l0.mlp.e%d." % e, h, O.silu) for e in range(2))
    right = sum(O.gated(tt, "l0.mlp.e%d." % e, s[:, e:e + 1] * h, O.silu) for e in range(2))
    assert np.abs(wrong - right).max() > 1e-2 * np.abs(right).max()
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [1] * 40), ref) < F32_TOL
    eng.close()


def mixed_cfg(vocab=97, width=72):
    a2 = att(heads=4, kv_heads=1, dim=16, vdim=40, diff=0.6)
    return md.gokinex_config(vocab, width, [("mamba2", SSD, DENSE), ("attention", ATT, MOE), ("attention", a2, None), ("mamba2", ssd(heads=2, vdim=20, state=16, groups=1), MOE),
                                            ("attention", att(kv_from=1), DENSE), ("attention", att(kv_from=2, heads=4, kv_heads=1, dim=16, vdim=40, diff=0.2), None),
                                            ("mamba2", SSD, None)], scale=4.0, bigram=BIGRAM)


def test_layer_order_and_shared_keys(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, keep=True)
    t = toks(cfg, 60)
    trace = []
    ref = O.forward(cfg, w, t, np.float64, trace)
    got = whole(eng, t)
    for r, x in enumerate(trace):
        assert np.abs(eng.read_residual(r, len(t)) - x).max() <= 4e-5 * np.abs(x).max(), f"layer {r}"
    assert rel(got, ref) < F32_TOL
    eng.close()


# ---- prefill against token-by-token decoding, portions down to two tokens, the engine's own chunking ----
@pytest.mark.parametrize("f32", [True, False])
def test_portions_and_decoding(tmp_path, f32):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, f32=f32)
    t = toks(cfg, 150)
    ref = O.forward(cfg, w, t, np.float64)
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
    refs = [O.forward(cfg, w, t, np.float64) for t in ts]
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


# ---- a far key among hundreds, where random weights would hide it: one key made to stand out, at and around page borders ----
@pytest.mark.parametrize("where", [0, 31, 32, 33, 95, 200])
def test_far_key_shows(tmp_path, where):
    """Token `where` is the only one of its id and its key row is made large, so queries hundreds of positions later put their weight
    on it in one map: losing that key (or its value) would change the logits far beyond the tolerance."""
    mixer = att(heads=2, kv_heads=1, dim=16, vdim=16, scale=1.0, diff=0.3, rot=None)
    cfg = md.gokinex_config(40, 48, [("attention", mixer, None)], scale=2.0)
    t = toks(cfg, 330, seed=3)
    t[t == 7] = 8
    t[where] = 7

    def sharpen(w):      # coordinate 0 of the mixer's input is positive for token 7 alone; map 1's keys read it, its queries are constant
        w["embed"][:, 0] = -3.0; w["embed"][7, 0] = 3.0
        for n in ("embed.norm", "l0.norm1"):
            w[n][0] = 1.0; w[n + ".b"][0] = 0.0
        w["l0.mix.k"][:16, 0] = 2.0
        for lo in (0, 32):
            w["l0.mix.q"][lo:lo + 16] = 0.0; w["l0.mix.q.b"][lo:lo + 16] = 1.5
    eng, w = build(tmp_path, cfg, max_tokens=400, tweak=sharpen)
    ref = O.forward(cfg, w, t, np.float64)
    t2 = t.copy(); t2[where] = 9
    assert rel(O.forward(cfg, w, t2, np.float64)[-20:], ref[-20:]) > 100 * F32_TOL          # the key matters to the last queries
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [290] + [1] * 40), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [29, 2, 2, 31, 1, 1, 64, 130, 3, 4, 63]), ref) < F32_TOL
    eng.close()


def test_rotation_and_wavelength_scaling_show(tmp_path):
    """The oracle itself tells the frequency rescaling and the pairing apart at these sizes; the engine follows the right one."""
    mixer = att(heads=2, kv_heads=1, dim=16, vdim=16, scale=0.7, rot={"dims": 16, "base": 50.0, "scaling": {"factor": 6.0, "low": 1.0, "high": 5.0, "original": 40}})
    cfg = md.gokinex_config(40, 48, [("attention", mixer, None)], scale=2.0)
    eng, w = build(tmp_path, cfg)
    t = toks(cfg, 200, seed=3)
    ref = O.forward(cfg, w, t, np.float64)
    plain = copy.deepcopy(cfg); del plain["layers"][0]["mixer"]["rot"]["scaling"]
    assert rel(O.forward(plain, w, t, np.float64), ref) > 100 * F32_TOL
    f = O.rot_freqs(mixer["rot"])
    base = O.rot_freqs({"dims": 16, "base": 50.0})
    assert f[0] == base[0] and f[-1] == base[-1] / 6.0 and any(b / 6.0 < a < b for a, b in zip(f, base))      # all three branches
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [150] + [1] * 50), ref) < F32_TOL
    eng.close()


def test_long_prompt_splits_keys_in_decoding(tmp_path):
    """Short portions deal the key pages out to several blocks and merge: same logits as the whole prompt."""
    cfg = md.gokinex_config(40, 48, [("attention", att(heads=3, kv_heads=1, dim=24, vdim=24, scale=0.8), DENSE), ("attention", att(heads=3, kv_heads=1, dim=24, vdim=24, scale=0.8, kv_from=0), None)], scale=2.0)
    eng, w = build(tmp_path, cfg, max_tokens=400)
    t = toks(cfg, 330, seed=6)
    ref = O.forward(cfg, w, t, np.float64)
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [140] + [1] * 60 + [2, 3, 4, 1] * 13), ref) < F32_TOL
    eng.close()


def test_far_tokens_through_the_state(tmp_path):
    """A slow decay carries the first tokens over hundreds of positions: changing token 0 changes the last logits."""
    def slow(w):
        w["l0.mix.dt_bias"] = np.full_like(w["l0.mix.dt_bias"], -5.0)
        w["l0.mix.A_log"] = np.full_like(w["l0.mix.A_log"], -4.0)
    cfg = md.gokinex_config(40, 48, [("mamba2", ssd(heads=2, vdim=16, state=8, groups=1), DENSE)], scale=2.0)
    eng, w = build(tmp_path, cfg, max_tokens=640, tweak=slow)
    t = toks(cfg, 600, seed=5)
    ref = O.forward(cfg, w, t, np.float64)
    t2 = t.copy(); t2[0] = (t2[0] + 1) % cfg["vocab"]
    assert rel(O.forward(cfg, w, t2, np.float64)[-20:], ref[-20:]) > 30 * F32_TOL
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [560] + [1] * 40)[-60:], ref[-60:]) < F32_TOL
    assert rel(in_cuts(eng, t, [70, 2, 200, 3, 64, 261])[-60:], ref[-60:]) < F32_TOL
    eng.close()


def test_scan_over_time_segments_four_columns_per_warp(tmp_path):
    """A long portion of a wide scan: time segments side by side, four value columns per warp; then the same in ragged portions."""
    cfg = md.gokinex_config(40, 64, [("mamba2", ssd(heads=16, vdim=64, state=64, groups=4, conv=4, norm_groups=8), None)], scale=2.0)
    eng, w = build(tmp_path, cfg, max_tokens=400)
    t = toks(cfg, 300, seed=7)
    ref = O.forward(cfg, w, t, np.float64)
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [257, 2, 1, 40]), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [64, 65, 33, 100, 38]), ref) < F32_TOL
    eng.close()


def test_long_decoding(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, max_tokens=700)
    t = toks(cfg, 650, seed=8)
    ref = O.forward(cfg, w, t, np.float64)
    got = in_cuts(eng, t, [3] + [1] * 647)
    assert rel(got, ref) < 2 * F32_TOL
    eng.close()


def test_first_tokens_and_single_token_requests(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg)
    for n in (1, 2, 3, 5):
        t = toks(cfg, n, seed=20 + n)
        ref = O.forward(cfg, w, t, np.float64)
        assert rel(whole(eng, t), ref) < F32_TOL
        assert rel(in_cuts(eng, t, [1] * n), ref) < F32_TOL
    # the pair row of a sequence's first token is the table's last one, whatever came through the slot before
    t = toks(cfg, 9, seed=30)
    ref = O.forward(cfg, w, t, np.float64)
    for _ in range(3):
        assert rel(in_cuts(eng, t, [1, 3, 5]), ref) < F32_TOL
    eng.close()


def test_bf16_close_to_oracle(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, f32=False)
    t = toks(cfg, 120)
    ref = O.forward(cfg, w, t, np.float64)
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
    ref = O.forward(cfg, w, ids[:total - 1], np.float64)
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
    """The device sampler and the repetition penalty on the implicit sequence, whose slot also carries the previous token."""
    cfg = mixed_cfg(vocab=80)
    eng, w = build(tmp_path, cfg)
    prompt = [5, 17, 3, 44]
    ids = np.zeros(32, np.uint32); ids[:4] = prompt
    for pos in range(3):
        eng.next_greedy(ids, pos, 1)
    tok, top6 = eng.next_sampled(ids, 3, 1.0, 0.8, 0.95, 0.01)
    ref = O.forward(cfg, w, prompt, np.float64)[-1]
    assert top6[0] == int(np.argmax(ref)) and tok == top6[0]          # a coin near 0 takes the most probable token
    eng.forward(5, 0); eng.forward(17, 1)                             # position 0 starts over: the pair row is the first token's again
    assert rel(eng.logits()[None, :], O.forward(cfg, w, [5, 17], np.float64)[-1:]) < F32_TOL
    pen = O.forward(cfg, w, [5, 17, 3], np.float64)[-1].copy()
    for i in (5, 17):
        pen[i] = pen[i] / 50.0 if pen[i] > 0 else pen[i] * 50.0
    ids[:3] = [5, 17, 3]
    assert eng.next_greedy(ids, 2, 0, 50.0) == int(np.argmax(pen))
    eng.close()


def test_bad_folders_are_refused(tmp_path):
    cfg = md.gokinex_config(30, 32, [("attention", att(kv_from=0), None)])
    with pytest.raises(E.NB200Error):          # kv_from names itself
        build(tmp_path, cfg, name="a")
    cfg = md.gokinex_config(30, 32, [("mamba2", SSD, None), ("attention", att(kv_from=0), None)])
    with pytest.raises(E.NB200Error):          # kv_from names a layer that is no attention
        build(tmp_path, cfg, name="b")
    cfg = md.gokinex_config(30, 32, [("mamba2", ssd(heads=3, groups=2), None)])
    with pytest.raises(E.NB200Error):          # heads not a multiple of groups
        build(tmp_path, cfg, name="c")


def test_replay_command(tmp_path):
    """bin/trace_run on a Gokinex folder: portions, single tokens, a step that wants nothing, two requests one after the other."""
    cfg = mixed_cfg()
    w = md.gokinex_random(cfg, 2)
    path = md.write_model_dir(str(tmp_path / "m"), cfg, w)
    a, b = toks(cfg, 70, seed=1), toks(cfg, 9, seed=2)
    ra, rb = O.forward(cfg, w, a, np.float64), O.forward(cfg, w, b, np.float64)
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
