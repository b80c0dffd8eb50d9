"""Model-folder reader and family registry, as far as they go without a GPU."""
import json
import os

import numpy as np
import pytest

from nano_b200 import engine as E, modeldir as md


def make(tmp_path, cfg, tensors=None):
    return md.write_model_dir(str(tmp_path / "m"), cfg, tensors if tensors is not None else {"embed": np.zeros((4, 8), np.float32)})


def test_unknown_architecture_is_named(tmp_path):
    p = make(tmp_path, {"architecture": "Nonesuch"})
    with pytest.raises(E.NB200Error, match="unknown architecture \"Nonesuch\""):
        E.Engine(p, 16)


def test_broken_folders_are_reported(tmp_path):
    with pytest.raises(E.NB200Error, match="cannot read"):
        E.Engine(str(tmp_path), 16)
    p = make(tmp_path, {"architecture": "Famudra"})
    open(os.path.join(p, "config.json"), "w").write('{"architecture": ')
    with pytest.raises(E.NB200Error, match="config.json"):
        E.Engine(p, 16)
    open(os.path.join(p, "config.json"), "w").write(json.dumps({"architecture": "Famudra"}))
    with open(os.path.join(p, "model.safetensors"), "r+b") as f:
        f.write((1 << 40).to_bytes(8, "little"))
    with pytest.raises(E.NB200Error, match="header length"):
        E.Engine(p, 16)


@pytest.mark.skipif(E.device_count() > 0, reason="box has a GPU")
def test_no_cpu_fallback_for_model_folders(tmp_path):
    cfg = md.famudra_config(16, 8, [("rglru", {"width": 8, "blocks": 1, "conv": 2}, None)])
    p = md.write_model_dir(str(tmp_path / "f"), cfg, md.famudra_random(cfg))
    with pytest.raises(E.NB200Error, match="no CUDA device"):
        E.Engine(p, 16)


def test_bf16_writer_rounds_to_nearest_even():
    a = np.array([1.0, 1.00390625, 1.01171875, -3.1415927, 0.0], np.float32)     # 1 + 2^-8 is a tie: even mantissa wins
    r = md.bf16_round(a)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.015625) and abs(r[3] + 3.140625) < 1e-6


@pytest.mark.skipif(E.device_count() > 0, reason="box has a GPU")
def test_rakarax_folder_reaches_the_layered_family(tmp_path):
    ret = {"heads": 1, "dim": 8, "vdim": 8, "decay": [0.9], "rot": {"dims": 4, "base": 100.0}}
    cfg = md.rakarax_config(16, 8, [("retention", ret, 12), ("retention", ret, 12, 0)], max_positions=32)
    w = md.rakarax_random(cfg)
    assert not any(k.startswith("l1.") for k in w)            # a layer with weights_of has no tensors of its own
    p = md.write_model_dir(str(tmp_path / "r"), cfg, w)
    with pytest.raises(E.NB200Error, match="no CUDA device"):
        E.Engine(p, 16)


def test_rakarax_oracle_is_causal_and_windowed():
    """The plain restatement itself: a prefix gives the same logits, and a token outside every window, decay 0 and a scan that
    forgets at once leaves no trace."""
    from rakarax_oracle import forward
    left = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 2, "scale": 0.4, "softcap": 10.0, "mask": {"size": 3}}
    right = {"inner": 12, "state": 3, "dt_rank": 2, "conv": 2}
    cfg = md.rakarax_config(20, 16, [("parallel", {"left": left, "right": right, "left_scale": 1.0, "right_scale": 0.0}, 8)], max_positions=32)
    w = md.rakarax_random(cfg, 3)
    t = np.random.default_rng(0).integers(0, 20, 24)
    full = forward(cfg, w, t)
    assert np.allclose(forward(cfg, w, t[:10]), full[:10], atol=1e-12)
    t2 = t.copy(); t2[5] = (t2[5] + 1) % 20
    other = forward(cfg, w, t2)
    # window 3 and two taps: position 5 reaches positions 5 .. 5 + 2 + 1 through the attention, not beyond
    assert np.abs(other[5] - full[5]).max() > 1e-6 and np.allclose(other[9:], full[9:], atol=1e-12)


GOK_ATT = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.4, "diff": 0.3, "rot": {"dims": 4, "base": 100.0}}
GOK_SSD = {"heads": 2, "vdim": 4, "state": 3, "groups": 1, "conv": 2, "norm_groups": 1}


@pytest.mark.skipif(E.device_count() > 0, reason="box has a GPU")
def test_gokinex_folder_reaches_the_layered_family(tmp_path):
    cfg = md.gokinex_config(16, 8, [("attention", GOK_ATT, {"kind": "dense", "ff": 12}), ("attention", dict(GOK_ATT, kv_from=0), None)], bigram={"buckets": 5, "mul_prev": 3, "mul_cur": 2})
    w = md.gokinex_random(cfg)
    assert "l0.mix.k" in w and "l1.mix.q" in w and "l1.mix.k" not in w and "l1.mix.v" not in w      # a layer with kv_from has no key/value projections
    assert w["bigram"].shape == (6, 8)                                                            # one more row, for the first token
    p = md.write_model_dir(str(tmp_path / "g"), cfg, w)
    with pytest.raises(E.NB200Error, match="no CUDA device"):
        E.Engine(p, 16)


def test_gokinex_oracle_is_causal_and_reads_what_it_should():
    """The plain restatement itself: a prefix gives the same logits; the pair table sees the previous token and only that one; a
    scan with a fast decay forgets; lambda 0 with equal maps leaves the first map alone."""
    import gokinex_oracle as O
    cfg = md.gokinex_config(20, 16, [("mamba2", GOK_SSD, None), ("attention", GOK_ATT, {"kind": "moe", "router": {"experts": 3, "top": 1}, "expert": {"ff": 6}, "shared": {"ff": 4}})],
                            scale=2.0, bigram={"buckets": 7, "mul_prev": 3, "mul_cur": 2})
    w = md.gokinex_random(cfg, 3)
    t = np.random.default_rng(0).integers(0, 20, 24)
    full = O.forward(cfg, w, t)
    assert np.allclose(O.forward(cfg, w, t[:10]), full[:10], atol=1e-12)
    tt = {k: v.astype(np.float64) for k, v in w.items()}
    e = O.embed(cfg, tt, t)
    t2 = t.copy(); t2[5] = (t2[5] + 1) % 20
    e2 = O.embed(cfg, tt, t2)
    changed = np.abs(e2 - e).max(-1) > 0
    assert changed[5] and changed[6] and not changed[:5].any() and not changed[7:].any()
    assert np.allclose(O.embed(cfg, tt, t[3:])[0], O.dyt(tt["embed"][t[3]] * 2.0 + tt["bigram"][7], tt, "embed.norm"))      # a first token takes the last row
    # interleaved pairs: rotating by position p equals a complex multiplication of (x[2i] + i x[2i+1])
    u = np.random.default_rng(1).standard_normal((3, 2, 8))
    r = O.rotate(u, {"dims": 4, "base": 100.0}, [0, 1, 5])
    z = (u[2, 1, 2] + 1j * u[2, 1, 3]) * np.exp(1j * 5 * 100.0 ** (-2.0 / 4))
    assert np.allclose([r[2, 1, 2], r[2, 1, 3]], [z.real, z.imag]) and np.array_equal(r[..., 4:], u[..., 4:]) and np.allclose(r[0], u[0])


VUM_WIN = {"heads": 2, "dim": 8, "vdim": 6, "kv_rank": 10, "scale": 0.4, "mask": {"size": 3}}
VUM_ROT = {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 8, "kv_rank": 10, "scale": 0.4, "rot": {"dims": 4, "base": 100.0}}
VUM_MOE = {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 6, "limit": 0.8}, "shared": {"ff": 4, "limit": 0.5}}


@pytest.mark.skipif(E.device_count() > 0, reason="box has a GPU")
def test_vumunex_folder_reaches_the_layered_family(tmp_path):
    cfg = md.vumunex_config(16, 8, [("latent_attention", VUM_WIN, {"kind": "dense", "ff": 12}), ("latent_attention_2", VUM_ROT, VUM_MOE)], streams=2, loop=(0, 1, 2))
    w = md.vumunex_random(cfg)
    assert w["l0.hc1.mix"].shape == (2, 2) and "l0.mix.sink" in w and "l1.mix.sink" not in w and w["l1.mix.dkv"].shape == (14, 8)
    p = md.write_model_dir(str(tmp_path / "v"), cfg, w)
    with pytest.raises(E.NB200Error, match="no CUDA device"):
        E.Engine(p, 16)


def test_vumunex_oracle_is_causal_windowed_and_routed():
    """The plain restatement itself: a prefix gives the same logits; a token outside the window leaves no trace; the sink takes weight
    away; the router's weights are the chosen scores over their sum; with one stream and unit connections the update is the plain
    pre-norm residual."""
    import vumunex_oracle as O
    cfg = md.vumunex_config(20, 16, [("latent_attention", VUM_WIN, None)], streams=None, residual_mult=0.5)
    w = md.vumunex_random(cfg, 3)
    t = np.random.default_rng(0).integers(0, 20, 24)
    full = O.forward(cfg, w, t)
    assert np.allclose(O.forward(cfg, w, t[:10]), full[:10], atol=1e-12)
    t2 = t.copy(); t2[5] = (t2[5] + 1) % 20
    other = O.forward(cfg, w, t2)
    assert np.abs(other[7] - full[7]).max() > 1e-6 and np.allclose(other[8:], full[8:], atol=1e-12)      # window 3: positions 5, 6, 7 see token 5
    tt = {k: np.asarray(v, np.float64) for k, v in w.items()}
    x = tt["embed"][t]
    h = O.layer_norm(x, tt["l0.norm1"], 1e-5)
    assert np.allclose(h.mean(-1) / tt["l0.norm1"].mean(), 0.0, atol=1.0)      # the mean is taken off before the gain
    y = O.latent_attention(VUM_WIN, tt, "l0.mix.", h, 1e-5) * tt["l0.ls1"]
    res = []
    O.forward(cfg, w, t, res)
    assert np.allclose(res[0], x + 0.5 * y, atol=1e-12)
    hot = dict(tt); hot["l0.mix.sink"] = tt["l0.mix.sink"] + 50.0
    assert np.abs(O.latent_attention(VUM_WIN, hot, "l0.mix.", h, 1e-5)).max() < 1e-12 * np.abs(y).max() + 1e-15
    f = {"router": {"experts": 5, "top": 2}}
    tr = {"r.router": np.random.default_rng(1).standard_normal((5, 16))}
    idx, wt = O.router(f, tr, "r.", h)
    z = h @ tr["r.router"].T
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    assert np.array_equal(idx[:, 0], s.argmax(-1)) and np.allclose(wt.sum(-1), 1.0)
    assert np.allclose(wt[:, 0], s.max(-1) / np.take_along_axis(s, idx, -1).sum(-1))
    g = np.array([[3.0, -3.0]])
    e = O.expert({"e.gate": np.eye(2), "e.up": np.eye(2), "e.down": np.eye(2)}, "e.", g, 1.0)
    assert np.allclose(e, [[1.0 * O.sigmoid(1.702) * 2.0, -3.0 * O.sigmoid(-3.0 * 1.702) * 0.0]])      # the gate is capped from above only, the other branch on both sides
