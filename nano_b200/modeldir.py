"""Model folders (config.json + model.safetensors) from the Python side: a writer, and random-weight Famudra, Rakarax, Gokinex and Vumunex models for
the benchmarks and tests.  The reader the engine uses is native (csrc/modeldir.cu); nothing here is on the compute path.

A safetensors file is an 8-byte little-endian header length, that many bytes of JSON (name -> dtype, shape, data_offsets) and
the tensor bytes.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict

import numpy as np


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_round(a: np.ndarray) -> np.ndarray:
    """The fp32 values a bfloat16 file would hold."""
    return (to_bf16_bits(a).astype(np.uint32) << 16).view(np.float32).reshape(np.shape(a))


def write_safetensors(path: str, tensors: Dict[str, np.ndarray], bf16: bool = True) -> None:
    header, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        arr = np.asarray(arr)
        if arr.dtype.kind == "i":
            data, dt = np.ascontiguousarray(arr, "<i4").tobytes(), "I32"
        elif bf16:
            data, dt = to_bf16_bits(arr).astype("<u2").tobytes(), "BF16"
        else:
            data, dt = np.ascontiguousarray(arr, "<f4").tobytes(), "F32"
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(data)]}
        blobs.append(data)
        off += len(data)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def write_model_dir(path: str, config: dict, tensors: Dict[str, np.ndarray], bf16: bool = True) -> str:
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    write_safetensors(os.path.join(path, "model.safetensors"), tensors, bf16)
    return path


def famudra_config(vocab: int, width: int, layers, loop=None, eps: float = 1e-5) -> dict:
    """layers: list of ("rglru", {width, blocks, conv}, mlp) / ("latent_attention", {heads, dim, vdim, kv_rank, q_rank, scale}, mlp);
    mlp: None or {"experts": n, "top": k, "ff": f, "shared_ff": s or None}."""
    out = []
    for kind, mixer, mlp in layers:
        m = None
        if mlp:
            m = {"kind": "moe", "router": {"experts": mlp["experts"], "top": mlp["top"]}, "expert": {"ff": mlp["ff"]},
                 "shared": {"ff": mlp["shared_ff"]} if mlp.get("shared_ff") else None}
        out.append({"type": kind, "mixer": dict(mixer), "mlp": m})
    cfg = {"architecture": "Famudra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": out}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def famudra_random(config: dict, seed: int = 0, gain: float = 1.0) -> Dict[str, np.ndarray]:
    """Random weights (bfloat16-representable fp32 arrays) for a Famudra config: projections ~ N(0, gain^2 / fan_in)."""
    rng = np.random.default_rng(seed)
    E, V = config["width"], config["vocab"]

    def lin(o, i, g=1.0):
        return bf16_round((rng.standard_normal((o, i), dtype=np.float32) * (gain * g / np.sqrt(i))).astype(np.float32))

    def vecn(n, lo, hi):
        return bf16_round(rng.uniform(lo, hi, size=n).astype(np.float32))

    t = {"embed": bf16_round(rng.standard_normal((V, E), dtype=np.float32)), "head": lin(V, E), "final.norm": vecn((), 0.8, 1.2)}
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        t[p + "norm1"] = vecn((), 0.8, 1.2)
        t[p + "shift"] = vecn(E, 0.0, 1.0)
        m = L["mixer"]
        if L["type"] == "rglru":
            C, B, K = m["width"], m["blocks"], m["conv"]
            bs = C // B
            t[p + "mix.y"] = lin(C, E); t[p + "mix.y.b"] = vecn(C, -0.2, 0.2)
            t[p + "mix.x"] = lin(C, E); t[p + "mix.x.b"] = vecn(C, -0.2, 0.2)
            t[p + "mix.conv"] = vecn((C, K), -0.6, 0.6); t[p + "mix.conv.b"] = vecn(C, -0.1, 0.1)
            t[p + "mix.ra"] = np.stack([lin(bs, bs) for _ in range(B)]); t[p + "mix.ra.b"] = vecn((B, bs), -0.5, 0.5)
            t[p + "mix.ri"] = np.stack([lin(bs, bs) for _ in range(B)]); t[p + "mix.ri.b"] = vecn((B, bs), -0.5, 0.5)
            t[p + "mix.lam"] = vecn(C, -4.0, 0.5)
            t[p + "mix.o"] = lin(E, C)
        else:
            H, D, VD, R, QR = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"] = lin(QR, E); t[p + "mix.dq.norm"] = vecn(QR, 0.7, 1.3)
            t[p + "mix.uq"] = lin(H * D, QR)
            t[p + "mix.dkv"] = lin(R, E); t[p + "mix.dkv.norm"] = vecn(R, 0.7, 1.3)
            t[p + "mix.uk"] = lin(H * D, R); t[p + "mix.uv"] = lin(H * VD, R)
            t[p + "mix.o"] = lin(E, H * VD)
        f = L.get("mlp")
        if f:
            t[p + "norm2"] = vecn((), 0.8, 1.2)
            t[p + "mlp.router"] = lin(f["router"]["experts"], E, 2.0)
            for e in range(f["router"]["experts"]):
                t[p + f"mlp.e{e}.up"] = lin(f["expert"]["ff"], E); t[p + f"mlp.e{e}.down"] = lin(E, f["expert"]["ff"])
            if f.get("shared"):
                t[p + "mlp.shared.up"] = lin(f["shared"]["ff"], E); t[p + "mlp.shared.down"] = lin(E, f["shared"]["ff"])
    return t


def rakarax_config(vocab: int, width: int, layers, max_positions: int = 512, eps: float = 1e-5) -> dict:
    """layers: list of (type, mixer, ff) or (type, mixer, ff, weights_of).
    type "retention": mixer {heads, dim, vdim, decay: [per head], rot: {dims, base} or None};
    type "parallel": mixer {left: {heads, kv_heads, dim, vdim, conv, scale, softcap, mask: {size} or None}, right: {inner, state,
    dt_rank, conv}, left_scale, right_scale}; ff: width of the dense feed-forward, or None for a layer without one.
    A layer with weights_of = j repeats layer j's entry and has no tensors of its own."""
    out = []
    for ent in layers:
        kind, mixer, ff = ent[:3]
        L = {"type": kind, "mixer": json.loads(json.dumps(mixer)), "mlp": {"kind": "dense", "ff": ff} if ff else None}
        if len(ent) > 3 and ent[3] is not None:
            src = {k: v for k, v in out[int(ent[3])].items() if k != "weights_of"}
            assert src == L, "a layer with weights_of repeats the entry of the layer it names"
            L["weights_of"] = int(ent[3])
        out.append(L)
    return {"architecture": "Rakarax", "vocab": vocab, "width": width, "max_positions": max_positions, "norm": {"eps": eps}, "layers": out}


def rakarax_random(config: dict, seed: int = 0, gain: float = 1.0) -> Dict[str, np.ndarray]:
    """Random weights (bfloat16-representable fp32 arrays) for a Rakarax config: projections ~ N(0, gain^2 / fan_in)."""
    rng = np.random.default_rng(seed)
    E, V = config["width"], config["vocab"]

    def lin(o, i, g=1.0):
        return bf16_round((rng.standard_normal((o, i), dtype=np.float32) * (gain * g / np.sqrt(i))).astype(np.float32))

    def vecn(n, lo, hi):
        return bf16_round(rng.uniform(lo, hi, size=n).astype(np.float32))

    t = {"embed": bf16_round(rng.standard_normal((V, E), dtype=np.float32)),
         "pos": bf16_round(0.5 * rng.standard_normal((config["max_positions"], E), dtype=np.float32)),
         "head": lin(V, E), "final.norm": vecn(E, -0.2, 0.2)}
    for i, L in enumerate(config["layers"]):
        if "weights_of" in L:
            continue
        p = f"l{i}."
        for n in ("norm1", "norm1b"):
            t[p + n] = vecn(E, -0.2, 0.2)
        m = L["mixer"]
        if L["type"] == "retention":
            H, D, VD = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"] = lin(H * D, E, 2.0); t[p + "mix.k"] = lin(H * D, E, 2.0)
            t[p + "mix.v"] = lin(H * VD, E); t[p + "mix.g"] = lin(H * VD, E, 2.0); t[p + "mix.o"] = lin(E, H * VD)
        else:
            a, r = m["left"], m["right"]
            H, G, D = a["heads"], a["kv_heads"], a["dim"]
            t[p + "mix.left.q"] = lin(H * D, E); t[p + "mix.left.k"] = lin(G * D, E)
            t[p + "mix.left.q.conv"] = vecn((H * D, a["conv"]), -0.6, 0.6); t[p + "mix.left.k.conv"] = vecn((G * D, a["conv"]), -0.6, 0.6)
            t[p + "mix.left.talk"] = bf16_round((np.eye(H) + 0.3 * rng.standard_normal((H, H))).astype(np.float32))
            t[p + "mix.left.temp"] = vecn(H, 0.5, 2.0)
            t[p + "mix.left.g"] = lin(H * a["vdim"], E, 2.0); t[p + "mix.left.o"] = lin(E, H * a["vdim"])
            C, N, R = r["inner"], r["state"], r["dt_rank"]
            t[p + "mix.right.in"] = lin(2 * C, E)
            t[p + "mix.right.conv"] = vecn((C, r["conv"]), -0.6, 0.6); t[p + "mix.right.conv.b"] = vecn(C, -0.1, 0.1)
            t[p + "mix.right.x"] = lin(R + 2 * N, C); t[p + "mix.right.dt"] = lin(C, R, 2.0); t[p + "mix.right.dt.b"] = vecn(C, -4.0, -1.0)
            t[p + "mix.right.A_log"] = bf16_round(np.log(rng.uniform(0.5, 8.0, size=(C, N))).astype(np.float32))
            t[p + "mix.right.D"] = vecn(C, 0.5, 1.5); t[p + "mix.right.o"] = lin(E, C)
        f = L.get("mlp")
        if f:
            for n in ("norm2", "norm2b"):
                t[p + n] = vecn(E, -0.2, 0.2)
            t[p + "mlp.up"] = lin(f["ff"], E, 1.5); t[p + "mlp.down"] = lin(E, f["ff"])
            t[p + "mlp.act"] = bf16_round(np.array([0.6, 0.3, 0.15, 0.05], np.float32) * rng.uniform(0.7, 1.3, size=4).astype(np.float32))
    return t


def gokinex_config(vocab: int, width: int, layers, scale: float = 1.0, bigram=None, eps: float = 1e-5) -> dict:
    """layers: list of (type, mixer, mlp).
    type "attention": mixer {heads, kv_heads, dim, vdim, scale, diff, rot: {dims, base, scaling: {factor, low, high, original} or
    absent} or absent, kv_from: j or absent}; type "mamba2": mixer {heads, vdim, state, groups, conv, norm_groups};
    mlp: None, {"kind": "dense", "ff": f} or {"kind": "moe", "router": {"experts": n, "top": k}, "expert": {"ff": f}, "shared": {"ff": s}
    (optional)}.  bigram: {"buckets": b, "mul_prev": p, "mul_cur": c} or None."""
    out = [{"type": kind, "mixer": json.loads(json.dumps(mixer)), "mlp": json.loads(json.dumps(mlp)) if mlp else None} for kind, mixer, mlp in layers]
    emb = {"scale": scale}
    if bigram:
        emb["bigram"] = dict(bigram)
    return {"architecture": "Gokinex", "vocab": vocab, "width": width, "embedding": emb, "norm": {"eps": eps}, "layers": out}


def gokinex_random(config: dict, seed: int = 0, gain: float = 1.0) -> Dict[str, np.ndarray]:
    """Random weights (bfloat16-representable fp32 arrays) for a Gokinex config: projections ~ N(0, gain^2 / fan_in)."""
    rng = np.random.default_rng(seed)
    E, V = config["width"], config["vocab"]

    def lin(o, i, g=1.0):
        return bf16_round((rng.standard_normal((o, i), dtype=np.float32) * (gain * g / np.sqrt(i))).astype(np.float32))

    def vecn(n, lo, hi):
        return bf16_round(rng.uniform(lo, hi, size=n).astype(np.float32))

    t = {}

    def dyt(name, alpha=(0.3, 0.9)):
        t[name] = vecn(E, 0.6, 1.4); t[name + ".b"] = vecn(E, -0.2, 0.2); t[name + ".alpha"] = vecn((), *alpha)

    t["embed"] = bf16_round(rng.standard_normal((V, E), dtype=np.float32))
    bg = config["embedding"].get("bigram")
    if bg:
        t["bigram"] = bf16_round(rng.standard_normal((bg["buckets"] + 1, E), dtype=np.float32))
    dyt("embed.norm", (0.2, 0.6)); dyt("final.norm")
    t["head"] = lin(V, E)
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        dyt(p + "norm1"); dyt(p + "norm1b", (0.5, 1.5))
        m = L["mixer"]
        if L["type"] == "attention":
            H, G, D, VD = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"] = lin(H * 2 * D, E, 2.0); t[p + "mix.q.b"] = vecn(H * 2 * D, -0.3, 0.3)
            if "kv_from" not in m:
                t[p + "mix.k"] = lin(G * 2 * D, E, 2.0); t[p + "mix.k.b"] = vecn(G * 2 * D, -0.3, 0.3)
                t[p + "mix.v"] = lin(G * VD, E); t[p + "mix.v.b"] = vecn(G * VD, -0.3, 0.3)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                t[p + "mix." + n] = bf16_round((rng.standard_normal(D) * 0.35 / np.sqrt(np.sqrt(D))).astype(np.float32))
            t[p + "mix.o"] = lin(E, H * VD); t[p + "mix.o.b"] = vecn(E, -0.2, 0.2)
        else:
            Hn, P, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, XW = Hn * P, Hn * P + 2 * G * N
            t[p + "mix.in"] = lin(2 * inner + 2 * G * N + Hn, E)
            t[p + "mix.conv"] = vecn((XW, K), -0.6, 0.6); t[p + "mix.conv.b"] = vecn(XW, -0.1, 0.1)
            t[p + "mix.dt_bias"] = vecn(Hn, -4.0, 0.5); t[p + "mix.A_log"] = bf16_round(np.log(rng.uniform(0.05, 8.0, size=Hn)).astype(np.float32))
            t[p + "mix.D"] = vecn(Hn, 0.5, 1.5); t[p + "mix.norm"] = vecn(inner, 0.6, 1.4); t[p + "mix.o"] = lin(E, inner)
        f = L.get("mlp")
        if not f:
            continue
        dyt(p + "norm2"); dyt(p + "norm2b", (0.5, 1.5))
        if f["kind"] == "dense":
            t[p + "mlp.gate"] = lin(f["ff"], E, 1.5); t[p + "mlp.up"] = lin(f["ff"], E); t[p + "mlp.down"] = lin(E, f["ff"])
        else:
            t[p + "mlp.router"] = lin(f["router"]["experts"], E, 2.0)
            for e in range(f["router"]["experts"]):
                q = p + f"mlp.e{e}."
                t[q + "gate"] = lin(f["expert"]["ff"], E, 1.5); t[q + "up"] = lin(f["expert"]["ff"], E); t[q + "down"] = lin(E, f["expert"]["ff"])
            if f.get("shared"):
                q = p + "mlp.shared."
                t[q + "gate"] = lin(f["shared"]["ff"], E, 1.5); t[q + "up"] = lin(f["shared"]["ff"], E); t[q + "down"] = lin(E, f["shared"]["ff"])
                t[q + "sg"] = lin(1, E, 2.0)
    return t


def vumunex_config(vocab: int, width: int, layers, streams=3, residual_mult=0.5, scale: float = 1.0, loop=None, eps: float = 1e-5) -> dict:
    """layers: list of (type, mixer, mlp).
    type "latent_attention": mixer {heads, dim, vdim, kv_rank, scale, mask: {size}}; type "latent_attention_2": mixer {heads, dim,
    rot_dim, vdim, kv_rank, scale, rot: {dims, base}}; mlp: None, {"kind": "dense", "ff": f} or {"kind": "moe", "router": {"experts": n,
    "top": k}, "expert": {"ff": f, "limit": l}, "shared": {"ff": s, "limit": l} (optional)}.  streams None: one plain residual stream
    (the key is left out, and vumunex_random writes no connection tensors)."""
    out = [{"type": kind, "mixer": json.loads(json.dumps(mixer)), "mlp": json.loads(json.dumps(mlp)) if mlp else None} for kind, mixer, mlp in layers]
    cfg = {"architecture": "Vumunex", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
           "residual_mult": residual_mult, "layers": out}
    if streams is not None:
        cfg["streams"] = int(streams)
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def vumunex_random(config: dict, seed: int = 0, gain: float = 1.0, layer_scale: bool = True) -> Dict[str, np.ndarray]:
    """Random weights (bfloat16-representable fp32 arrays) for a Vumunex config: projections ~ N(0, gain^2 / fan_in)."""
    rng = np.random.default_rng(seed)
    E, V = config["width"], config["vocab"]
    S = config.get("streams")

    def lin(o, i, g=1.0):
        return bf16_round((rng.standard_normal((o, i), dtype=np.float32) * (gain * g / np.sqrt(i))).astype(np.float32))

    def vecn(n, lo, hi):
        return bf16_round(rng.uniform(lo, hi, size=n).astype(np.float32))

    t = {"embed": bf16_round(rng.standard_normal((V, E), dtype=np.float32)), "head": lin(V, E), "final.norm": vecn(E, 0.7, 1.3)}
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        H, D, VD, R, RD = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m.get("rot_dim", 0)
        t[p + "norm1"] = vecn(E, 0.7, 1.3)
        t[p + "mix.q"] = lin(H * (D + RD), E, 2.0)
        t[p + "mix.dkv"] = lin(R + RD, E, 2.0); t[p + "mix.dkv.norm"] = vecn(R, 0.7, 1.3)
        t[p + "mix.uk"] = lin(H * D, R, 2.0); t[p + "mix.uv"] = lin(H * VD, R)
        if L["type"] == "latent_attention":
            t[p + "mix.sink"] = vecn(H, -1.0, 2.0)
        t[p + "mix.g"] = lin(H * VD, E, 2.0); t[p + "mix.o"] = lin(E, H * VD)
        subs = [1]
        f = L.get("mlp")
        if f:
            subs.append(2)
            t[p + "norm2"] = vecn(E, 0.7, 1.3)
            if f["kind"] == "dense":
                t[p + "mlp.up"] = lin(f["ff"], E, 1.5); t[p + "mlp.down"] = lin(E, f["ff"])
            else:
                t[p + "mlp.router"] = lin(f["router"]["experts"], E, 3.0)
                for e in range(f["router"]["experts"]):
                    q = p + f"mlp.e{e}."
                    t[q + "gate"] = lin(f["expert"]["ff"], E, 2.0); t[q + "up"] = lin(f["expert"]["ff"], E, 2.0); t[q + "down"] = lin(E, f["expert"]["ff"])
                if f.get("shared"):
                    q = p + "mlp.shared."
                    t[q + "gate"] = lin(f["shared"]["ff"], E, 2.0); t[q + "up"] = lin(f["shared"]["ff"], E, 2.0); t[q + "down"] = lin(E, f["shared"]["ff"])
        for q in subs:
            if layer_scale:
                t[p + f"ls{q}"] = vecn(E, 0.5, 1.5)
            if S is not None:
                t[p + f"hc{q}.in"] = vecn(S, 0.2, 0.6); t[p + f"hc{q}.out"] = vecn(S, 0.5, 1.5)
                t[p + f"hc{q}.mix"] = bf16_round((np.eye(S) * 0.9 + 0.1 * rng.standard_normal((S, S))).astype(np.float32))
    return t
