"""A plain, slow restatement of the Gokinex design in numpy, one function per mechanism.  It shares no code with the engine: it is
what the engine's kernels are held against in tests/test_gpu_gokinex.py.

Gokinex: a decoder over a residual stream x.  The token row (times a fixed scale) plus a hashed row for the (previous, current)
token pair passes a Dynamic-Tanh norm; every layer is  x += post(mixer(pre(x)))  and then, where it has a feed-forward,
x += post2(ff(pre2(x)))  with Dynamic-Tanh norms  dyt(u) = tanh(alpha u) * w + b  on both sides of each sublayer.  Mixers:
"attention" (grouped-query differential attention: two softmax maps per head over shared values, combined with a learned
weight, per-head unit RMS; rotary positions on part of each map, interleaved pairs, frequencies rescaled by wavelength; a layer
may read another layer's keys and values) and "mamba2" (state-space duality: a scalar decay per head and token, an N x P state
per head, a short causal convolution in front, a gated, group-normed output).  Feed-forwards: dense gated gelu, or a mixture of
silu experts chosen by sigmoid scores that scale the expert's INPUT, plus an always-on shared expert behind a sigmoid gate.
"""
import math

import numpy as np


def dyt(u, t, name):
    """Dynamic Tanh: elementwise, nothing is averaged."""
    return np.tanh(float(t[name + ".alpha"]) * u) * t[name] + t[name + ".b"]


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def unit_rms(u, eps):
    return u / np.sqrt((u ** 2).mean(-1, keepdims=True) + eps)


def embed(cfg, t, tokens):
    """token row x scale + pair row; the first token of a sequence takes the table's last row"""
    e = cfg["embedding"]
    x = t["embed"][tokens] * e["scale"]
    bg = e.get("bigram")
    if bg:
        rows = np.empty(len(tokens), np.int64)
        for i, tok in enumerate(tokens):
            rows[i] = bg["buckets"] if i == 0 else (int(tokens[i - 1]) * bg["mul_prev"] + int(tok) * bg["mul_cur"]) % bg["buckets"]
        x = x + t["bigram"][rows]
    return dyt(x, t, "embed.norm")


def rot_freqs(rot):
    """f_i = base^(-2i/dims), then rescaled by wavelength: short waves stay, long waves are slowed by `factor`, a linear blend between"""
    dims = rot["dims"]
    f = np.array([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], np.float64)
    sc = rot.get("scaling")
    if sc:
        out = f.copy()
        for i, fi in enumerate(f):
            wave = 2.0 * math.pi / fi
            if wave < sc["original"] / sc["high"]:
                continue
            if wave > sc["original"] / sc["low"]:
                out[i] = fi / sc["factor"]
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out[i] = (1.0 - s) * fi / sc["factor"] + s * fi
        f = out
    return f


def rotate(u, rot, positions):
    """u [T, ..., dim]: coordinates (2i, 2i+1), i < dims/2, turn by positions * f_i; the rest pass"""
    if not rot or not rot.get("dims"):
        return u
    dims = rot["dims"]
    ang = np.asarray(positions, np.float64)[:, None] * rot_freqs(rot)[None, :]          # [T, dims/2]
    shape = (len(positions),) + (1,) * (u.ndim - 2) + (dims // 2,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    out = u.copy()
    a, b = u[..., 0:dims:2], u[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def attention_kv(m, t, p, h):
    """keys (rotated, as a cache would hold them) [T, G, 2, dim] and values [T, G, vdim] of an attention layer"""
    T = h.shape[0]
    G, D, VD = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ t[p + "k"].T + t[p + "k.b"]).reshape(T, G, 2, D)
    v = (h @ t[p + "v"].T + t[p + "v.b"]).reshape(T, G, VD)
    return rotate(k, m.get("rot"), np.arange(T)), v


def attention(m, t, p, h, kv, eps):
    """differential attention: o = softmax(q1 k1) v - lambda softmax(q2 k2) v per head, unit RMS over the head, times (1 - diff)"""
    T = h.shape[0]
    H, G, D, VD = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate((h @ t[p + "q"].T + t[p + "q.b"]).reshape(T, H, 2, D), m.get("rot"), np.arange(T))
    k, v = kv
    lam = math.exp(float((t[p + "lq1"] * t[p + "lk1"]).sum())) - math.exp(float((t[p + "lq2"] * t[p + "lk2"]).sum())) + m["diff"]
    out = np.zeros((T, H, VD), h.dtype)
    causal = np.tril(np.ones((T, T), bool))
    for hd in range(H):
        g = hd // (H // G)
        maps = []
        for which in range(2):
            s = (q[:, hd, which] @ k[:, g, which].T) * m["scale"]
            s = np.where(causal, s, -np.inf)
            w = np.exp(s - s.max(-1, keepdims=True))
            maps.append((w / w.sum(-1, keepdims=True)) @ v[:, g])
        out[:, hd] = unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"])
    return out.reshape(T, H * VD) @ t[p + "o"].T + t[p + "o.b"]


def mamba2(m, t, p, h, eps):
    """in-projection [z | x | B | C | dt]; causal convolution + silu over [x | B | C]; per head S <- exp(-exp(A_log) dt) S + dt B x^T,
    y = S^T C + D x; y silu(z), unit RMS in norm_groups parts, gain, out-projection"""
    T = h.shape[0]
    Hn, P, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = Hn * P
    u = h @ t[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    pad = np.concatenate([np.zeros((K - 1, xbc.shape[1]), u.dtype), xbc])
    conv = np.zeros_like(xbc)
    for j in range(K):          # the last tap meets the current token
        conv += pad[j:j + T] * t[p + "conv"][:, j]
    xbc = silu(conv + t[p + "conv.b"])
    x, B, C = xbc[:, :inner].reshape(T, Hn, P), xbc[:, inner:inner + G * N].reshape(T, G, N), xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + t[p + "dt_bias"])
    y = np.zeros((T, Hn, P), u.dtype)
    for hd in range(Hn):
        g = hd // (Hn // G)
        S = np.zeros((N, P), u.dtype)
        rate = math.exp(float(t[p + "A_log"][hd]))
        for i in range(T):
            S = math.exp(-rate * dt[i, hd]) * S + dt[i, hd] * np.outer(B[i, g], x[i, hd])
            y[i, hd] = S.T @ C[i, g] + t[p + "D"][hd] * x[i, hd]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = unit_rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * t[p + "norm"]
    return y @ t[p + "o"].T


def gated(t, p, h, act):
    return (act(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def dense_ff(f, t, p, h):
    return gated(t, p, h, gelu_tanh)


def moe_ff(f, t, p, h, chosen=None):
    """sigmoid scores; the `top` largest choose the experts; a score scales the expert's input; shared expert behind a sigmoid gate"""
    NE, top = f["router"]["experts"], f["router"]["top"]
    s = sigmoid(h @ t[p + "router"].T)
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        order = sorted(range(NE), key=lambda e: (-s[i, e], e))[:top]
        if chosen is not None:
            chosen.append(order)
        for e in order:
            out[i] += gated(t, p + "e%d." % e, s[i, e] * h[i:i + 1], silu)[0]
    if f.get("shared"):
        out = out + gated(t, p + "shared.", h, silu) * sigmoid(h @ t[p + "shared.sg"].T)
    return out


def forward(cfg, tensors, tokens, dtype=np.float64, trace=None):
    """logits [T, vocab] of one sequence run whole; trace (a list) receives the residual stream after every layer"""
    t = {k: np.asarray(v).astype(dtype) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    tokens = np.asarray(tokens, np.int64)
    x = embed(cfg, t, tokens)
    kvs = {}
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        m = L["mixer"]
        h = dyt(x, t, p + "norm1")
        if L["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kvs[i] = attention_kv(m, t, p + "mix.", h)
                src = i
            d = attention(m, t, p + "mix.", h, kvs[src], eps)
        elif L["type"] == "mamba2":
            d = mamba2(m, t, p + "mix.", h, eps)
        else:
            raise ValueError(L["type"])
        x = x + dyt(d, t, p + "norm1b")
        f = L.get("mlp")
        if f:
            h = dyt(x, t, p + "norm2")
            d = dense_ff(f, t, p + "mlp.", h) if f["kind"] == "dense" else moe_ff(f, t, p + "mlp.", h)
            x = x + dyt(d, t, p + "norm2b")
        if trace is not None:
            trace.append(x.copy())
    return dyt(x, t, "final.norm") @ t["head"].T
