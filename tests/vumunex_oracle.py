"""A plain, slow restatement of the Vumunex design in numpy (float64), one function per mechanism.  It shares no code with the engine:
it is what the engine's kernels are held against in tests/test_gpu_vumunex.py.

Vumunex: a decoder over `streams` copies of a residual stream (hyper-connections).  The token row is multiplied by a fixed scale and
copied into every stream.  A sublayer (mixer, then feed-forward) reads  u = sum_s in[s] x_s,  runs on a bias-free layer norm of u and
writes back  x_t <- sum_s mix[s, t] x_s + m * out[t] * (ls * y)  with a per-channel layer scale ls and one multiplier m for the whole
model.  Mixers are latent attentions with an output gate: keys and values are up-projections of one RMS-normed latent row per token;
"latent_attention" has no positions, a sliding window and a softmax whose denominator holds one more learned term per head (a sink);
"latent_attention_2" carries a rotated part beside the latent (one rotated key part for all heads), is causal and uses the ordinary
softmax.  Feed-forwards: dense with the exact gelu, or a mixture of clamped gated experts chosen by their softmax scores plus a shared
expert.  A span of layers may run several times with the same weights, every pass with a cache of its own.
"""
import math

import numpy as np


def layer_norm(u, w, eps):
    """bias-free layer norm: (u - mean) / sqrt(mean of squared deviations + eps) * w"""
    c = u - u.mean(-1, keepdims=True)
    return c / np.sqrt((c ** 2).mean(-1, keepdims=True) + eps) * w


def rms_norm(u, w, eps):
    return u / np.sqrt((u ** 2).mean(-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def rotate_pairs(u, rot, positions):
    """u [T, ..., n]: coordinates (2i, 2i+1), i < dims/2, turn by the angle positions * base^(-2i/dims); the rest pass"""
    dims = int(rot["dims"])
    out = u.copy()
    for i in range(dims // 2):
        a = positions * float(rot["base"]) ** (-2.0 * i / dims)
        shape = (len(positions),) + (1,) * (u.ndim - 2)
        c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
        p, q = u[..., 2 * i], u[..., 2 * i + 1]
        out[..., 2 * i] = p * c - q * s
        out[..., 2 * i + 1] = q * c + p * s
    return out


def latent_attention(m, t, p, h, eps):
    """h [T, E] from position 0.  m: the mixer's config entry; p: tensor prefix '<layer>.mix.'.
    Covers both kinds: a rotated part when m has rot_dim, a window when it has mask, a sink when the tensor is there."""
    T = h.shape[0]
    H, D, VD, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    RD = int(m.get("rot_dim", 0))
    pos = np.arange(T, dtype=np.float64)
    q = (h @ t[p + "q"].T).reshape(T, H, D + RD)
    z = h @ t[p + "dkv"].T
    c = rms_norm(z[:, :R], t[p + "dkv.norm"], eps)
    k = (c @ t[p + "uk"].T).reshape(T, H, D)
    v = (c @ t[p + "uv"].T).reshape(T, H, VD)
    score = np.einsum("ihd,jhd->hij", q[:, :, :D], k)
    if RD:
        qr = rotate_pairs(q[:, :, D:], m["rot"], pos)
        kr = rotate_pairs(z[:, R:R + RD], m["rot"], pos)
        score = score + np.einsum("ihd,jd->hij", qr, kr)
    score = score * m["scale"]
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = j <= i
    if m.get("mask"):
        seen &= (i - j) < int(m["mask"]["size"])
    score = np.where(seen[None], score, -np.inf)
    mx = score.max(-1, keepdims=True)
    if (p + "sink") in t:
        mx = np.maximum(mx, t[p + "sink"].reshape(H, 1, 1))
    w = np.exp(score - mx)
    den = w.sum(-1, keepdims=True)
    if (p + "sink") in t:
        den = den + np.exp(t[p + "sink"].reshape(H, 1, 1) - mx)
    w = w / den
    o = np.einsum("hij,jhd->ihd", w, v).reshape(T, H * VD)
    o = o * sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T


def dense_ff(t, p, h):
    return gelu_erf(h @ t[p + "up"].T) @ t[p + "down"].T


def expert(t, p, h, limit):
    g = np.minimum(h @ t[p + "gate"].T, limit)
    u = np.clip(h @ t[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ t[p + "down"].T


def router(f, t, p, h):
    """-> chosen experts [T, top] and their weights (scores over ALL experts, renormalised over the chosen)"""
    z = h @ t[p + "router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    s = s / s.sum(-1, keepdims=True)
    top = f["router"]["top"]
    idx = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    ws = np.take_along_axis(s, idx, -1)
    return idx, ws / (ws.sum(-1, keepdims=True) + 1e-20)


def moe_ff(f, t, p, h):
    idx, w = router(f, t, p, h)
    out = np.zeros((h.shape[0], t[p + "e0.down"].shape[0]))
    for i in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[i, j])
            out[i] += w[i, j] * expert(t, p + f"e{e}.", h[i:i + 1], f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + expert(t, p + "shared.", h, f["shared"]["limit"])
    return out


def run_order(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def sublayer_update(cfg, t, p, q, xs, fn):
    """one sublayer on the streams xs [S, T, E]: q = 1 (mixer) or 2 (feed-forward); fn maps the normed input to the output"""
    m = float(cfg.get("residual_mult", 1.0))
    eps = cfg["norm"]["eps"]
    S = xs.shape[0]
    hc = p + f"hc{q}."
    has = (hc + "in") in t
    w_in = t[hc + "in"] if has else np.ones(S)
    w_out = t[hc + "out"] if has else np.ones(S)
    w_mix = t[hc + "mix"] if has else np.eye(S)
    u = np.einsum("s,ste->te", w_in, xs)
    y = fn(layer_norm(u, t[p + f"norm{q}"], eps))
    if (p + f"ls{q}") in t:
        y = y * t[p + f"ls{q}"]
    return np.einsum("sr,ste->rte", w_mix, xs) + m * w_out[:, None, None] * y[None]


def forward(cfg, tensors, tokens, residuals=None):
    """tokens of one sequence from position 0 -> logits [T, vocab]; residuals (a list) receives the sum of the streams after every layer run"""
    t = {k: np.asarray(v, np.float64) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    S = int(cfg.get("streams", 1))
    x = t["embed"][np.asarray(tokens)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    xs = np.repeat(x[None], S, 0)
    for li in run_order(cfg):
        L = cfg["layers"][li]
        p = f"l{li}."
        xs = sublayer_update(cfg, t, p, 1, xs, lambda h: latent_attention(L["mixer"], t, p + "mix.", h, eps))
        f = L.get("mlp")
        if f:
            if f["kind"] == "dense":
                xs = sublayer_update(cfg, t, p, 2, xs, lambda h: dense_ff(t, p + "mlp.", h))
            else:
                xs = sublayer_update(cfg, t, p, 2, xs, lambda h: moe_ff(f, t, p + "mlp.", h))
        if residuals is not None:
            residuals.append(xs.sum(0))
    return layer_norm(xs.sum(0), t["final.norm"], eps) @ t["head"].T
