"""The Zulozen decoder, plainly: float64 numpy, whole sequences, no cache, one function per
mechanism. It shares no code with the library; the GPU tests compare the library with it.

A layer is  x += m * norm_b(mixer(norm_a(x)))  and then  x += m * norm_d(ff(norm_c(x)))  (RMS norms
with a weight; m one number of the model). The mixer is a softmax attention with grouped queries whose
q and k are RMS-normed over the whole projection (all heads at once) before a rotation of interleaved
pairs on the first channels of each head; a query sees the keys of its own block of positions (blocks
of a fixed size counted from the sequence's start) up to itself; the softmax denominator holds one more
term exp(sink[head]); each head's output is scaled by a sigmoid gate (one number per head) computed from
the mixer's input. The feed-forward is dense (squared ReLU, biases) or routed: sigmoid router scores,
the best `top` experts, each fed the row times its score, plus a shared expert fed the row itself.
"""
from __future__ import annotations

import numpy as np


def rms_norm(x, w, eps):
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * np.asarray(w, dtype=np.float64)


def rotate_interleaved(x, positions, rot_dims, base):
    """x [tokens, heads, dim]: channels (2i, 2i+1), i < rot_dims / 2, turned by position * base^(-2i / rot_dims)."""
    out = np.array(x, dtype=np.float64)
    half = rot_dims // 2
    freq = np.float64(base) ** (-2.0 * np.arange(half) / rot_dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]           # [tokens, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = out[..., 0:rot_dims:2].copy(), out[..., 1:rot_dims:2].copy()
    out[..., 0:rot_dims:2] = u * c - v * s
    out[..., 1:rot_dims:2] = v * c + u * s
    return out


def block_mask(n, block):
    """[n, n] True where query i sees key j: j <= i and both in the same block of `block` positions (None: all before)."""
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    m = j <= i
    if block:
        m &= (i // block) == (j // block)
    return m


def sink_softmax(scores, mask, sink):
    """Weights over keys for scores [n, n]; the denominator also holds exp(sink)."""
    s = np.where(mask, scores, -np.inf)
    top = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.where(mask, np.exp(s - top), 0.0)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - top))


def project_qkv(h, t, cfg, eps, positions=None):
    """q [n, H, D], k [n, G, D], v [n, G, Dv] of the normed rows h: q and k normed over all their columns, then rotated."""
    H, G, D, Dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg.get("vdim", cfg["dim"])
    n = h.shape[0]
    q = rms_norm(h @ t["q"].T, t["q.norm"], eps).reshape(n, H, D)
    k = rms_norm(h @ t["k"].T, t["k.norm"], eps).reshape(n, G, D)
    v = (h @ t["v"].T).reshape(n, G, Dv)
    pos = np.arange(n) if positions is None else positions
    rot = cfg.get("rot")
    if rot and rot["dims"]:
        q = rotate_interleaved(q, pos, rot["dims"], rot["base"])
        k = rotate_interleaved(k, pos, rot["dims"], rot["base"])
    return q, k, v


def attend(q, k, v, scale, block, sink, gate=None):
    """[n, H, Dv]: every head's weighted values; gate [n, H] (already a sigmoid) scales them."""
    n, H, _ = q.shape
    G = k.shape[1]
    mask = block_mask(n, block)
    out = np.zeros((n, H, v.shape[2]))
    for hd in range(H):
        g = hd // (H // G)
        w = sink_softmax((q[:, hd] @ k[:, g].T) * scale, mask, float(sink[hd]) if sink is not None else -np.inf)
        out[:, hd] = w @ v[:, g]
        if gate is not None:
            out[:, hd] *= gate[:, hd:hd + 1]
    return out


def attention(h, t, cfg, eps):
    """h [tokens, width] (the normed rows); t: the mixer's tensors by short name; cfg: the mixer's sizes."""
    q, k, v = project_qkv(h, t, cfg, eps)
    gate = 1.0 / (1.0 + np.exp(-(h @ t["g"].T)))                    # [tokens, heads]
    out = attend(q, k, v, cfg["scale"], (cfg.get("mask") or {}).get("size"), t["sink"], gate)
    return out.reshape(h.shape[0], -1) @ t["o"].T


def dense_ff(h, t):
    a = np.maximum(h @ t["up"].T + t["up.b"], 0.0) ** 2
    return a @ t["down"].T + t["down.b"]


def gated_expert(h, t, name):
    g = h @ t[name + ".gate"].T
    return ((g / (1.0 + np.exp(-g))) * (h @ t[name + ".up"].T)) @ t[name + ".down"].T


def routed_ff(h, t, cfg, margins=None):
    """`margins` (a list) receives per row the gap between the last chosen router logit and the best one left out."""
    E, top = cfg["router"]["experts"], cfg["router"]["top"]
    logits = h @ t["router"].T
    score = 1.0 / (1.0 + np.exp(-logits))                            # [tokens, experts]
    out = np.zeros_like(h)
    if margins is not None:
        ordered = -np.sort(-logits, axis=1)
        margins.append(ordered[:, top - 1] - ordered[:, top] if top < E else np.full(h.shape[0], np.inf))
    for r in range(h.shape[0]):
        for e in np.argsort(-score[r], kind="stable")[:top]:
            out[r] += gated_expert(score[r, e] * h[r:r + 1], t, f"e{e}")[0]
    if cfg.get("shared"):
        out += gated_expert(h, t, "shared")
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: np.asarray(v, dtype=np.float64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, probe=None, margins=None):
    """Logits [tokens, vocab] of one sequence; `probe(i, x)` sees the stream after every layer; `margins`
    (a list) collects every routed layer's per-row margins of the choice."""
    eps, m = config["norm"]["eps"], config["residual_mult"]
    x = np.asarray(tensors["embed"], dtype=np.float64)[np.asarray(tokens)]
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        w = {k: np.asarray(tensors[p + k], dtype=np.float64) for k in ("norm1", "norm1b")}
        y = attention(rms_norm(x, w["norm1"], eps), sub(tensors, p + "mix."), L["mixer"], eps)
        x = x + m * rms_norm(y, w["norm1b"], eps)
        if L.get("mlp") is not None:
            t = sub(tensors, p + "mlp.")
            hn = rms_norm(x, tensors[p + "norm2"], eps)
            y = dense_ff(hn, t) if L["mlp"]["kind"] == "dense" else routed_ff(hn, t, L["mlp"], margins)
            x = x + m * rms_norm(y, tensors[p + "norm2b"], eps)
        if probe is not None:
            probe(i, x)
    return rms_norm(x, tensors["final.norm"], eps) @ np.asarray(tensors["head"], dtype=np.float64).T
