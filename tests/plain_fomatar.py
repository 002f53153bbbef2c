"""A plain, slow implementation of the Fomatar decoder, one function per mechanism, in float64
on the CPU. It runs whole sequences from their first token and keeps no cache: the library's
cuts, batches, pages and states are all compared with this one pass. It shares no code with
the library.

Notation: T tokens, W model width; weights come as a dict name -> float64 tensor, linear
weights [out, in]. ``cfg`` is the config.json dict.
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w None: no weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def logsigmoid(z):
    return -softplus(-z)


def silu(z):
    return z * torch.sigmoid(z)


def bigram_rows(tokens, bigram_cfg):
    """Row of the bigram table for every token: hashed (previous, current), the last row for the first."""
    rows = []
    for t, tok in enumerate(tokens):
        if t == 0:
            rows.append(bigram_cfg["buckets"])
        else:
            rows.append((tokens[t - 1] * bigram_cfg["mul_prev"] + tok * bigram_cfg["mul_cur"]) % bigram_cfg["buckets"])
    return rows


def embedding(tokens, P, cfg):
    x = P["embed"][torch.tensor(tokens)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + P["bigram"][torch.tensor(bigram_rows(list(tokens), bg))]
    return x


def token_shift(h, shift):
    """h_t + (h_(t-1) - h_t) * shift, zeros before the first token."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * shift


def window_scores_core(q, k, v, scale, window, r1, r2):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]: softmax over the last ``window`` keys of
    (q . k) scale - r1 ln(1 + r2 distance)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1)
        for hd in range(H):
            g = hd // (H // G)
            dist = torch.arange(i - lo, -1, -1, dtype=F64)                  # i - j for j = lo..i
            s = (k[lo:i + 1, g] @ q[i, hd]) * scale - r1[hd] * torch.log1p(r2[hd] * dist)
            out[i, hd] = torch.softmax(s, 0) @ v[lo:i + 1, g]
    return out


def window_attention(h, P, p, m, eps):
    """Grouped-query attention without rotation: per-head RMS norm of q and k, a logarithmic
    distance penalty, a sliding window, softmax, an output gate."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ P[p + "q"].T).view(T, H, D), P[p + "q.norm"], eps)
    k = rms_norm((h @ P[p + "k"].T).view(T, G, D), P[p + "k.norm"], eps)
    v = (h @ P[p + "v"].T).view(T, G, Dv)
    out = window_scores_core(q, k, v, m["scale"], m["mask"]["size"], P[p + "r1"], P[p + "r2"])
    gate = torch.sigmoid(h @ P[p + "g"].T)
    return (out.reshape(T, H * Dv) * gate) @ P[p + "o"].T


def matrix_memory_core(q, k, v, gi, gf):
    """q, k [T, H, D] (q already scaled), v [T, H, Dv], log gates gi, gf [T, H] -> S^T q / denominator."""
    T, H, D = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for hd in range(H):
        S = torch.zeros(D, v.shape[2], dtype=F64)
        n = torch.zeros(D, dtype=F64)
        mx = 0.0
        for t in range(T):
            m_new = max(float(gf[t, hd]) + mx, float(gi[t, hd]))
            a = math.exp(float(gf[t, hd]) + mx - m_new)
            b = math.exp(float(gi[t, hd]) - m_new)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = m_new
            den = max(abs(float(n @ q[t, hd])), math.exp(-mx)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
    return out


def matrix_memory(h, P, p, m, eps):
    """The matrix memory with exponential gates and a running maximum that starts at zero."""
    T = h.shape[0]
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ P[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ P[p + "k"].T).view(T, H, D)
    v = (h @ P[p + "v"].T).view(T, H, Dv)
    gi = cap * torch.tanh((h @ P[p + "i"].T + P[p + "i.b"]) / cap)
    gf = logsigmoid(cap * torch.tanh((h @ P[p + "f"].T + P[p + "f.b"]) / cap))
    out = matrix_memory_core(q, k, v, gi, gf)
    out = rms_norm(out, None, eps).reshape(T, H * Dv) * P[p + "norm"]
    return (out * torch.sigmoid(h @ P[p + "g"].T)) @ P[p + "o"].T


def parallel_mixer(h, P, p, m, eps):
    left = window_attention(h, P, p + "left.", m["left"], eps)
    right = matrix_memory(h, P, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, P[p + "left.out"], eps) + rms_norm(right, P[p + "right.out"], eps))


def short_conv(x, w):
    """Causal convolution over time per channel; w [channels, taps], the last tap is the current token's."""
    T, taps = x.shape[0], w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F64), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_core(q, k, v, beta, decay):
    """q, k [T, G, D] unit vectors (q scaled), v [T, H, Dv], beta [T, H], decay [T, H, D] -> S^T q."""
    T, G, D = q.shape
    H, Dv = v.shape[1], v.shape[2]
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(D, Dv, dtype=F64)
        for t in range(T):
            S = decay[t, hd].unsqueeze(1) * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    return out


def channel_delta(h, P, p, m, eps):
    """Gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ P[p + "q"].T, P[p + "q.conv"])).view(T, G, D)
    k = silu(short_conv(h @ P[p + "k"].T, P[p + "k.conv"])).view(T, G, D)
    v = silu(short_conv(h @ P[p + "v"].T, P[p + "v.conv"])).view(T, H, Dv)
    q = unit(q) * D ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ P[p + "b"].T)
    a = (h @ P[p + "a1"].T) @ P[p + "a2"].T + P[p + "dt_bias"]
    decay = torch.exp(-torch.exp(P[p + "A_log"]).view(1, H, 1) * softplus(a).view(T, H, D))
    out = delta_core(q, k, v, beta, decay)
    out = rms_norm(out, P[p + "norm"], eps).reshape(T, H * Dv)
    gate = torch.sigmoid((h @ P[p + "g1"].T) @ P[p + "g2"].T)
    return (out * gate) @ P[p + "o"].T


def dense_ff(h, P, p):
    return gelu_tanh(h @ P[p + "up"].T) @ P[p + "down"].T


def layer(x, i, P, cfg):
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    h = token_shift(rms_norm(x, P[p + "norm1"], eps), P[p + "shift"])
    if L["type"] == "parallel":
        x = x + parallel_mixer(h, P, p + "mix.", L["mixer"], eps)
    elif L["type"] == "channel_delta":
        x = x + channel_delta(h, P, p + "mix.", L["mixer"], eps)
    else:
        raise ValueError(L["type"])
    if L.get("mlp"):
        x = x + dense_ff(rms_norm(x, P[p + "norm2"], eps), P, p + "mlp.")
    return x


def layer_runs(cfg):
    """(layer, pass number or None) in the order they run; the pass number stands at a pass's first layer."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, t if i == loop["start"] else None))
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(tokens, P, cfg, keep_layers=False):
    """Logits [T, vocab] of one sequence from its first token (and the residual stream after every layer run)."""
    x0 = embedding(tokens, P, cfg)
    x = x0
    kept = []
    for i, t in layer_runs(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + P["loop.step"][t]
        x = layer(x, i, P, cfg)
        kept.append(x)
    logits = rms_norm(x, P["final.norm"], cfg["norm"]["eps"]) @ P["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(kept)) if keep_layers else logits
