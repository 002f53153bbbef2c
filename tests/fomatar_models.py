"""Small Fomatar configurations and random weights for the tests, made here by the tensor naming
rule itself (not from the library's tensor lists), stored in bfloat16 as a model folder."""
import json
import os

import torch


def delta(dim, vdim, heads, kv_heads, conv, mlp=None):
    return {"type": "channel_delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim},
            "mlp": {"ff": mlp, "kind": "dense"} if mlp else None}


def parallel(left, right, mlp=None):
    dim, vdim, heads, kv_heads, window, scale = left
    rdim, rvdim, rheads, cap = right
    return {"type": "parallel",
            "mixer": {"left": {"dim": dim, "vdim": vdim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window},
                               "scale": scale},
                      "right": {"dim": rdim, "vdim": rvdim, "heads": rheads, "gate_cap": cap}},
            "mlp": {"ff": mlp, "kind": "dense"} if mlp else None}


def config(width, vocab, layers, loop=None, bigram=(53, 31, 17), softcap=12.0, eps=1e-5):
    cfg = {"architecture": "Fomatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


# every size differs from every other; q/k heads shared by groups of 3 (attention) and 2 (delta rule); key and
# value sizes differ; a looped stretch of two layers, three passes; layers with and without feed-forward
MIXED = config(64, 97, [
    parallel((24, 40, 6, 2, 9, 0.3), (20, 24, 3, 8.0), mlp=104),
    delta(12, 20, 4, 2, 3),
    delta(16, 8, 2, 1, 2, mlp=72),
    parallel((16, 16, 2, 2, 5, 0.25), (8, 36, 2, 6.0)),
], loop=(1, 3, 3))
# no bigram, no loop, no soft cap; a window longer than a page of the cache, value heads of 70 and 33 channels
# (more than one block of columns in the scans needs > 128: see WIDE), a convolution of one tap
PLAIN = config(72, 131, [
    delta(24, 70, 2, 2, 1, mlp=96),
    parallel((32, 48, 4, 1, 70, 0.18), (40, 33, 2, 10.0), mlp=80),
], bigram=None, softcap=None)
# the stretch that runs twice starts at the first layer; a width that is no multiple of 8 (no tensor-core product)
FROM_START = config(44, 61, [
    parallel((8, 12, 2, 1, 4, 0.35), (12, 8, 2, 5.0)),
    delta(8, 12, 2, 2, 4, mlp=36),
], loop=(0, 2, 2), bigram=(7, 5, 3))
# wide heads: 160 value channels (ten blocks of columns per head in the scans), key size 72; attention heads
# of 64 channels for keys and values alike (in bfloat16 the tensor-core kernel for prompts), 3 query heads per
# kv head, a window of 130 over pages of 64
WIDE = config(96, 83, [
    delta(72, 160, 2, 1, 4),
    parallel((64, 64, 3, 1, 130, 0.125), (72, 140, 1, 15.0), mlp=128),
], loop=None)
# no attention at all (a cache without keys and values), one head, the whole model one looped stretch
DELTA_ONLY = config(48, 50, [delta(16, 24, 1, 1, 3, mlp=64), delta(8, 8, 3, 3, 2)], loop=(0, 2, 2), bigram=(11, 3, 5))
CONFIGS = {"mixed": MIXED, "plain": PLAIN, "from_start": FROM_START, "wide": WIDE, "delta_only": DELTA_ONLY}


def tensor_shapes(cfg, ranks=(8, 16)):
    """name -> (shape, kind of values) by the naming rule."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": ((V, W), "embed"), "final.norm": ((W,), "norm"), "head": ((V, W), "head")}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        out["bigram"] = ((bg["buckets"] + 1, W), "embed")
    if cfg.get("loop"):
        out["loop.step"] = ((cfg["loop"]["times"], W), "embed")
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        out[p + "norm1"] = ((W,), "norm")
        out[p + "shift"] = ((W,), "fraction")
        m = L["mixer"]
        if L["type"] == "channel_delta":
            H, G, D, Dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            q = p + "mix."
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                out[q + n] = ((rows, W), "linear")
                out[q + n + ".conv"] = ((rows, taps), "conv")
            out[q + "b"] = ((H, W), "linear")
            out[q + "A_log"] = ((H,), "log_rate")
            out[q + "dt_bias"] = ((H * D,), "log_rate")
            out[q + "norm"] = ((Dv,), "norm")
            out[q + "a1"] = ((ranks[0], W), "linear")
            out[q + "a2"] = ((H * D, ranks[0]), "low")
            out[q + "g1"] = ((ranks[1], W), "linear")
            out[q + "g2"] = ((H * Dv, ranks[1]), "low")
            out[q + "o"] = ((W, H * Dv), "linear")
        else:
            lf, rt = m["left"], m["right"]
            q = p + "mix.left."
            H, G, D, Dv = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
            out[q + "q"], out[q + "k"], out[q + "v"] = ((H * D, W), "linear"), ((G * D, W), "linear"), ((G * Dv, W), "linear")
            out[q + "g"], out[q + "o"] = ((H * Dv, W), "linear"), ((W, H * Dv), "linear")
            out[q + "q.norm"], out[q + "k.norm"] = ((D,), "norm"), ((D,), "norm")
            out[q + "r1"], out[q + "r2"] = ((H,), "positive"), ((H,), "fraction")
            out[q + "out"] = ((W,), "norm")
            q = p + "mix.right."
            H, D, Dv = rt["heads"], rt["dim"], rt["vdim"]
            out[q + "q"], out[q + "k"] = ((H * D, W), "linear"), ((H * D, W), "linear")
            out[q + "v"], out[q + "g"], out[q + "o"] = ((H * Dv, W), "linear"), ((H * Dv, W), "linear"), ((W, H * Dv), "linear")
            out[q + "norm"] = ((H * Dv,), "norm")
            out[q + "i"], out[q + "i.b"] = ((H, W), "linear"), ((H,), "small")
            out[q + "f"], out[q + "f.b"] = ((H, W), "linear"), ((H,), "forget")
            out[q + "out"] = ((W,), "norm")
        if L.get("mlp"):
            out[p + "norm2"] = ((W,), "norm")
            out[p + "mlp.up"] = ((L["mlp"]["ff"], W), "linear")
            out[p + "mlp.down"] = ((W, L["mlp"]["ff"]), "linear")
    return out


def random_weights(cfg, seed, ranks=(8, 16)):
    """name -> bfloat16 tensor. Values are of the order a trained model has, so that every mechanism
    moves the logits (gates around their working points), with matrices small enough that a stretch of
    layers run three times does not multiply a rounding error of bfloat16 beyond what a test can bound."""
    gen = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg, ranks).items():
        r = torch.randn(shape, generator=gen)
        if kind == "linear":
            t = r * (0.75 / shape[-1] ** 0.5)
        elif kind == "low":
            t = r * (2.0 / shape[-1] ** 0.5)
        elif kind == "embed":
            t = r * 0.8
        elif kind == "head":
            t = r * (4.0 / W ** 0.5)
        elif kind == "norm":
            t = 1.0 + 0.3 * r
        elif kind == "fraction":
            t = (0.3 + 0.25 * r).clamp(0.0, 0.9)
        elif kind == "positive":
            t = (1.5 + 0.8 * r).clamp(0.02, 3.0)
        elif kind == "conv":
            t = 0.2 + 0.6 * r
        elif kind == "log_rate":
            t = -2.5 + 0.9 * r
        elif kind == "small":
            t = 0.5 * r
        elif kind == "forget":
            t = 3.5 + 1.5 * r
        else:
            raise ValueError(kind)
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed, ranks=(8, 16), weights=None):
    from camelid_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    weights = weights if weights is not None else random_weights(cfg, seed, ranks)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    return weights


def as_float64(weights):
    return {n: t.to(torch.float64) for n, t in weights.items()}
