"""Small Zulozen configurations and random weights for the tests, made here by the tensor naming
rule itself (not from the library's tensor lists), stored in bfloat16 as a model folder."""
import json
import os

import torch


def attn(dim, vdim, heads, kv_heads, block, rot, scale, base=10000.0):
    m = {"dim": dim, "vdim": vdim, "heads": heads, "kv_heads": kv_heads, "scale": scale}
    if block:
        m["mask"] = {"size": block}
    if rot is not None:
        m["rot"] = {"dims": rot, "base": base}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp=None):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def config(width, vocab, layers, mult=0.4, eps=1e-5):
    return {"architecture": "Zulozen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}


# every size differs from every other: three query heads to a kv head, values wider than keys, blocks of 9
# positions; one query head per kv head with the whole head rotated, blocks of 70 over pages of 64; a layer
# without feed-forward and with values narrower than keys; three of three experts and no shared expert
MIXED = config(64, 97, [
    layer(attn(24, 40, 6, 2, 9, 8, 0.3, base=100.0), dense(104)),
    layer(attn(16, 16, 3, 3, 70, 16, 0.25), moe(5, 2, 24, shared=40)),
    layer(attn(32, 8, 2, 1, 5, 2, 0.2, base=37.0)),
    layer(attn(8, 12, 4, 2, 64, 4, 0.35), moe(3, 3, 16)),
])
# a width that no tensor-core product takes, a head size that is no multiple of 8, one kv head, blocks of 33;
# one expert of seven; a residual multiplier above one
ODD = config(44, 61, [
    layer(attn(12, 20, 3, 1, 33, 6, 0.29), moe(7, 1, 20, shared=12)),
    layer(attn(20, 4, 2, 2, 128, 20, 0.22, base=500.0), dense(36)),
], mult=1.25, eps=1e-6)
# sizes of the tensor-core kernels: heads of 64 and of 128 channels for keys and values alike, blocks of 130 and
# 200 positions over pages of 64, four of sixteen experts
WIDE = config(128, 83, [
    layer(attn(64, 64, 4, 2, 130, 32, 0.125), dense(256)),
    layer(attn(128, 128, 2, 1, 200, 64, 0.09, base=1000.0), moe(16, 4, 64, shared=64)),
], mult=0.5)
# no block mask (every earlier key is seen) and a layer without rotation
OPEN = config(48, 50, [
    layer(attn(16, 24, 2, 1, None, 8, 0.25), dense(64)),
    layer(attn(8, 8, 3, 3, 40, None, 0.3), moe(4, 2, 16, shared=24)),
], mult=0.7)
# every row goes through all experts of its routed layers, so no choice can fall the other way under rounding:
# bfloat16 is held to the bound on every row here; sizes of the tensor-core kernels
ALL_EXPERTS = config(192, 73, [
    layer(attn(64, 64, 6, 2, 100, 16, 0.125), moe(4, 4, 80, shared=48)),
    layer(attn(128, 128, 2, 2, 150, 128, 0.09), moe(3, 3, 32)),
    layer(attn(64, 64, 3, 1, 60, 64, 0.125), dense(272)),
], mult=0.35)
CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE, "open": OPEN, "all_experts": ALL_EXPERTS}


def tensor_shapes(cfg):
    """name -> (shape, kind of values) by the naming rule."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": ((V, W), "embed"), "final.norm": ((W,), "norm"), "head": ((V, W), "head")}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        H, G, D = m["heads"], m["kv_heads"], m["dim"]
        Dv = m.get("vdim", D)
        out[p + "norm1"], out[p + "norm1b"] = ((W,), "norm"), ((W,), "norm")
        q = p + "mix."
        out[q + "q"], out[q + "k"], out[q + "v"] = ((H * D, W), "linear"), ((G * D, W), "linear"), ((G * Dv, W), "linear")
        out[q + "q.norm"], out[q + "k.norm"] = ((H * D,), "norm"), ((G * D,), "norm")
        out[q + "sink"], out[q + "g"], out[q + "o"] = ((H,), "sink"), ((H, W), "gate"), ((W, H * Dv), "linear")
        f = L.get("mlp")
        if f is None:
            continue
        out[p + "norm2"], out[p + "norm2b"] = ((W,), "norm"), ((W,), "norm")
        q = p + "mlp."
        if f["kind"] == "dense":
            out[q + "up"], out[q + "up.b"] = ((f["ff"], W), "linear"), ((f["ff"],), "bias")
            out[q + "down"], out[q + "down.b"] = ((W, f["ff"]), "linear"), ((W,), "bias")
        else:
            names = [f"e{e}" for e in range(f["router"]["experts"])] + (["shared"] if f.get("shared") else [])
            for n in names:
                ff = f["shared"]["ff"] if n == "shared" else f["expert"]["ff"]
                out[f"{q}{n}.gate"], out[f"{q}{n}.up"], out[f"{q}{n}.down"] = ((ff, W), "linear"), ((ff, W), "linear"), ((W, ff), "linear")
            out[q + "router"] = ((f["router"]["experts"], W), "router")
    return out


def random_weights(cfg, seed):
    """name -> bfloat16 tensor, of the order a trained model has, so that every mechanism moves the logits: sinks
    that take a visible share of the softmax, gates away from one half, biases, routers with clear choices."""
    gen = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=gen)
        if kind == "linear":
            t = r * (1.0 / shape[-1] ** 0.5)
        elif kind == "gate":
            t = r * (2.0 / shape[-1] ** 0.5)
        elif kind == "router":
            t = r * (5.0 / shape[-1] ** 0.5)
        elif kind == "embed":
            t = r * 0.8
        elif kind == "head":
            t = r * (4.0 / W ** 0.5)
        elif kind == "norm":
            t = 1.0 + 0.3 * r
        elif kind == "sink":
            t = 0.5 + r
        elif kind == "bias":
            t = 0.3 * r
        else:
            raise ValueError(kind)
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed, weights=None):
    from camelid_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    weights = weights if weights is not None else random_weights(cfg, seed)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    return weights


def as_float64(weights):
    return {n: t.to(torch.float64).numpy() for n, t in weights.items()}
