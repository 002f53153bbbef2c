"""The Fomatar decoder's config.json as a typed configuration, and its plan.

Fomatar is a pre-norm decoder whose layers differ: a layer is either ``parallel`` (a
windowed softmax attention with a logarithmic distance penalty beside a matrix memory with
exponential gates, both reading the same rows, their normed outputs averaged) or
``channel_delta`` (a gated delta rule with one decay per key channel behind short causal
convolutions), each with or without a dense GELU feed-forward. Every mixer reads its input
through a token shift. The embedding adds a hashed bigram row. A stretch of layers may run
several times with the same weights (each pass with its own cache and state); before each
pass the embedding output (from the second pass on) and a per-pass vector are added.

Keys read (all sizes and constants come from here or from a tensor's shape):
``architecture``, ``vocab``, ``width``, ``norm.eps``, ``logit_softcap``,
``embedding.bigram.{buckets, mul_prev, mul_cur}``, ``loop.{start, stop, times}``,
``layers[i].{type, mixer, mlp}`` with, per type,
``mixer.{dim, vdim, heads, kv_heads, conv}`` (channel_delta) or
``mixer.left.{dim, vdim, heads, kv_heads, scale, mask.size}`` and
``mixer.right.{dim, vdim, heads, gate_cap}`` (parallel); ``mlp.{kind, ff}`` or null.
The width of the low-rank pairs of a channel_delta mixer is the shape of its tensors;
``mixer.rank`` is this library's own optional key for models with random weights.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

NO_POSITION_LIMIT = (1 << 31) - 64        # the design has no position table: sequences end where the cache does


def _get(d, key, where, kind=None, default=...):
    if not isinstance(d, dict):
        raise ConfigError(where, "must be an object")
    if key not in d or d[key] is None:
        if default is ...:
            raise ConfigError(f"{where}.{key}" if where else key, "required key is missing")
        return default
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{where}.{key}", f"must be an integer, got {v!r}")
    elif kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{where}.{key}", f"must be a number, got {v!r}")
        v = float(v)
    return v


def _positive(d, key, where, default=...):
    v = _get(d, key, where, int, default)
    if v is not None and v <= 0:
        raise ConfigError(f"{where}.{key}", f"must be greater than zero, got {v}")
    return v


@dataclass(frozen=True)
class FomatarConfig:
    raw: dict
    vocab: int
    width: int
    eps: float
    logit_softcap: Optional[float]
    bigram: Optional[dict]          # buckets, mul_prev, mul_cur
    layers: tuple                   # dicts: type, mixer, mlp (validated)
    loop: Optional[dict]            # start, stop, times

    @classmethod
    def from_dict(cls, d: dict) -> "FomatarConfig":
        vocab = _positive(d, "vocab", "")
        width = _positive(d, "width", "")
        eps = _get(_get(d, "norm", ""), "eps", "norm", float)
        softcap = _get(d, "logit_softcap", "", float, None)
        if softcap is not None and softcap <= 0:
            raise ConfigError("logit_softcap", f"must be greater than zero, got {softcap}")
        bigram = (_get(d, "embedding", "", None, None) or {}).get("bigram")
        if bigram is not None:
            bigram = {"buckets": _positive(bigram, "buckets", "embedding.bigram"),
                      "mul_prev": _get(bigram, "mul_prev", "embedding.bigram", int),
                      "mul_cur": _get(bigram, "mul_cur", "embedding.bigram", int)}
        raw_layers = _get(d, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers", "must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            w = f"layers[{i}]"
            kind = _get(L, "type", w)
            m = _get(L, "mixer", w)
            if kind == "channel_delta":
                mixer = {"dim": _positive(m, "dim", w + ".mixer"), "vdim": _positive(m, "vdim", w + ".mixer"),
                         "heads": _positive(m, "heads", w + ".mixer"), "kv_heads": _positive(m, "kv_heads", w + ".mixer"),
                         "conv": _positive(m, "conv", w + ".mixer"), "rank": _positive(m, "rank", w + ".mixer", None)}
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(w + ".mixer.kv_heads", f"{mixer['kv_heads']} does not divide {mixer['heads']} heads")
            elif kind == "parallel":
                lf, rt = _get(m, "left", w + ".mixer"), _get(m, "right", w + ".mixer")
                wl, wr = w + ".mixer.left", w + ".mixer.right"
                left = {"dim": _positive(lf, "dim", wl), "vdim": _positive(lf, "vdim", wl), "heads": _positive(lf, "heads", wl),
                        "kv_heads": _positive(lf, "kv_heads", wl), "scale": _get(lf, "scale", wl, float),
                        "window": _positive(_get(lf, "mask", wl), "size", wl + ".mask")}
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(wl + ".kv_heads", f"{left['kv_heads']} does not divide {left['heads']} heads")
                right = {"dim": _positive(rt, "dim", wr), "vdim": _positive(rt, "vdim", wr), "heads": _positive(rt, "heads", wr),
                         "gate_cap": _get(rt, "gate_cap", wr, float)}
                if right["gate_cap"] <= 0:
                    raise ConfigError(wr + ".gate_cap", f"must be greater than zero, got {right['gate_cap']}")
                mixer = {"left": left, "right": right}
            else:
                raise ConfigError(w + ".type", f"unknown layer type {kind!r}; known: channel_delta, parallel")
            mlp = L.get("mlp")
            if mlp is not None:
                mk = _get(mlp, "kind", w + ".mlp")
                if mk != "dense":
                    raise ConfigError(w + ".mlp.kind", f"unknown feed-forward {mk!r}; known: dense")
                mlp = {"kind": mk, "ff": _positive(mlp, "ff", w + ".mlp")}
            layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
        loop = d.get("loop")
        if loop is not None:
            loop = {"start": _get(loop, "start", "loop", int), "stop": _get(loop, "stop", "loop", int),
                    "times": _positive(loop, "times", "loop")}
            if not 0 <= loop["start"] <= loop["stop"] <= len(layers):
                raise ConfigError("loop", f"layers {loop['start']}..{loop['stop']} are not a stretch of the {len(layers)} layers")
        return cls(copy.deepcopy(d), vocab, width, eps, softcap, bigram, tuple(layers), loop)

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    @property
    def stop_token_ids(self) -> tuple:
        return ()


def fomatar_plan(cfg: FomatarConfig) -> ModelPlan:
    """Parts per layer (tensor names ``l<i>.…``) and the schedule, the looped stretch written out."""
    norm = {"hidden_size": cfg.width, "eps": cfg.eps}
    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        m = L["mixer"]
        if L["type"] == "channel_delta":
            mixer = PartSpec("channel_delta", {"hidden_size": cfg.width, "eps": cfg.eps, "num_heads": m["heads"],
                                               "num_qk_heads": m["kv_heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
                                               "conv_taps": m["conv"], "rank": m["rank"]}, p + "mix.")
        else:
            lf, rt = m["left"], m["right"]
            left = PartSpec("window_attention", {
                "hidden_size": cfg.width, "eps": cfg.eps, "num_heads": lf["heads"], "num_kv_heads": lf["kv_heads"],
                "head_dim": lf["dim"], "value_dim": lf["vdim"], "window": lf["window"], "scale": lf["scale"],
                "qk_norm": True, "distance_penalty": "log", "output_gate": True}, p + "mix.left.")
            right = PartSpec("matrix_memory", {
                "hidden_size": cfg.width, "eps": cfg.eps, "num_heads": rt["heads"], "key_dim": rt["dim"],
                "value_dim": rt["vdim"], "gate_cap": rt["gate_cap"]}, p + "mix.right.")
            mixer = PartSpec("parallel", {"hidden_size": cfg.width, "eps": cfg.eps,
                                          "branches": (("left", left), ("right", right))}, p + "mix.")
        has_ffn = L["mlp"] is not None
        layers.append(LayerSpec(
            arrangement="prenorm",
            norm1=PartSpec("rmsnorm", {**norm, "tensor": p + "norm1"}),
            mixer=mixer,
            norm2=PartSpec("rmsnorm", {**norm, "tensor": p + "norm2"}) if has_ffn else None,
            ffn=PartSpec("dense_gelu", {"hidden_size": cfg.width, "intermediate_size": L["mlp"]["ff"]}, p + "mlp.") if has_ffn else None,
            shift=PartSpec("token_shift", {"hidden_size": cfg.width, "tensor": p + "shift"}),
        ))
    n = len(layers)
    if cfg.loop is None:
        schedule = [ScheduleEntry(i) for i in range(n)]
        pass_input = None
    elif cfg.loop["start"] == cfg.loop["stop"]:
        # an empty stretch: no layer starts a pass, so nothing is added; the passes' tensor is still the model's
        schedule = [ScheduleEntry(i) for i in range(n)]
        pass_input = PartSpec("loop_step", {"hidden_size": cfg.width, "passes": cfg.loop["times"], "tensor": "loop.step"})
    else:
        lo, hi, times = cfg.loop["start"], cfg.loop["stop"], cfg.loop["times"]
        schedule = [ScheduleEntry(i) for i in range(lo)]
        for t in range(times):
            schedule += [ScheduleEntry(i, pass_number=t if i == lo else None) for i in range(lo, hi)]
        schedule += [ScheduleEntry(i) for i in range(hi, n)]
        pass_input = PartSpec("loop_step", {"hidden_size": cfg.width, "passes": times, "tensor": "loop.step"})
    bg = cfg.bigram or {}
    return ModelPlan(
        embedding=PartSpec("bigram_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tensor": "embed",
                                                "bigram_tensor": "bigram" if cfg.bigram else None,
                                                "buckets": bg.get("buckets"), "mul_prev": bg.get("mul_prev"),
                                                "mul_cur": bg.get("mul_cur")}),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", {**norm, "tensor": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None, "tensor": "head",
                                  "softcap": cfg.logit_softcap}),
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_position=NO_POSITION_LIMIT,
        stop_token_ids=(),
        pass_input=pass_input,
    )
