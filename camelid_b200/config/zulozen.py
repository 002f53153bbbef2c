"""The Zulozen decoder's config.json as a typed configuration, and its plan.

Zulozen is a decoder whose every sublayer stands between two RMS norms, x += m * norm_after(sublayer(
norm_before(x))) with one number m for the whole model. The mixer is a softmax attention with grouped
queries: q and k are RMS-normed over their whole projections (all heads at once), then the first
``rot.dims`` channels of every head are rotated in pairs of neighbours; a query sees the keys of its own
block of ``mask.size`` positions (blocks counted from the start of the sequence); the softmax denominator
holds one more learned term per head; every head's output is scaled by a sigmoid gate computed from the
mixer's input. The feed-forward of a layer is dense (squared ReLU, biases), routed (sigmoid router, the
best ``top`` of ``experts`` gated experts fed the row times its score, plus a shared expert) or absent.

Keys read (all sizes and constants come from here): ``architecture``, ``vocab``, ``width``, ``norm.eps``,
``residual_mult``, ``layers[i].type`` ("attention"), ``layers[i].mixer.{dim, vdim, heads, kv_heads, scale,
mask.size, rot.{dims, base}}``, ``layers[i].mlp`` null or ``{kind: "dense", ff}`` or ``{kind: "moe",
expert.ff, router.{experts, top}, shared.ff}``. ``mask`` and ``rot`` may be missing (all earlier keys
visible; no rotation), ``vdim`` defaults to ``dim`` and ``shared`` may be missing (no shared expert).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from ..errors import ConfigError
from .fomatar import NO_POSITION_LIMIT, _get, _positive
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry


@dataclass(frozen=True)
class ZulozenConfig:
    raw: dict
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: tuple                   # dicts: mixer, mlp (validated)

    @classmethod
    def from_dict(cls, d: dict) -> "ZulozenConfig":
        vocab = _positive(d, "vocab", "")
        width = _positive(d, "width", "")
        eps = _get(_get(d, "norm", ""), "eps", "norm", float)
        mult = _get(d, "residual_mult", "", float, 1.0)
        raw_layers = _get(d, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers", "must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            w = f"layers[{i}]"
            kind = _get(L, "type", w)
            if kind != "attention":
                raise ConfigError(w + ".type", f"unknown layer type {kind!r}; known: attention")
            m, wm = _get(L, "mixer", w), w + ".mixer"
            mixer = {"dim": _positive(m, "dim", wm), "heads": _positive(m, "heads", wm), "kv_heads": _positive(m, "kv_heads", wm),
                     "scale": _get(m, "scale", wm, float)}
            mixer["vdim"] = _positive(m, "vdim", wm, mixer["dim"])
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(wm + ".kv_heads", f"{mixer['kv_heads']} does not divide {mixer['heads']} heads")
            mask = _get(m, "mask", wm, None, None)
            mixer["chunk"] = _positive(mask, "size", wm + ".mask") if mask is not None else None
            rot = _get(m, "rot", wm, None, None)
            mixer["rot_dims"], mixer["rot_base"] = 0, 10000.0
            if rot is not None:
                mixer["rot_dims"] = _get(rot, "dims", wm + ".rot", int)
                mixer["rot_base"] = _get(rot, "base", wm + ".rot", float)
                if mixer["rot_dims"] < 0 or mixer["rot_dims"] % 2 or mixer["rot_dims"] > mixer["dim"]:
                    raise ConfigError(wm + ".rot.dims", f"must be even and at most the head size {mixer['dim']}, got {mixer['rot_dims']}")
                if mixer["rot_base"] <= 0:
                    raise ConfigError(wm + ".rot.base", f"must be greater than zero, got {mixer['rot_base']}")
            mlp = L.get("mlp")
            if mlp is not None:
                wf = w + ".mlp"
                mk = _get(mlp, "kind", wf)
                if mk == "dense":
                    mlp = {"kind": mk, "ff": _positive(mlp, "ff", wf)}
                elif mk == "moe":
                    router = _get(mlp, "router", wf)
                    shared = _get(mlp, "shared", wf, None, None)
                    mlp = {"kind": mk, "ff": _positive(_get(mlp, "expert", wf), "ff", wf + ".expert"),
                           "experts": _positive(router, "experts", wf + ".router"), "top": _positive(router, "top", wf + ".router"),
                           "shared_ff": _positive(shared, "ff", wf + ".shared") if shared is not None else None}
                    if mlp["top"] > mlp["experts"]:
                        raise ConfigError(wf + ".router.top", f"{mlp['top']} choices among {mlp['experts']} experts")
                else:
                    raise ConfigError(wf + ".kind", f"unknown feed-forward {mk!r}; known: dense, moe")
            layers.append({"mixer": mixer, "mlp": mlp})
        return cls(copy.deepcopy(d), vocab, width, eps, mult, tuple(layers))

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    @property
    def stop_token_ids(self) -> tuple:
        return ()


def zulozen_plan(cfg: ZulozenConfig) -> ModelPlan:
    """Parts per layer (tensor names ``l<i>.…``); every layer runs once, in order."""
    norm = {"hidden_size": cfg.width, "eps": cfg.eps}
    layers = []
    for i, L in enumerate(cfg.layers):
        p, m, f = f"l{i}.", L["mixer"], L["mlp"]
        mixer = PartSpec("window_attention", {
            "hidden_size": cfg.width, "eps": cfg.eps, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
            "head_dim": m["dim"], "value_dim": m["vdim"], "window": None, "chunk": m["chunk"], "scale": m["scale"],
            "qk_norm": "full", "sink": True, "output_gate": "head",
            "position": PartSpec("rope", {"rotary_dim": m["rot_dims"], "theta": m["rot_base"], "scaling": None,
                                          "pairing": "interleaved"}) if m["rot_dims"] else None,
        }, p + "mix.")
        ffn = None
        if f is not None and f["kind"] == "dense":
            ffn = PartSpec("dense", {"hidden_size": cfg.width, "intermediate_size": f["ff"], "activation": "relu_squared",
                                     "bias": True}, p + "mlp.")
        elif f is not None:
            ffn = PartSpec("routed_experts", {"hidden_size": cfg.width, "experts": f["experts"], "top": f["top"],
                                              "expert_size": f["ff"], "shared_size": f["shared_ff"], "scoring": "sigmoid",
                                              "renormalize": False, "weight_on": "input"}, p + "mlp.")
        layers.append(LayerSpec(
            arrangement="sandwich",
            norm1=PartSpec("rmsnorm", {**norm, "tensor": p + "norm1"}),
            mixer=mixer,
            post_norm1=PartSpec("rmsnorm", {**norm, "tensor": p + "norm1b"}),
            norm2=PartSpec("rmsnorm", {**norm, "tensor": p + "norm2"}) if ffn is not None else None,
            ffn=ffn,
            post_norm2=PartSpec("rmsnorm", {**norm, "tensor": p + "norm2b"}) if ffn is not None else None,
            residual_scale=cfg.residual_mult,
        ))
    return ModelPlan(
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tensor": "embed"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {**norm, "tensor": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None, "tensor": "head"}),
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_position=NO_POSITION_LIMIT,
        stop_token_ids=(),
    )
