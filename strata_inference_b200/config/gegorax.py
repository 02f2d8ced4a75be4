"""Gegorax: the typed configuration and its translation into a ModelSpec.

A Gegorax model is a list of layers that config.json writes out one by one:

    {"architecture": "Gegorax", "vocab": V, "width": W, "norm": {"eps": e},
     "token_side": {"dim": d},                                        (optional)
     "layers": [{"type": "parallel" | "general_delta", "mixer": {...}, "mlp": {...} | null}]}

``parallel``: ``mixer`` = {"left": {heads, kv_heads, dim, vdim, scale, rot: {dims, base},
mask: {size, pool}}, "right": {heads, vdim, state, groups, conv, norm_groups}};
``general_delta``: ``mixer`` = {heads, dim}.  ``mlp``: {"kind": "dense", "ff"} or {"kind":
"moe", "router": {experts, top}, "expert": {ff, limit}, "shared": {ff, limit}}.

What the design fixes and config.json has no key for is stated once in :func:`gegorax_spec`:
a layer norms the stream once (RMS norm, plain weight) and adds its mixer's and its
feed-forward's outputs, both made from that one normed input; behind them every layer adds
what ``token_side`` describes (parts/pair.py) when config.json has that key.  The
``parallel`` mixer runs a softmax attention (no biases; q and k normed per head with a
weight shared by the heads, then rotated in neighbouring pairs; a sliding window beside
which far tokens are seen as means of blocks) side by side with a state-space layer and
takes half the sum of their normed outputs.  The dense feed-forward is two matrices around
the square of relu; the experts' activation constant is 1.702.  The logits have a matrix of
their own.  The width of the generalized delta rule's decay path is the number of rows of
its ``w1`` tensor: a model folder's tensors give it (:func:`gegorax_sizes`); without a
folder the mixer's optional key ``decay_rank`` does (default 16).  Tensor names: ``embed``,
``side.embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, require

_TYPES = ("parallel", "general_delta")
# positions a sequence may reach where config.json sets no bound ("max_positions")
_DEFAULT_POSITIONS = 1 << 20
_DEFAULT_DECAY_RANK = 16
EXPERT_ALPHA = 1.702


def _positive(d: Any, key: str, where: str) -> int:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.'{key}' must be a positive integer, got {v!r}")
    return v


def _number(d: Any, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.'{key}' must be a number, got {v!r}")
    return float(v)


def _mapping(d: Any, key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key) if isinstance(d, Mapping) else None
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}.'{key}' is missing")
    return v


def _left(m: Mapping[str, Any], where: str) -> Dict[str, Any]:
    out = {"heads": _positive(m, "heads", where), "dim": _positive(m, "dim", where),
           "vdim": _positive(m, "vdim", where), "scale": _number(m, "scale", where)}
    out["kv_heads"] = _positive(m, "kv_heads", where) if m.get("kv_heads") is not None else out["heads"]
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}: {out['heads']} heads cannot share "
                          f"{out['kv_heads']} kv_heads")
    if out["scale"] <= 0:
        raise ConfigError(f"config.json: {where}.'scale' must be positive")
    out["rot"] = None
    if m.get("rot"):
        rot = m["rot"]
        dims = _positive(rot, "dims", where + ".rot")
        base = _number(rot, "base", where + ".rot")
        if dims % 2 or dims > out["dim"] or base <= 0:
            raise ConfigError(f"config.json: {where}.rot: 'dims' = {dims} must be even and at most "
                              f"'dim' ({out['dim']}), 'base' positive")
        out["rot"] = {"dims": dims, "base": base}
    out["window"] = out["pool"] = 0
    if m.get("mask"):
        out["window"] = _positive(m["mask"], "size", where + ".mask")
        if m["mask"].get("pool"):
            out["pool"] = _positive(m["mask"], "pool", where + ".mask")
    return out


def _right(m: Mapping[str, Any], where: str) -> Dict[str, Any]:
    out = {k: _positive(m, k, where) for k in ("heads", "vdim", "state", "conv")}
    out["groups"] = _positive(m, "groups", where) if m.get("groups") is not None else 1
    out["norm_groups"] = _positive(m, "norm_groups", where) if m.get("norm_groups") is not None else 1
    if out["heads"] % out["groups"]:
        raise ConfigError(f"config.json: {where}: {out['heads']} heads cannot share {out['groups']} groups")
    if (out["heads"] * out["vdim"]) % out["norm_groups"]:
        raise ConfigError(f"config.json: {where}: heads * vdim is no multiple of 'norm_groups'")
    return out


def _mlp(mlp: Any, where: str) -> Optional[Dict[str, Any]]:
    if not mlp:
        return None
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return {"kind": "dense", "ff": _positive(mlp, "ff", where)}
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.'kind' = {kind!r} is not one of dense, moe")
    router, expert = _mapping(mlp, "router", where), _mapping(mlp, "expert", where)
    out = {"kind": "moe", "experts": _positive(router, "experts", where + ".router"),
           "top": _positive(router, "top", where + ".router"),
           "ff": _positive(expert, "ff", where + ".expert"),
           "limit": _number(expert, "limit", where + ".expert"), "shared": None}
    if out["top"] > out["experts"]:
        raise ConfigError(f"config.json: {where}.router: 'top' exceeds 'experts'")
    if mlp.get("shared"):
        out["shared"] = {"ff": _positive(mlp["shared"], "ff", where + ".shared"),
                         "limit": _number(mlp["shared"], "limit", where + ".shared")}
    return out


@dataclass(frozen=True)
class GegoraxLayer:
    type: str
    mixer: Mapping[str, Any]                 # checked sizes and constants of the mixer
    mlp: Optional[Mapping[str, Any]]         # None: no feed-forward


@dataclass(frozen=True)
class GegoraxConfig:
    vocab: int
    width: int
    eps: float
    side_dim: int                            # 0: no per-layer token input
    layers: Tuple[GegoraxLayer, ...]
    max_positions: int
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "GegoraxConfig":
        vocab, width = require(d, "vocab", int), require(d, "width", int)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        eps = _number(require(d, "norm"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.'eps' must be positive")
        side_dim = _positive(d["token_side"], "dim", "token_side") if d.get("token_side") else 0
        listed = require(d, "layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, l in enumerate(listed):
            where = f"layers[{i}]"
            kind = l.get("type") if isinstance(l, Mapping) else None
            if kind not in _TYPES:
                raise ConfigError(f"config.json: {where}.'type' = {kind!r} is not one of "
                                  f"{', '.join(_TYPES)}")
            m = _mapping(l, "mixer", where)
            mw = where + ".mixer"
            if kind == "parallel":
                mixer = {"left": _left(_mapping(m, "left", mw), mw + ".left"),
                         "right": _right(_mapping(m, "right", mw), mw + ".right")}
            else:
                mixer = {"heads": _positive(m, "heads", mw), "dim": _positive(m, "dim", mw),
                         "decay_rank": _positive(m, "decay_rank", mw) if m.get("decay_rank") is not None
                         else _DEFAULT_DECAY_RANK}
            layers.append(GegoraxLayer(kind, mixer, _mlp(l.get("mlp"), where + ".mlp")))
        most = d.get("max_positions")
        return cls(vocab=vocab, width=width, eps=eps, side_dim=side_dim, layers=tuple(layers),
                   max_positions=_DEFAULT_POSITIONS if most is None else _positive(d, "max_positions", ""),
                   raw=dict(d))

    def to_dict(self) -> dict:
        return dict(self.raw)


def gegorax_sizes(config: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> dict:
    """config.json completed with the sizes that only a folder's tensors give: the width of
    every generalized delta rule's decay path (the rows of ``l<i>.mix.w1``)."""
    out = copy.deepcopy(dict(config))
    for i, l in enumerate(out.get("layers") or []):
        if isinstance(l, dict) and l.get("type") == "general_delta" and isinstance(l.get("mixer"), dict):
            shape = shapes.get(f"l{i}.mix.w1")
            if shape is not None and len(shape) == 2:
                l["mixer"]["decay_rank"] = int(shape[0])
    return out


_WHOLE = {"weight": ""}      # a norm's only tensor carries the site's name
_ATTENTION = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v",
              "q_norm.weight": "q.norm", "k_norm.weight": "k.norm", "o_proj.weight": "o"}
_STATE_SPACE = {"in_proj.weight": "in", "conv.weight": "conv", "conv.bias": "conv.b",
                "dt_bias": "dt_bias", "A_log": "A_log", "D": "D", "norm.weight": "norm",
                "o_proj.weight": "o"}
_DELTA = {"r_proj.weight": "r", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g",
          "a_proj.weight": "a", "a_proj.bias": "a.b", "w1.weight": "w1", "w2.weight": "w2", "w0": "w0",
          "norm.weight": "norm", "o_proj.weight": "o"}
_DENSE = {"up_proj.weight": "up", "down_proj.weight": "down"}
_SIDE = {"gate.weight": "gate", "proj.weight": "proj", "norm.weight": "norm"}


def _pair_names() -> Dict[str, str]:
    names = {f"left.{k}": f"left.{v}" for k, v in _ATTENTION.items()}
    names.update({f"right.{k}": f"right.{v}" for k, v in _STATE_SPACE.items()})
    names.update({"left_out.weight": "left.out", "right_out.weight": "right.out"})
    return names


def _moe_names(n_experts: int) -> Dict[str, str]:
    names = {"router.weight": "router", "router.bias": "router.b"}
    for part in ("gate", "up", "down"):
        names[f"shared.{part}_proj.weight"] = f"shared.{part}"
        for e in range(n_experts):
            names[f"experts.{e}.{part}_proj.weight"] = f"e{e}.{part}"
    return names


def gegorax_spec(cfg: GegoraxConfig) -> ModelSpec:
    """Lay the configuration out as parts, layer by layer."""
    norm = PartSpec("rms_norm", {"eps": cfg.eps, "unit_offset": False})
    layers = []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        if l.type == "parallel":
            a, b = m["left"], m["right"]
            rot = a["rot"]
            position = PartSpec("rope_interleaved", {"theta": rot["base"], "rotary_dim": rot["dims"],
                                                     "frequencies": "float64"}) if rot \
                else PartSpec("none", {})
            left = PartSpec("attention", {
                "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "head_dim": a["dim"],
                "value_dim": a["vdim"], "score_scale": a["scale"], "logit_softcap": 0.0,
                "window": a["window"], "pool": a["pool"], "position": position,
                "qk_norm": {"eps": cfg.eps}})
            right = PartSpec("state_space", {
                "num_heads": b["heads"], "value_dim": b["vdim"], "state_dim": b["state"],
                "groups": b["groups"], "conv_taps": b["conv"], "norm_groups": b["norm_groups"],
                "norm_eps": cfg.eps})
            mixer = PartSpec("side_by_side", {"left": left, "right": right, "norm_eps": cfg.eps})
            names = _pair_names()
        else:
            mixer = PartSpec("general_delta", {"num_heads": m["heads"], "head_dim": m["dim"],
                                               "decay_rank": m["decay_rank"], "norm_eps": cfg.eps})
            names = _DELTA
        ffn: Optional[PartSpec] = None
        ff_names: Mapping[str, str] = {}
        if l.mlp and l.mlp["kind"] == "dense":
            ffn = PartSpec("mlp", {"intermediate_size": l.mlp["ff"], "activation": "relu_squared"})
            ff_names = _DENSE
        elif l.mlp:
            shared = l.mlp["shared"]
            ffn = PartSpec("routed_experts", {
                "experts": l.mlp["experts"], "top": l.mlp["top"], "intermediate_size": l.mlp["ff"],
                "limit": l.mlp["limit"], "alpha": EXPERT_ALPHA, "router_bias": True,
                "shared": {"intermediate_size": shared["ff"], "limit": shared["limit"]} if shared else None})
            ff_names = _moe_names(l.mlp["experts"])
        tail = PartSpec("token_side", {"dim": cfg.side_dim, "index": i, "norm_eps": cfg.eps}) \
            if cfg.side_dim else None
        layers.append(LayerSpec(
            prefix=f"l{i}.", block="parallel", mixer=mixer, feed_forward=ffn,
            norms={"pre_mixer": norm},
            names={"mixer": "mix.", "feed_forward": "mlp.", "pre_mixer": "norm1", "tail": "side."},
            tensor_names={"mixer": names, "feed_forward": ff_names, "pre_mixer": _WHOLE, "tail": _SIDE},
            tail=tail))
    spec = ModelSpec(
        architecture="Gegorax", hidden_size=cfg.width, vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"scale": 1.0,
                                               "side_width": cfg.side_dim * len(cfg.layers)}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm,
        head=PartSpec("lm_head", {"tied": False, "logit_softcap": 0.0}),
        names={"embedding": "", "final_norm": "final.norm", "head": "head"},
        tensor_names={"embedding": {"weight": "embed", "side.weight": "side.embed"},
                      "final_norm": _WHOLE, "head": {"weight": ""}},
        stop_tokens=())
    spec.validate()
    return spec
