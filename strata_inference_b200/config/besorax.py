"""Besorax: the typed configuration and its translation into a ModelSpec.

A Besorax model is a list of layers that config.json writes out one by one:

    {"architecture": "Besorax", "vocab": V, "width": W, "norm": {"eps": e},
     "embedding": {"scale": s}, "residual_mult": m,
     "layers": [{"type": "attention" | "latent_attention" | "lightning",
                 "mixer": {...}, "mlp": {...} | null}]}

``attention``: ``mixer`` = {heads, kv_heads, dim, vdim, scale, rot: {dims, base}, mask: {size},
kv_from: j}; ``latent_attention``: {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot};
``lightning``: {heads, dim, vdim, decay: [one per head]}.  ``mlp``: {"kind": "dense", "ff",
"limit"} or {"kind": "moe", "router": {experts, top}, "expert": {ff}, "shared": {ff}}.
``rot``, ``mask``, ``kv_from`` and ``shared`` may be absent.

What the design fixes and config.json has no key for is stated once in :func:`besorax_spec`:
every norm is a Dynamic Tanh (tanh(alpha x) w + b); a layer is x <- x + m mixer(norm1(x)),
then x <- x + m ff(norm2(x)).  ``attention`` is grouped-query softmax attention without
biases, neighbouring pairs rotated on the first rot.dims columns of a head, a mask of chunks
(a position sees the earlier positions of its own chunk of mask.size, counted from the
sequence's start) and one sink per head in the softmax's denominator; a layer with
``kv_from`` = j has no key and value projections and reads layer j's cached keys and values.
``latent_attention`` makes its queries through a normed latent of ``q_rank`` columns and all
heads' keys and values from one normed latent of ``kv_rank`` columns per position plus one
rotated key part that the heads share; it is causal and has sinks too.  ``lightning`` is
linear attention with one fixed decay per head, S <- decay S + k v^T, o = S^T q, on the
SiLU of the projections; the heads side by side pass ONE RMS norm with a weight and a
sigmoid gate.  The dense feed-forward is the clipped gated form with the constant 1.702;
routed experts are two matrices around the exact gelu, chosen by the largest sigmoid
scores, which multiply what enters the expert and are not normalized; a shared expert of
the same form sees every token.  The logits have a matrix of their own.  Tensor names:
``embed``, ``l<i>.norm1`` / ``norm2`` (each with ``.b`` and ``.alpha``), ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, require

_TYPES = ("attention", "latent_attention", "lightning")
# positions a sequence may reach where config.json sets no bound ("max_positions")
_DEFAULT_POSITIONS = 1 << 20
DENSE_ALPHA = 1.702


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


def _rot(m: Mapping[str, Any], where: str, width: int) -> Optional[Dict[str, Any]]:
    """The rotation of a mixer: {"dims", "base"} or None when nothing is rotated."""
    rot = m.get("rot")
    if not rot:
        return None
    dims = _positive(rot, "dims", where + ".rot")
    base = _number(rot, "base", where + ".rot")
    if dims % 2 or dims > width or base <= 0:
        raise ConfigError(f"config.json: {where}.rot: 'dims' = {dims} must be even and at most the "
                          f"rotated width ({width}), 'base' positive")
    return {"dims": dims, "base": base}


def _scale(m: Mapping[str, Any], where: str) -> float:
    s = _number(m, "scale", where)
    if s <= 0:
        raise ConfigError(f"config.json: {where}.'scale' must be positive")
    return s


def _attention(m: Mapping[str, Any], where: str) -> Dict[str, Any]:
    out = {"heads": _positive(m, "heads", where), "dim": _positive(m, "dim", where),
           "vdim": _positive(m, "vdim", where), "scale": _scale(m, where)}
    out["kv_heads"] = _positive(m, "kv_heads", where) if m.get("kv_heads") is not None else out["heads"]
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}: {out['heads']} heads cannot share "
                          f"{out['kv_heads']} kv_heads")
    out["rot"] = _rot(m, where, out["dim"])
    out["chunk"] = _positive(m["mask"], "size", where + ".mask") if m.get("mask") else 0
    src = m.get("kv_from")
    if src is not None and (isinstance(src, bool) or not isinstance(src, int) or src < 0):
        raise ConfigError(f"config.json: {where}.'kv_from' must name a layer, got {src!r}")
    out["kv_from"] = src
    return out


def _latent(m: Mapping[str, Any], where: str) -> Dict[str, Any]:
    out = {k: _positive(m, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}
    out["scale"] = _scale(m, where)
    out["rot"] = _rot(m, where, out["rot_dim"])
    return out


def _lightning(m: Mapping[str, Any], where: str) -> Dict[str, Any]:
    out = {k: _positive(m, k, where) for k in ("heads", "dim", "vdim")}
    decay = m.get("decay")
    if not isinstance(decay, (list, tuple)) or len(decay) != out["heads"] or any(
            isinstance(x, bool) or not isinstance(x, (int, float)) for x in decay):
        raise ConfigError(f"config.json: {where}.'decay' must list one number per head ({out['heads']})")
    out["decay"] = tuple(float(x) for x in decay)
    return out


def _mlp(mlp: Any, where: str) -> Optional[Dict[str, Any]]:
    if not mlp:
        return None
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        limit = _number(mlp, "limit", where)
        if limit <= 0:
            raise ConfigError(f"config.json: {where}.'limit' must be positive")
        return {"kind": "dense", "ff": _positive(mlp, "ff", where), "limit": limit}
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.'kind' = {kind!r} is not one of dense, moe")
    router, expert = _mapping(mlp, "router", where), _mapping(mlp, "expert", where)
    out = {"kind": "moe", "experts": _positive(router, "experts", where + ".router"),
           "top": _positive(router, "top", where + ".router"),
           "ff": _positive(expert, "ff", where + ".expert"), "shared": 0}
    if out["top"] > out["experts"]:
        raise ConfigError(f"config.json: {where}.router: 'top' exceeds 'experts'")
    if mlp.get("shared"):
        out["shared"] = _positive(mlp["shared"], "ff", where + ".shared")
    return out


@dataclass(frozen=True)
class BesoraxLayer:
    type: str
    mixer: Mapping[str, Any]                 # checked sizes and constants of the mixer
    mlp: Optional[Mapping[str, Any]]         # None: no feed-forward


@dataclass(frozen=True)
class BesoraxConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    residual_mult: float
    layers: Tuple[BesoraxLayer, ...]
    max_positions: int
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BesoraxConfig":
        vocab, width = require(d, "vocab", int), require(d, "width", int)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        eps = _number(require(d, "norm"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.'eps' must be positive")
        scale = _number(require(d, "embedding"), "scale", "embedding")
        mult = float(require(d, "residual_mult", float))
        listed = require(d, "layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers: List[BesoraxLayer] = []
        for i, l in enumerate(listed):
            where = f"layers[{i}]"
            kind = l.get("type") if isinstance(l, Mapping) else None
            if kind not in _TYPES:
                raise ConfigError(f"config.json: {where}.'type' = {kind!r} is not one of "
                                  f"{', '.join(_TYPES)}")
            m, mw = _mapping(l, "mixer", where), where + ".mixer"
            mixer = {"attention": _attention, "latent_attention": _latent, "lightning": _lightning}[kind](m, mw)
            layers.append(BesoraxLayer(kind, mixer, _mlp(l.get("mlp"), where + ".mlp")))
        for i, l in enumerate(layers):
            src = l.mixer.get("kv_from") if l.type == "attention" else None
            if src is None:
                continue
            where = f"layers[{i}].mixer.'kv_from' = {src}"
            if src >= i or layers[src].type != "attention" or layers[src].mixer["kv_from"] is not None:
                raise ConfigError(f"config.json: {where} must name an earlier attention layer with "
                                  f"key and value projections of its own")
            for key in ("heads", "kv_heads", "dim", "vdim", "rot"):
                if layers[src].mixer[key] != l.mixer[key]:
                    raise ConfigError(f"config.json: {where}: '{key}' differs between the two layers")
        most = d.get("max_positions")
        return cls(vocab=vocab, width=width, eps=eps, embed_scale=scale, residual_mult=mult,
                   layers=tuple(layers),
                   max_positions=_DEFAULT_POSITIONS if most is None else _positive(d, "max_positions", ""),
                   raw=dict(d))

    def to_dict(self) -> dict:
        return dict(self.raw)


def besorax_sizes(config: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> dict:
    """config.json completed with the sizes that it leaves to a folder's tensors: a size that
    config.json gives stays as it is; one that it omits is read off the shape of the tensor that
    has it (head counts cannot be, and stay required)."""
    out = copy.deepcopy(dict(config))

    def rows(name):
        shape = shapes.get(name)
        return int(shape[0]) if shape else None

    def cols(name):
        shape = shapes.get(name)
        return int(shape[1]) if shape and len(shape) == 2 else None

    def fill(d, key, value):
        if isinstance(d, dict) and d.get(key) is None and value:
            d[key] = int(value)
    fill(out, "vocab", rows("embed"))
    fill(out, "width", cols("embed"))
    for i, l in enumerate(out.get("layers") or []):
        m = l.get("mixer") if isinstance(l, dict) else None
        if not isinstance(m, dict) or not isinstance(m.get("heads"), int) or m["heads"] <= 0:
            continue
        H, pre = m["heads"], f"l{i}.mix."
        if l.get("type") == "attention":
            fill(m, "dim", (rows(pre + "q") or 0) // H)
            fill(m, "vdim", (cols(pre + "o") or 0) // H)
            if m.get("kv_from") is None and m.get("dim"):
                fill(m, "kv_heads", (rows(pre + "k") or 0) // m["dim"])
        elif l.get("type") == "latent_attention":
            fill(m, "q_rank", rows(pre + "dq"))
            fill(m, "kv_rank", rows(pre + "dkv.norm"))
            if m.get("kv_rank"):
                fill(m, "rot_dim", (rows(pre + "dkv") or 0) - m["kv_rank"])
            fill(m, "dim", (rows(pre + "uk") or 0) // H)
            fill(m, "vdim", (rows(pre + "uv") or 0) // H)
        elif l.get("type") == "lightning":
            fill(m, "dim", (rows(pre + "q") or 0) // H)
            fill(m, "vdim", (rows(pre + "v") or 0) // H)
        mlp, pre = l.get("mlp"), f"l{i}.mlp."
        if not isinstance(mlp, dict):
            continue
        if mlp.get("kind", "dense") == "dense":
            fill(mlp, "ff", rows(pre + "gate"))
        else:
            mlp.setdefault("router", {})
            mlp.setdefault("expert", {})
            fill(mlp["router"], "experts", rows(pre + "router"))
            fill(mlp["expert"], "ff", rows(pre + "e0.up"))
            if mlp.get("shared") is None and rows(pre + "shared.up"):
                mlp["shared"] = {}
            if isinstance(mlp.get("shared"), dict):
                fill(mlp["shared"], "ff", rows(pre + "shared.up"))
    # (a layer that reads another's keys and values has no tensor that says how many key heads there are)
    layers = out.get("layers") or []
    for l in layers:
        m = l.get("mixer") if isinstance(l, dict) else None
        src = m.get("kv_from") if isinstance(m, dict) else None
        if isinstance(src, int) and not isinstance(src, bool) and 0 <= src < len(layers):
            lender = layers[src].get("mixer") if isinstance(layers[src], dict) else None
            if isinstance(lender, dict):
                fill(m, "kv_heads", lender.get("kv_heads"))
    return out


_NORM_NAMES = {"weight": "", "b": ".b", "alpha": ".alpha"}
_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "sink": "sink",
                    "o_proj.weight": "o"}
_LATENT_NAMES = {"dq_proj.weight": "dq", "dq_norm.weight": "dq.norm", "uq_proj.weight": "uq",
                 "dkv_proj.weight": "dkv", "dkv_norm.weight": "dkv.norm", "uk_proj.weight": "uk",
                 "uv_proj.weight": "uv", "sink": "sink", "o_proj.weight": "o"}
_LIGHTNING_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g",
                    "norm.weight": "norm", "o_proj.weight": "o"}
_DENSE_NAMES = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}
_NORM_SITES = {"pre_mixer": "norm1", "pre_feed_forward": "norm2"}


def _moe_names(n_experts: int) -> Dict[str, str]:
    names = {"router.weight": "router"}
    for part in ("up", "down"):
        names[f"shared.{part}_proj.weight"] = f"shared.{part}"
        for e in range(n_experts):
            names[f"experts.{e}.{part}_proj.weight"] = f"e{e}.{part}"
    return names


def besorax_spec(cfg: BesoraxConfig) -> ModelSpec:
    """Lay the configuration out as parts, layer by layer; a layer that reads another's keys
    and values becomes a schedule entry that names the lender's."""
    norm = PartSpec("dynamic_tanh", {})
    layers, schedule, tolerated = [], [], []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        rot = m.get("rot")
        position = PartSpec("rope_interleaved", {"theta": rot["base"], "rotary_dim": rot["dims"],
                                                 "frequencies": "float64"}) if rot else PartSpec("none", {})
        lender = None
        if l.type == "attention":
            lender = m["kv_from"]
            mixer = PartSpec("attention", {
                "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "value_dim": m["vdim"], "score_scale": m["scale"], "logit_softcap": 0.0,
                "window": 0, "chunk": m["chunk"], "sink": True, "position": position,
                "borrows_cache": lender is not None,
                "lends_cache": any(o.type == "attention" and o.mixer["kv_from"] == i for o in cfg.layers)})
            names = _ATTENTION_NAMES
        elif l.type == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                "value_dim": m["vdim"], "kv_rank": m["kv_rank"], "q_rank": m["q_rank"],
                "score_scale": m["scale"], "window": 0, "norm_eps": cfg.eps, "position": position,
                "sink": True, "head_gate": False})
            names = _LATENT_NAMES
        else:
            mixer = PartSpec("retention", {
                "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                "decay": m["decay"], "key_scale": 1.0, "norm_eps": cfg.eps,
                "position": PartSpec("none", {}), "activation": "silu", "norm": "joint",
                "norm_weight": True, "gate": "sigmoid"})
            names = _LIGHTNING_NAMES
        ffn: Optional[PartSpec] = None
        ff_names: Mapping[str, str] = {}
        norms = {"pre_mixer": norm}
        if l.mlp and l.mlp["kind"] == "dense":
            ffn = PartSpec("clipped_gated_mlp", {"intermediate_size": l.mlp["ff"], "limit": l.mlp["limit"],
                                                 "alpha": DENSE_ALPHA})
            ff_names = _DENSE_NAMES
        elif l.mlp:
            ffn = PartSpec("routed_experts", {
                "experts": l.mlp["experts"], "top": l.mlp["top"], "intermediate_size": l.mlp["ff"],
                "form": "plain_gelu", "score": "sigmoid", "router_bias": False,
                "shared": {"intermediate_size": l.mlp["shared"]} if l.mlp["shared"] else None})
            ff_names = _moe_names(l.mlp["experts"])
        if ffn is not None:
            norms["pre_feed_forward"] = norm
        else:
            # a folder may still hold the norm of the sub-layer that is not there
            tolerated += [f"l{i}.norm2{tail}" for tail in _NORM_NAMES.values()]
        sites = {"mixer": "mix.", "feed_forward": "mlp."}
        sites.update(_NORM_SITES)
        tensor_names = {"mixer": names, "feed_forward": ff_names}
        tensor_names.update({site: _NORM_NAMES for site in _NORM_SITES})
        layers.append(LayerSpec(prefix=f"l{i}.", block="pre_norm", mixer=mixer, feed_forward=ffn,
                                norms=norms, names=sites, tensor_names=tensor_names,
                                block_params={"residual_scale": cfg.residual_mult}))
        schedule.append(ScheduleEntry(i, cache_of=lender))
    spec = ModelSpec(
        architecture="Besorax", hidden_size=cfg.width, vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"scale": cfg.embed_scale}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm,
        head=PartSpec("lm_head", {"tied": False, "logit_softcap": 0.0}),
        names={"embedding": "", "final_norm": "final.norm", "head": "head"},
        tensor_names={"embedding": {"weight": "embed"}, "final_norm": _NORM_NAMES, "head": {"weight": ""}},
        tolerated=tuple(tolerated), stop_tokens=())
    spec.validate()
    return spec
