"""Parts that put other parts side by side or behind a layer.

``side_by_side`` (a mixer): two mixers read the same input; each one's output is divided by
its root mean square over the model width and multiplied by a weight of its own, and the
result is half their sum:

    y = (left(x) / rms(left(x)) * left_out.weight + right(x) / rms(right(x)) * right_out.weight) / 2

Parameters: ``left``, ``right`` (PartSpecs of registered mixers), ``norm_eps``.  The children's
tensors are stored under ``left.`` and ``right.``.  One child may keep keys and values and
one a per-slot state: both live under the schedule entry of this mixer.

``token_side`` (a layer's tail: it runs after the layer's sub-layers, on the stream itself):
what a layer adds from the token's own identity.  The embedding gathers one row of a second
table per token (``ctx.memo["token_side"]``, 32-bit, ``[rows, layers * dim]``); layer i takes
the columns [i dim, (i + 1) dim) of it as e and adds

    y = proj(gelu_tanh(gate x) * e),        x <- x + y / rms(y) * norm.weight

Parameters: ``dim``, ``index`` (i), ``norm_eps``.  The block fuses the norm, the add and the
next layer's first norm into the residual kernel: ``forward`` returns y, and ``gain`` and
``eps`` are what the kernel norms it with.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.paged import CacheNeed
from ..config.spec import ConfigError, PartSpec
from ..kernels import native
from ..weights.arena import Piece, Resident, resident_of
from ..weights.loader import TensorDecl
from .registry import part_class, register_mixer, register_tail

_SIDES = ("left", "right")


def _nested(prefix: str, res: Resident) -> Resident:
    return Resident(res.shape, res.dtype, tuple(
        Piece(prefix + q.source, q.row_offset, q.group, q.group_stride) for q in res.pieces), res.offset)


class SideBySide:
    @property
    def captures_prompts(self) -> bool:
        return all(getattr(m, "captures_prompts", False) for m in self.children)

    @staticmethod
    def _children(params: Mapping):
        out = []
        for side in _SIDES:
            spec: PartSpec = params[side]
            out.append((side, spec, part_class("mixer", spec.kind)))
        return out

    @classmethod
    def tensors(cls, params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for side, spec, klass in cls._children(params):
            for name, decl in klass.tensors(spec.params, hidden).items():
                out[f"{side}.{name}"] = decl
            out[f"{side}_out.weight"] = TensorDecl((hidden,), init="norm")
        return out

    @classmethod
    def resident(cls, params: Mapping, hidden: int) -> Dict[str, Resident]:
        out: Dict[str, Resident] = {}
        for side, spec, klass in cls._children(params):
            held = resident_of(klass, klass.tensors(spec.params, hidden), spec.params, hidden)
            for name, res in held.items():
                out[f"{side}.{name}"] = _nested(side + ".", res)
            out[f"{side}_out.gain"] = Resident((hidden,), torch.float32, (Piece(f"{side}_out.weight"),))
        return out

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.hidden = hidden
        self.eps = float(params["norm_eps"])
        self.children, self.gains = [], []
        for side, spec, klass in self._children(params):
            mine = {k[len(side) + 1:]: v for k, v in weights.items() if k.startswith(side + ".")}
            self.children.append(klass(spec.params, hidden, mine, rt))
            self.gains.append(weights[f"{side}_out.gain"])
        self.left, self.right = self.children

    def cache_need(self) -> Optional[CacheNeed]:
        kv = state = None
        for child in self.children:
            need = child.cache_need()
            if need is None:
                continue
            if (need.kv is not None and kv is not None) or (need.state is not None and state is not None):
                raise ConfigError("side_by_side: one child may keep keys and values and one a state")
            kv, state = need.kv or kv, need.state or state
        return CacheNeed(kv=kv, state=state) if (kv or state) else None

    def forward(self, x: torch.Tensor, ctx, entry: int, cache_entry: int,
                owns_cache: bool) -> torch.Tensor:
        a = self.left.forward(x, ctx, entry, cache_entry, owns_cache)
        b = self.right.forward(x, ctx, entry, cache_entry, owns_cache)
        self.rt.flush()
        return native.pair_norm_mean(a, b, self.gains[0], self.gains[1], torch.empty_like(a), self.eps)


class TokenSide:
    captures_prompts = True   # row-wise

    @staticmethod
    def _sizes(params: Mapping):
        dim, index = int(params["dim"]), int(params["index"])
        if dim <= 0 or index < 0:
            raise ConfigError(f"token_side: dim {dim}, index {index}")
        return dim, index

    @classmethod
    def tensors(cls, params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        dim, _ = cls._sizes(params)
        return {"gate.weight": TensorDecl((dim, hidden)), "proj.weight": TensorDecl((hidden, dim)),
                "norm.weight": TensorDecl((hidden,), init="norm")}

    @classmethod
    def resident(cls, params: Mapping, hidden: int) -> Dict[str, Resident]:
        dim, _ = cls._sizes(params)
        return {"gate.weight": Resident((dim, hidden), pieces=(Piece("gate.weight"),)),
                "proj.weight": Resident((hidden, dim), pieces=(Piece("proj.weight"),)),
                "norm.gain": Resident((hidden,), torch.float32, (Piece("norm.weight"),))}

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.dim, self.index = self._sizes(params)
        self.eps = float(params["norm_eps"])
        self.w_gate = rt.cast_matrix(weights["gate.weight"])
        self.w_proj = rt.cast_matrix(weights["proj.weight"])
        self.gain = weights["norm.gain"]

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """``x``: the stream's rows in the activation type; returns y (before its norm)."""
        rows = ctx.memo.get("token_side")
        if rows is None or rows.shape[1] < (self.index + 1) * self.dim:
            raise ValueError("token_side: the embedding left no (or too narrow) rows for the layers")
        t = self.rt.linear(x, self.w_gate)
        self.rt.flush()
        g = native.gelu_gate_rows(t, rows, self.index * self.dim, torch.empty_like(t))
        return self.rt.linear(g, self.w_proj)


register_mixer("side_by_side", SideBySide)
register_tail("token_side", TokenSide)
