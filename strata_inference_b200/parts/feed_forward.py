"""``gated_mlp``: the dense gated feed-forward: down(act(gate(x)) * up(x)), no biases; act is the
tanh-GELU or SiLU (``activation``: "gelu_pytorch_tanh", "silu").

Reference: src/model/layer.rs:696-710 (two products, the gated activation,
the down product), src/backend/cpu.rs:1190-1199 (tanh-GELU).  The gate and up
matrices are kept as ONE matrix so that one product makes both halves; when
the intermediate size allows it their rows are interleaved in groups of 8
(8 gate rows, then the 8 matching up rows), which puts a gate value and its
up value into the same thread of the weight-streaming kernel, whose epilogue
then writes act(gate) * up directly.

``mlp``: the feed-forward without a gate, down(act(up(x))), no biases; act is the square of
relu (``activation``: "relu_squared"), the tanh-GELU or SiLU.

``clipped_gated_mlp``: the dense form of the routed experts' clipped activation,
down(g * sigmoid(alpha g) * (u + 1)) with g = min(gate x, limit), u = clamp(up x, +-limit);
parameters ``intermediate_size``, ``limit``, ``alpha`` (default 1.702).

``routed_experts``: many small gated feed-forwards of which every row uses ``top``.  Parameters:
``experts``, ``top``, ``intermediate_size``, ``limit``, ``alpha`` (default 1.702), ``router_bias``,
``shared`` (None, or {"intermediate_size", "limit"}: one more expert that every row uses).
    expert(x) = down(g * sigmoid(alpha g) * (u + 1)),  g = min(gate x, limit),  u = clamp(up x, +-limit)
    z = router x + bias (32-bit);  the ``top`` largest z choose the experts (ties: the lower index),
    their weights are the softmax over the chosen z alone;  y = sum_k p_k expert_k(x) + shared(x)
``score`` "sigmoid" (default "softmax_top"): a chosen expert's weight is the sigmoid of its own
logit, not normalized over the chosen.  ``form`` "plain_gelu" (default "clipped_gated"): an
expert, and the shared one, is down(gelu(up x)) with the exact gelu and no gate matrix, and a
row's weight multiplies what ENTERS its expert, y = sum_k expert_k(p_k x) + shared(x); as the
experts have no biases, up(p x) = p up(x), so the weight is applied in 32-bit to the up
product's output in front of the gelu.
Few rows, and every recorded step: each (row, expert) pair streams its expert's matrices
(csrc/routed.cu routed_rows).  Many rows: the pairs are sorted by expert on the device into a
layout [experts, most rows of any expert, width] (that one number is read on the host; a recorded
step takes its number of rows instead and reads nothing) and all experts run as two batched library
products around one activation launch.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..config.spec import ConfigError
from ..kernels import native
from ..weights.arena import Piece, Resident
from ..weights.loader import TensorDecl
from .registry import register_feed_forward

from typing import Optional

# activation of the gate -> (elementwise kernel's code, fused epilogue of the products or None)
_ACTIVATIONS = {"gelu_pytorch_tanh": (native.ACT_GELU_TANH, native.EPI_GEGLU),
                "silu": (native.ACT_SILU, native.EPI_SWIGLU)}
_GROUP = 8


class GatedMLP:
    chain_safe = True      # deferred results are read by this runtime's and native's launchers only
    captures_prompts = True   # row-wise: a recorded step of prompts may be replayed for others

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        inter = params["intermediate_size"]
        return {
            "gate_proj.weight": TensorDecl((inter, hidden)),
            "up_proj.weight": TensorDecl((inter, hidden)),
            "down_proj.weight": TensorDecl((hidden, inter)),
        }

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        """Gate and up as ONE matrix: runs of 8 gate rows followed by the 8 matching up
        rows when the intermediate size is a multiple of 8, else all gates, then all ups."""
        inter = int(params["intermediate_size"])
        if inter % _GROUP == 0:
            pieces = (Piece("gate_proj.weight", 0, _GROUP, 2 * _GROUP),
                      Piece("up_proj.weight", _GROUP, _GROUP, 2 * _GROUP))
        else:
            pieces = (Piece("gate_proj.weight", 0), Piece("up_proj.weight", inter))
        return {
            "gate_up_proj.weight": Resident((2 * inter, hidden), pieces=pieces),
            "down_proj.weight": Resident((hidden, inter), pieces=(Piece("down_proj.weight"),)),
        }

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.inter = int(params["intermediate_size"])
        act = params.get("activation", "gelu_pytorch_tanh")
        if act not in _ACTIVATIONS:
            raise ConfigError(f"gated_mlp: activation {act!r} is not supported; "
                              f"known: {', '.join(_ACTIVATIONS)}")
        self.act, self.epilogue = _ACTIVATIONS[act]
        self.group = _GROUP if self.inter % _GROUP == 0 else 0
        self.w_gate_up = rt.cast_matrix(weights["gate_up_proj.weight"])
        self.w_down = rt.cast_matrix(weights["down_proj.weight"])

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        rt = self.rt
        R = x.shape[0]
        if (self.epilogue is not None and self.group == _GROUP and x.dtype == torch.bfloat16
                and x.shape[1] % 8 == 0
                and (R <= rt.skinny_max_rows or R > rt.gated_gemm_min_rows
                     or (rt.chain is not None and R <= rt.chain_max_rows
                         and self.epilogue == native.EPI_GEGLU))):
            t = rt.linear(x, self.w_gate_up, epilogue=self.epilogue)
        else:
            gate_up = rt.linear(x, self.w_gate_up)
            t = torch.empty((R, self.inter), dtype=x.dtype, device=x.device)
            native.gelu_mul(gate_up, t, self.group, self.act)
        return rt.linear(t, self.w_down)


_PLAIN_ACTIVATIONS = {"relu_squared": native.ACT_RELU_SQUARED, "gelu_pytorch_tanh": native.ACT_GELU_TANH,
                      "silu": native.ACT_SILU}


class PlainMLP:
    captures_prompts = True   # row-wise: a recorded step of prompts may be replayed for others

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        inter = params["intermediate_size"]
        return {"up_proj.weight": TensorDecl((inter, hidden)),
                "down_proj.weight": TensorDecl((hidden, inter))}

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        inter = int(params["intermediate_size"])
        return {"up_proj.weight": Resident((inter, hidden), pieces=(Piece("up_proj.weight"),)),
                "down_proj.weight": Resident((hidden, inter), pieces=(Piece("down_proj.weight"),))}

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.inter = int(params["intermediate_size"])
        act = params.get("activation", "relu_squared")
        if act not in _PLAIN_ACTIVATIONS:
            raise ConfigError(f"mlp: activation {act!r} is not supported; "
                              f"known: {', '.join(_PLAIN_ACTIVATIONS)}")
        self.act = _PLAIN_ACTIVATIONS[act]
        self.w_up = rt.cast_matrix(weights["up_proj.weight"])
        self.w_down = rt.cast_matrix(weights["down_proj.weight"])

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        if self.act == native.ACT_RELU_SQUARED:
            # (the products have this activation as an epilogue; where a library product is
            # taken the runtime applies it behind)
            up = self.rt.linear(x, self.w_up, epilogue=native.EPI_RELU2)
        else:
            up = self.rt.linear(x, self.w_up)
            native.activate(up, up, self.act)
        return self.rt.linear(up, self.w_down)


class ClippedGatedMLP:
    captures_prompts = True   # row-wise: a recorded step of prompts may be replayed for others

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        inter = params["intermediate_size"]
        return {"gate_proj.weight": TensorDecl((inter, hidden)),
                "up_proj.weight": TensorDecl((inter, hidden)),
                "down_proj.weight": TensorDecl((hidden, inter))}

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        """Gate and up as ONE matrix, laid out as the gated feed-forward's: runs of 8 gate rows
        followed by the 8 matching up rows when the intermediate size is a multiple of 8 (the
        products' clipped epilogue then writes the activated middle itself), else all gates,
        then all ups."""
        inter = int(params["intermediate_size"])
        if inter % _GROUP == 0:
            pieces = (Piece("gate_proj.weight", 0, _GROUP, 2 * _GROUP),
                      Piece("up_proj.weight", _GROUP, _GROUP, 2 * _GROUP))
        else:
            pieces = (Piece("gate_proj.weight", 0), Piece("up_proj.weight", inter))
        return {"gate_up_proj.weight": Resident((2 * inter, hidden), pieces=pieces),
                "down_proj.weight": Resident((hidden, inter), pieces=(Piece("down_proj.weight"),))}

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.inter = int(params["intermediate_size"])
        self.limit = float(params["limit"])
        self.alpha = float(params.get("alpha", 1.702))
        if self.inter <= 0 or self.limit <= 0:
            raise ConfigError(f"clipped_gated_mlp: intermediate_size {self.inter}, limit {self.limit}")
        self.w_gate_up = rt.cast_matrix(weights["gate_up_proj.weight"])
        self.w_down = rt.cast_matrix(weights["down_proj.weight"])

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        rt, R = self.rt, x.shape[0]
        group = _GROUP if self.inter % _GROUP == 0 else 0
        # (the products' epilogue has the design's constant 1.702 built in)
        if (group and self.alpha == 1.702 and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                and (R <= rt.skinny_max_rows or R > rt.gated_gemm_min_rows)):
            mid = rt.linear(x, self.w_gate_up, epilogue=native.EPI_CLIPPED, cap=self.limit)
        else:
            gu = rt.linear(x, self.w_gate_up)
            rt.flush()
            mid = torch.empty((R, self.inter), dtype=x.dtype, device=x.device)
            native.expert_activate(gu, mid, None, self.limit, self.alpha, native.FORM_CLIPPED_GATED, group)
        return rt.linear(mid, self.w_down)


_FORMS = {"clipped_gated": native.FORM_CLIPPED_GATED, "plain_gelu": native.FORM_PLAIN_GELU}
_SCORES = {"softmax_top": native.SCORE_SOFTMAX_TOP, "sigmoid": native.SCORE_SIGMOID}


class RoutedExperts:
    captures_prompts = True   # a recorded step reads the choices on the device only
    reads_sizes_on_host = True   # a launched step of many rows reads how many rows chose each expert

    @staticmethod
    def _sizes(params: Mapping):
        E, top, ff = int(params["experts"]), int(params["top"]), int(params["intermediate_size"])
        if E <= 0 or not 0 < top <= min(E, 32) or ff <= 0:
            raise ConfigError(f"routed_experts: {E} experts of {ff}, {top} a row (at most 32)")
        shared = params.get("shared") or None
        sff = int(shared["intermediate_size"]) if shared else 0
        if shared and sff <= 0:
            raise ConfigError("routed_experts: the shared expert's intermediate_size must be positive")
        return E, top, ff, sff

    @staticmethod
    def _form(params: Mapping) -> int:
        form, score = params.get("form", "clipped_gated"), params.get("score", "softmax_top")
        if form not in _FORMS or score not in _SCORES:
            raise ConfigError(f"routed_experts: form {form!r} and score {score!r}; known: "
                              f"{', '.join(_FORMS)}; {', '.join(_SCORES)}")
        return _FORMS[form]

    @classmethod
    def tensors(cls, params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        E, top, ff, sff = cls._sizes(params)
        out = {"router.weight": TensorDecl((E, hidden))}
        if params.get("router_bias", True):
            out["router.bias"] = TensorDecl((E,), init="norm")
        gated = cls._form(params) == native.FORM_CLIPPED_GATED
        for e in range(E):
            if gated:
                out[f"experts.{e}.gate_proj.weight"] = TensorDecl((ff, hidden))
            out[f"experts.{e}.up_proj.weight"] = TensorDecl((ff, hidden))
            out[f"experts.{e}.down_proj.weight"] = TensorDecl((hidden, ff))
        if sff:
            if gated:
                out["shared.gate_proj.weight"] = TensorDecl((sff, hidden))
            out["shared.up_proj.weight"] = TensorDecl((sff, hidden))
            out["shared.down_proj.weight"] = TensorDecl((hidden, sff))
        return out

    @classmethod
    def resident(cls, params: Mapping, hidden: int) -> Dict[str, Resident]:
        """All experts' gate and up matrices as one [experts, 2 ff, hidden] (an expert's gate
        rows, then its up rows; experts without a gate: [experts, ff, hidden], the up rows
        alone) and their down matrices as one [experts, hidden, ff]; the router's matrix 32-bit."""
        E, top, ff, sff = cls._sizes(params)
        gated = cls._form(params) == native.FORM_CLIPPED_GATED
        per = 2 if gated else 1
        gu, down = [], []
        for e in range(E):
            if gated:
                gu.append(Piece(f"experts.{e}.gate_proj.weight", e * 2 * ff))
            gu.append(Piece(f"experts.{e}.up_proj.weight", e * per * ff + (ff if gated else 0)))
            down.append(Piece(f"experts.{e}.down_proj.weight", e * hidden))
        out = {"router.weight": Resident((E, hidden), torch.float32, (Piece("router.weight"),)),
               "experts.gate_up.weight": Resident((E * per * ff, hidden), pieces=tuple(gu)),
               "experts.down.weight": Resident((E * hidden, ff), pieces=tuple(down))}
        if params.get("router_bias", True):
            out["router.bias"] = Resident((E,), torch.float32, (Piece("router.bias"),))
        if sff and not gated:
            out["shared.gate_up.weight"] = Resident((sff, hidden), pieces=(Piece("shared.up_proj.weight"),))
        elif sff:
            out["shared.gate_up.weight"] = Resident((2 * sff, hidden), pieces=(
                Piece("shared.gate_proj.weight", 0), Piece("shared.up_proj.weight", sff)))
        if sff:
            out["shared.down.weight"] = Resident((hidden, sff), pieces=(Piece("shared.down_proj.weight"),))
        return out

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.hidden = hidden
        self.E, self.top, self.ff, self.sff = self._sizes(params)
        self.form = self._form(params)
        self.score = _SCORES[params.get("score", "softmax_top")]
        self.plain = self.form == native.FORM_PLAIN_GELU
        self.per = 1 if self.plain else 2          # matrix rows per middle column
        self.limit = 0.0 if self.plain else float(params["limit"])
        self.alpha = float(params.get("alpha", 1.702))
        self.w_router = weights["router.weight"]
        self.b_router = weights.get("router.bias")
        self.w_gu = rt.cast_matrix(weights["experts.gate_up.weight"]).view(self.E, self.per * self.ff, hidden)
        self.w_down = rt.cast_matrix(weights["experts.down.weight"]).view(self.E, hidden, self.ff)
        self.shared_limit = float(params["shared"]["limit"]) if self.sff and not self.plain else 0.0
        self.w_sgu = rt.cast_matrix(weights["shared.gate_up.weight"]) if self.sff else None
        self.w_sdown = rt.cast_matrix(weights["shared.down.weight"]) if self.sff else None
        # up to this many rows every (row, expert) pair streams its own expert's matrices
        self.pair_rows = 32

    def choose(self, x: torch.Tensor):
        """(ids int32 [rows, top], weights 32-bit [rows, top]) of the rows' experts."""
        R = x.shape[0]
        if R <= self.pair_rows and (self.hidden + self.E + 4) * 4 <= 48 * 1024:
            ids = torch.empty((R, self.top), dtype=torch.int32, device=x.device)
            p = torch.empty((R, self.top), dtype=torch.float32, device=x.device)
            native.router_rows(x, self.w_router, self.b_router, ids, p, self.score)
            return ids, p
        x32 = x if x.dtype == torch.float32 else native.cast_rows(
            x, torch.empty(x.shape, dtype=torch.float32, device=x.device))
        with native.profile_region("library product (router, 32-bit)", (R + self.E) * self.hidden * 4,
                                   2.0 * R * self.E * self.hidden):
            z = torch.matmul(x32, self.w_router.t())
        ids = torch.empty((R, self.top), dtype=torch.int32, device=x.device)
        p = torch.empty((R, self.top), dtype=torch.float32, device=x.device)
        native.router_topk(z, self.b_router, ids, p, self.score)
        return ids, p

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        rt, R = self.rt, x.shape[0]
        rt.flush()
        ids, p = self.choose(x)
        base: Optional[torch.Tensor] = None
        if self.sff and self.plain:
            # (the gelu is an epilogue of the up product where a hand-written product runs)
            base = rt.linear(rt.linear(x, self.w_sgu, epilogue=native.EPI_GELU), self.w_sdown)
        elif self.sff:
            gu = rt.linear(x, self.w_sgu)
            mid = torch.empty((R, self.sff), dtype=x.dtype, device=x.device)
            native.expert_activate(gu, mid, None, self.shared_limit, self.alpha, self.form)
            base = rt.linear(mid, self.w_sdown)
        out = torch.empty((R, self.hidden), dtype=x.dtype, device=x.device)
        # (the streamed kernels keep a row and its `top` middles in shared memory)
        streams = self.hidden * 4 <= 48 * 1024 and self.top * self.ff * 4 <= 48 * 1024
        if R <= self.pair_rows and streams and R * self.top < 65536:
            return native.routed_rows(x, self.w_gu, self.w_down, ids, p, base, out, self.limit, self.alpha,
                                      self.form)
        # The pairs sorted by expert and laid out [experts, most, width] with `most` the largest
        # number of rows any expert got (the one number read on the host; rows behind an
        # expert's own are zeros): all experts run as ONE batched library product for gate and
        # up, one activation launch and one batched product for down.  `where[r, k]`: the
        # place of row r's k-th pair in that layout.
        # A recorded step reads nothing on the host: every expert gets room for all the step's
        # rows (an expert is chosen at most once a row).  For the 33 to 64 rows of such a step
        # that is a few products' worth of zeros on the tensor cores, against the streamed
        # kernels' sums on the CUDA cores (64 rows of 4 experts each: 558 us a layer).
        E, top, W = self.E, self.top, self.hidden
        flat = ids.view(-1).to(torch.int64)
        order = torch.argsort(flat, stable=True)
        counts = torch.zeros(E, dtype=torch.int64, device=x.device).index_add_(
            0, flat, torch.ones_like(flat))
        most = R if ctx.graph_capture else int(counts.max().item())
        most = -(-most // 8) * 8
        by_expert = flat[order]
        place = by_expert * most + (torch.arange(order.numel(), device=x.device)
                                    - (torch.cumsum(counts, 0) - counts)[by_expert])
        xs = torch.zeros((E * most, W), dtype=x.dtype, device=x.device)
        xs.index_copy_(0, place, x.index_select(0, torch.div(order, top, rounding_mode="floor")))
        where = torch.empty(order.numel(), dtype=torch.int32, device=x.device)
        where[order] = place.to(torch.int32)
        esz = x.element_size()
        with native.profile_region(f"library product (experts, {E} x {most} rows, gate and up)",
                                   (E * most * (W + self.per * self.ff) + self.w_gu.numel()) * esz,
                                   2.0 * E * most * W * self.per * self.ff):
            gu = torch.bmm(xs.view(E, most, W), self.w_gu.transpose(1, 2))
        mid = torch.empty((E * most, self.ff), dtype=x.dtype, device=x.device)
        row_weight = None
        if self.plain:
            # a pair's weight enters its expert: on the sorted rows, in front of the gelu
            row_weight = torch.zeros(E * most, dtype=torch.float32, device=x.device)
            row_weight.index_copy_(0, place, p.view(-1).index_select(0, order))
        native.expert_activate(gu.view(E * most, self.per * self.ff), mid, row_weight, self.limit, self.alpha,
                               self.form)
        with native.profile_region(f"library product (experts, {E} x {most} rows, down)",
                                   (E * most * (W + self.ff) + self.w_down.numel()) * esz,
                                   2.0 * E * most * W * self.ff):
            ys = torch.bmm(mid.view(E, most, self.ff), self.w_down.transpose(1, 2))
        return native.routed_combine(ys.view(E * most, W), where.view(R, top), None if self.plain else p,
                                     base, out)


register_feed_forward("gated_mlp", GatedMLP)
register_feed_forward("mlp", PlainMLP)
register_feed_forward("clipped_gated_mlp", ClippedGatedMLP)
register_feed_forward("routed_experts", RoutedExperts)
