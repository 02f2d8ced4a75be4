"""Mixers that carry a matrix per head from token to token instead of keys and values.

Both keep their state in the cache's per-slot state (``StateNeed``, 32-bit, zeroed when a
slot is taken), read and write it by the step's device tensors only (so their steps can be
recorded and replayed) and take any split of a sequence into steps: a step continues from
what the slot holds.  One product makes every projection of the mixer's input; what enters
the recurrence besides the projections (unit norms, decays, gates, the state) is 32-bit
(csrc/recurrent.cu).

``gated_delta``  the gated delta rule.  Parameters: ``num_heads`` H (value heads),
    ``num_kv_heads`` G (q and k heads; value head h reads q/k head h // (H / G)),
    ``head_dim`` (q, k), ``value_dim``, ``conv_taps``, ``norm_eps``.
    q, k, v pass a causal convolution over the last ``conv_taps`` tokens per channel (no
    bias, zeros before the start) and SiLU; q and k become unit vectors per head
    (x / sqrt(sum x^2 + 1e-6)), q times head_dim^-1/2; beta = sigmoid(b_proj x);
    decay = exp(-exp(A_log) * softplus(a_proj x + dt_bias)); per head
        S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    then o / rms(o) * norm.weight (one per value dimension) * silu(g_proj x), and o_proj.
    State: the matrices and the convolutions' last ``conv_taps - 1`` inputs.

``matrix_memory``  the matrix memory with exponential gates (mLSTM).  Parameters:
    ``num_heads``, ``head_dim``, ``value_dim``, ``gate_cap`` c, ``norm_eps``.
    i = c tanh((i_proj x + bias) / c);  f = log sigmoid(c tanh((f_proj x + bias) / c));
        m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise with k
        o = S^T q / (max(|n . q|, e^-m') + 1e-6),      q = q_proj x * head_dim^-1/2
    then per head o / rms(o), times norm.weight (one per head and dimension) and
    sigmoid(g_proj x), and o_proj.  State: S, n and m (m starts at 0).

``retention``  linear attention with one fixed decay per head and no softmax or denominator.
    Parameters: ``num_heads``, ``head_dim``, ``value_dim``, ``decay`` (one number per head),
    ``key_scale`` (on k, after the rotation), ``norm_eps``, ``position`` (a PartSpec of a
    rotary position part with half-split pairs, or "none").
        q, k rotated by the token's position;  k <- key_scale k
        S <- decay_h S + k v^T;  o = S^T q
    then per head o / rms(o) (no weight), times silu(g_proj x), and o_proj.  State: S.
    Options, each with the behaviour above as its default: ``activation`` "silu" (q, k and v
    pass SiLU before anything else; lightning attention feeds its recurrence so);
    ``norm`` "joint" (the heads side by side are divided by ONE root mean square instead of
    one per head); ``norm_weight`` True (a stored ``norm.weight``, one per head and column,
    multiplies the normed output); ``gate`` "sigmoid" (instead of SiLU).

``state_space``  the selective state-space layer in its dual (matrix) form.  Parameters:
    ``num_heads`` H, ``value_dim`` P (a head's channels; inner = H P), ``state_dim`` N,
    ``groups`` G (head h reads B and C of group h // (H / G)), ``conv_taps``, ``norm_groups``,
    ``norm_eps``.  One product makes z | x | B | C | dt; x, B and C pass a causal convolution
    per channel with a bias and SiLU;
        dt = softplus(dt + dt_bias);  S <- exp(-exp(A_log_h) dt) S + dt B x^T;  y = S^T C + D_h x
    then y * silu(z), divided by its root mean square in ``norm_groups`` equal parts, times
    norm.weight, and o_proj.  State: S (N x P per head) and the convolution's last
    ``conv_taps - 1`` inputs.

``general_delta``  the delta rule with a decay and a removal rate per key channel.
    Parameters: ``num_heads``, ``head_dim`` d (keys, values and the read-out vector alike),
    ``decay_rank`` (the width of the decay's two-matrix path), ``norm_eps``.
        w = exp(-e^-1/2 sigmoid(w2 tanh(w1 x) + w0));  a = sigmoid(a_proj x + bias)
        u = k / sqrt(sum k^2 + 1e-6);  S <- diag(w) S - (a u)(u^T S) + k v^T;  o = S^T r
    then per head o / rms(o), times norm.weight (one per head and dimension) and
    sigmoid(g_proj x), and o_proj.  State: S (d x d per head).
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.paged import CacheNeed, StateNeed
from ..config.spec import ConfigError, PartSpec
from ..kernels import native
from ..weights.arena import Piece, Resident
from ..weights.loader import TensorDecl
from .registry import part_class, register_mixer


def _pieces(rows):
    """Pieces stacked in the given order: [(stored name, rows)] -> (pieces, total rows)."""
    out, at = [], 0
    for name, n in rows:
        out.append(Piece(name, at))
        at += n
    return tuple(out), at


def _round4(n: int) -> int:
    return -(-n // 4) * 4


class GatedDeltaRule:
    captures_prompts = True      # sequences, slots and counts are read on the device only

    @staticmethod
    def _sizes(params: Mapping):
        H, G = int(params["num_heads"]), int(params["num_kv_heads"])
        kd, vd, taps = int(params["head_dim"]), int(params["value_dim"]), int(params["conv_taps"])
        if H <= 0 or G <= 0 or H % G:
            raise ConfigError(f"gated_delta: {H} heads cannot share {G} q/k heads")
        if not 0 < kd <= 512 or vd <= 0 or not 1 <= taps <= 64:
            raise ConfigError(f"gated_delta: head_dim {kd} (at most 512), value_dim {vd}, "
                              f"{taps} taps (1 to 64)")
        return H, G, kd, vd, taps

    @classmethod
    def _in_rows(cls, params: Mapping):
        H, G, kd, vd, _ = cls._sizes(params)
        return [("q_proj.weight", G * kd), ("k_proj.weight", G * kd), ("v_proj.weight", H * vd),
                ("g_proj.weight", H * vd), ("b_proj.weight", H), ("a_proj.weight", H)]

    @classmethod
    def tensors(cls, params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        H, G, kd, vd, taps = cls._sizes(params)
        out = {name: TensorDecl((n, hidden)) for name, n in cls._in_rows(params)}
        out.update({
            "q_conv.weight": TensorDecl((G * kd, taps), init="norm"),
            "k_conv.weight": TensorDecl((G * kd, taps), init="norm"),
            "v_conv.weight": TensorDecl((H * vd, taps), init="norm"),
            "A_log": TensorDecl((H,), init="norm"),
            "dt_bias": TensorDecl((H,), init="norm"),
            "norm.weight": TensorDecl((vd,), init="norm"),
            "o_proj.weight": TensorDecl((hidden, H * vd)),
        })
        return out

    @classmethod
    def resident(cls, params: Mapping, hidden: int) -> Dict[str, Resident]:
        H, G, kd, vd, taps = cls._sizes(params)
        pieces, n_in = _pieces(cls._in_rows(params))
        conv, channels = _pieces([("q_conv.weight", G * kd), ("k_conv.weight", G * kd),
                                  ("v_conv.weight", H * vd)])
        return {
            "in_proj.weight": Resident((n_in, hidden), pieces=pieces),
            "conv.weight": Resident((channels, taps), torch.float32, conv),
            "A_log": Resident((H,), torch.float32, (Piece("A_log"),)),
            "dt_bias": Resident((H,), torch.float32, (Piece("dt_bias"),)),
            "norm.gain": Resident((vd,), torch.float32, (Piece("norm.weight"),)),
            "o_proj.weight": Resident((hidden, H * vd), pieces=(Piece("o_proj.weight"),)),
        }

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.H, self.G, self.kd, self.vd, self.taps = self._sizes(params)
        self.eps = float(params["norm_eps"])
        self.channels = 2 * self.G * self.kd + self.H * self.vd
        self.matrices = self.H * self.vd * self.kd       # floats of a slot's state before the history
        self.w_in = rt.cast_matrix(weights["in_proj.weight"])
        self.w_o = rt.cast_matrix(weights["o_proj.weight"])
        self.conv_w = weights["conv.weight"]
        self.a_log, self.dt_bias = weights["A_log"], weights["dt_bias"]
        self.norm_gain = weights["norm.gain"]

    def cache_need(self) -> Optional[CacheNeed]:
        # (whole groups of 4 floats, so that every slot's state begins on a 16-byte boundary)
        return CacheNeed(state=StateNeed((_round4(self.matrices + (self.taps - 1) * self.channels),)))

    def forward(self, x: torch.Tensor, ctx, entry: int, cache_entry: int,
                owns_cache: bool) -> torch.Tensor:
        if not owns_cache:
            raise ValueError("gated_delta: a recurrent state cannot be lent to another run")
        rt, H, G, kd, vd = self.rt, self.H, self.G, self.kd, self.vd
        R = x.shape[0]
        state = ctx.state(cache_entry)
        proj = rt.linear(x, self.w_in)
        f32 = dict(dtype=torch.float32, device=x.device)
        qn, kn = torch.empty((R, G * kd), **f32), torch.empty((R, G * kd), **f32)
        vc = torch.empty((R, H * vd), **f32)
        beta, decay = torch.empty((R, H), **f32), torch.empty((R, H), **f32)
        native.delta_prepare(proj, self.conv_w, self.a_log, self.dt_bias, state, self.matrices,
                             qn, kn, vc, beta, decay, ctx, H, G, kd, vd, self.taps)
        o = torch.empty((R, H * vd), **f32)
        native.delta_scan(qn, kn, vc, decay, beta, state, o, ctx, H, G, kd, vd)
        y = torch.empty((R, H * vd), dtype=proj.dtype, device=x.device)
        gate = proj[:, self.channels:self.channels + H * vd]
        native.head_norm_gate(o, None, self.norm_gain, gate, y, H, vd, self.eps, native.GATE_SILU)
        return rt.linear(y, self.w_o)


class MatrixMemory:
    captures_prompts = True      # sequences, slots and counts are read on the device only

    @staticmethod
    def _sizes(params: Mapping):
        H, kd, vd = int(params["num_heads"]), int(params["head_dim"]), int(params["value_dim"])
        if H <= 0 or not 0 < kd <= 512 or vd <= 0:
            raise ConfigError(f"matrix_memory: {H} heads, head_dim {kd} (at most 512), value_dim {vd}")
        return H, kd, vd

    @classmethod
    def _in_rows(cls, params: Mapping):
        H, kd, vd = cls._sizes(params)
        return [("q_proj.weight", H * kd), ("k_proj.weight", H * kd), ("v_proj.weight", H * vd),
                ("g_proj.weight", H * vd), ("i_proj.weight", H), ("f_proj.weight", H)]

    @classmethod
    def tensors(cls, params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        H, kd, vd = cls._sizes(params)
        out = {name: TensorDecl((n, hidden)) for name, n in cls._in_rows(params)}
        out.update({
            "i_proj.bias": TensorDecl((H,), init="norm"),
            "f_proj.bias": TensorDecl((H,), init="norm"),
            "norm.weight": TensorDecl((H * vd,), init="norm"),
            "o_proj.weight": TensorDecl((hidden, H * vd)),
        })
        return out

    @classmethod
    def resident(cls, params: Mapping, hidden: int) -> Dict[str, Resident]:
        H, kd, vd = cls._sizes(params)
        pieces, n_in = _pieces(cls._in_rows(params))
        return {
            "in_proj.weight": Resident((n_in, hidden), pieces=pieces),
            "i_proj.bias": Resident((H,), torch.float32, (Piece("i_proj.bias"),)),
            "f_proj.bias": Resident((H,), torch.float32, (Piece("f_proj.bias"),)),
            "norm.gain": Resident((H * vd,), torch.float32, (Piece("norm.weight"),)),
            "o_proj.weight": Resident((hidden, H * vd), pieces=(Piece("o_proj.weight"),)),
        }

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.H, self.kd, self.vd = self._sizes(params)
        self.eps = float(params["norm_eps"])
        self.cap = float(params["gate_cap"])
        if self.cap <= 0:
            raise ConfigError(f"matrix_memory: gate_cap {self.cap} must be positive")
        self.w_in = rt.cast_matrix(weights["in_proj.weight"])
        self.w_o = rt.cast_matrix(weights["o_proj.weight"])
        self.bias_i, self.bias_f = weights["i_proj.bias"], weights["f_proj.bias"]
        self.norm_gain = weights["norm.gain"]

    def cache_need(self) -> Optional[CacheNeed]:
        # S with n as one more column, then the running maxima
        return CacheNeed(state=StateNeed((_round4(self.H * (self.vd + 1) * self.kd + self.H),)))

    def forward(self, x: torch.Tensor, ctx, entry: int, cache_entry: int,
                owns_cache: bool) -> torch.Tensor:
        if not owns_cache:
            raise ValueError("matrix_memory: a recurrent state cannot be lent to another run")
        rt, H, kd, vd = self.rt, self.H, self.kd, self.vd
        R = x.shape[0]
        state = ctx.state(cache_entry)
        proj = rt.linear(x, self.w_in)
        o = torch.empty((R, H * (vd + 1)), dtype=torch.float32, device=x.device)
        m = torch.empty((R, H), dtype=torch.float32, device=x.device)
        native.memory_scan(proj, self.bias_i, self.bias_f, self.cap, state, o, m, ctx, H, kd, vd)
        y = torch.empty((R, H * vd), dtype=proj.dtype, device=x.device)
        gate = proj[:, 2 * H * kd + H * vd:2 * H * kd + 2 * H * vd]
        native.head_norm_gate(o, m, self.norm_gain, gate, y, H, vd, self.eps, native.GATE_SIGMOID)
        return rt.linear(y, self.w_o)


class Retention:
    captures_prompts = True      # sequences, slots and counts are read on the device only

    @staticmethod
    def _sizes(params: Mapping):
        H, kd, vd = int(params["num_heads"]), int(params["head_dim"]), int(params["value_dim"])
        if H <= 0 or not 0 < kd <= 512 or vd <= 0:
            raise ConfigError(f"retention: {H} heads, head_dim {kd} (at most 512), value_dim {vd}")
        if len(params["decay"]) != H:
            raise ConfigError(f"retention: {len(params['decay'])} decays for {H} heads")
        return H, kd, vd

    @classmethod
    def _in_rows(cls, params: Mapping):
        H, kd, vd = cls._sizes(params)
        return [("q_proj.weight", H * kd), ("k_proj.weight", H * kd), ("v_proj.weight", H * vd),
                ("g_proj.weight", H * vd)]

    @classmethod
    def tensors(cls, params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        H, kd, vd = cls._sizes(params)
        out = {name: TensorDecl((n, hidden)) for name, n in cls._in_rows(params)}
        out["o_proj.weight"] = TensorDecl((hidden, H * vd))
        if params.get("norm_weight"):
            out["norm.weight"] = TensorDecl((H * vd,), init="norm")
        return out

    @classmethod
    def resident(cls, params: Mapping, hidden: int) -> Dict[str, Resident]:
        H, kd, vd = cls._sizes(params)
        pieces, n_in = _pieces(cls._in_rows(params))
        out = {"in_proj.weight": Resident((n_in, hidden), pieces=pieces),
               "o_proj.weight": Resident((hidden, H * vd), pieces=(Piece("o_proj.weight"),))}
        if params.get("norm_weight"):
            out["norm.gain"] = Resident((H * vd,), torch.float32, (Piece("norm.weight"),))
        return out

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.H, self.kd, self.vd = self._sizes(params)
        self.eps = float(params["norm_eps"])
        self.key_scale = float(params.get("key_scale", 1.0))
        # (64-bit numbers of the configuration, rounded once)
        self.decay = torch.tensor([float(d) for d in params["decay"]], dtype=torch.float64).to(
            torch.float32).to(rt.device)
        pos: PartSpec = params.get("position") or PartSpec("none", {})
        position = part_class("position", pos.kind)(pos.params, self.kd, {}, rt)
        if not hasattr(position, "rotary"):
            raise ConfigError("retention: the position part must offer rotary()")
        self.inv_freq, self.rot, style = position.rotary()
        if self.rot and style != native.ROPE_HALF_SPLIT:
            raise ConfigError("retention: q and k are rotated in half-split pairs")
        self.w_in = rt.cast_matrix(weights["in_proj.weight"])
        self.w_o = rt.cast_matrix(weights["o_proj.weight"])
        act, norm, gate = params.get("activation"), params.get("norm", "head"), params.get("gate", "silu")
        if act not in (None, "silu") or norm not in ("head", "joint") or gate not in ("silu", "sigmoid"):
            raise ConfigError(f"retention: activation {act!r}, norm {norm!r}, gate {gate!r}; known: "
                              f"None or 'silu', 'head' or 'joint', 'silu' or 'sigmoid'")
        self.silu_inputs = act == "silu"
        self.joint_norm = norm == "joint"
        self.gate_act = native.GATE_SIGMOID if gate == "sigmoid" else native.GATE_SILU
        self.norm_gain = weights.get("norm.gain")

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(state=StateNeed((_round4(self.H * self.vd * self.kd),)))

    def forward(self, x: torch.Tensor, ctx, entry: int, cache_entry: int,
                owns_cache: bool) -> torch.Tensor:
        if not owns_cache:
            raise ValueError("retention: a recurrent state cannot be lent to another run")
        rt, H, kd, vd = self.rt, self.H, self.kd, self.vd
        R = x.shape[0]
        state = ctx.state(cache_entry)
        proj = rt.linear(x, self.w_in)
        f32 = dict(dtype=torch.float32, device=x.device)
        qn, kn = torch.empty((R, H * kd), **f32), torch.empty((R, H * kd), **f32)
        vc = torch.empty((R, H * vd), **f32)
        native.retention_prepare(proj, self.inv_freq, self.rot, ctx.row_pos, qn, kn, vc, H, kd, vd,
                                 self.key_scale, self.silu_inputs)
        o = torch.empty((R, H * vd), **f32)
        native.retention_scan(qn, kn, vc, self.decay, state, o, ctx, H, kd, vd)
        y = torch.empty((R, H * vd), dtype=proj.dtype, device=x.device)
        gate = proj[:, 2 * H * kd + H * vd:2 * H * kd + 2 * H * vd]
        # (one root mean square over all heads: the row as a single head of heads * vd columns)
        heads, width = (1, H * vd) if self.joint_norm else (H, vd)
        native.head_norm_gate(o, None, self.norm_gain, gate, y, heads, width, self.eps, self.gate_act)
        return rt.linear(y, self.w_o)


class StateSpace:
    captures_prompts = True      # sequences, slots and counts are read on the device only

    @staticmethod
    def _sizes(params: Mapping):
        H, P, N = int(params["num_heads"]), int(params["value_dim"]), int(params["state_dim"])
        G, taps = int(params.get("groups") or 1), int(params["conv_taps"])
        parts = int(params.get("norm_groups") or 1)
        if H <= 0 or G <= 0 or H % G:
            raise ConfigError(f"state_space: {H} heads cannot share {G} groups")
        if not 0 < N <= 512 or P <= 0 or not 1 <= taps <= 64:
            raise ConfigError(f"state_space: state_dim {N} (at most 512), value_dim {P}, "
                              f"{taps} taps (1 to 64)")
        if parts <= 0 or (H * P) % parts:
            raise ConfigError(f"state_space: {H * P} channels cannot be normed in {parts} equal parts")
        return H, P, N, G, taps, parts

    @classmethod
    def tensors(cls, params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        H, P, N, G, taps, _ = cls._sizes(params)
        inner, channels = H * P, H * P + 2 * G * N
        return {
            "in_proj.weight": TensorDecl((inner + channels + H, hidden)),
            "conv.weight": TensorDecl((channels, taps), init="norm"),
            "conv.bias": TensorDecl((channels,), init="norm"),
            "dt_bias": TensorDecl((H,), init="norm"),
            "A_log": TensorDecl((H,), init="norm"),
            "D": TensorDecl((H,), init="norm"),
            "norm.weight": TensorDecl((inner,), init="norm"),
            "o_proj.weight": TensorDecl((hidden, inner)),
        }

    @classmethod
    def resident(cls, params: Mapping, hidden: int) -> Dict[str, Resident]:
        H, P, N, G, taps, _ = cls._sizes(params)
        inner, channels = H * P, H * P + 2 * G * N
        f32 = torch.float32
        return {
            "in_proj.weight": Resident((inner + channels + H, hidden), pieces=(Piece("in_proj.weight"),)),
            "conv.weight": Resident((channels, taps), f32, (Piece("conv.weight"),)),
            "conv.bias": Resident((channels,), f32, (Piece("conv.bias"),)),
            "dt_bias": Resident((H,), f32, (Piece("dt_bias"),)),
            "A_log": Resident((H,), f32, (Piece("A_log"),)),
            "D": Resident((H,), f32, (Piece("D"),)),
            "norm.gain": Resident((inner,), f32, (Piece("norm.weight"),)),
            "o_proj.weight": Resident((hidden, inner), pieces=(Piece("o_proj.weight"),)),
        }

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.H, self.P, self.N, self.G, self.taps, self.parts = self._sizes(params)
        self.eps = float(params["norm_eps"])
        self.inner = self.H * self.P
        self.channels = self.inner + 2 * self.G * self.N
        self.matrices = self.H * self.P * self.N       # floats of a slot's state before the history
        self.w_in = rt.cast_matrix(weights["in_proj.weight"])
        self.w_o = rt.cast_matrix(weights["o_proj.weight"])
        self.conv_w, self.conv_b = weights["conv.weight"], weights["conv.bias"]
        self.a_log, self.dt_bias, self.skip = weights["A_log"], weights["dt_bias"], weights["D"]
        self.norm_gain = weights["norm.gain"]

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(state=StateNeed((_round4(self.matrices + (self.taps - 1) * self.channels),)))

    def forward(self, x: torch.Tensor, ctx, entry: int, cache_entry: int,
                owns_cache: bool) -> torch.Tensor:
        if not owns_cache:
            raise ValueError("state_space: a recurrent state cannot be lent to another run")
        rt, H, P, N, G = self.rt, self.H, self.P, self.N, self.G
        R = x.shape[0]
        state = ctx.state(cache_entry)
        proj = rt.linear(x, self.w_in)
        rt.flush()
        f32 = dict(dtype=torch.float32, device=x.device)
        xbc = torch.empty((R, self.channels), **f32)
        keep, take = torch.empty((R, H), **f32), torch.empty((R, H), **f32)
        native.ssm_prepare(proj, self.conv_w, self.conv_b, self.a_log, self.dt_bias, state,
                           self.matrices, xbc, keep, take, ctx, H, self.inner, self.channels, self.taps)
        o = torch.empty((R, self.inner), **f32)
        native.gated_scan(xbc[:, self.inner + G * N:], xbc[:, self.inner:self.inner + G * N],
                          xbc[:, :self.inner], keep, take, state, o, ctx, H, G, N, P)
        y = torch.empty((R, self.inner), dtype=proj.dtype, device=x.device)
        native.ssm_finish(o, xbc, proj[:, :self.inner], self.skip, self.norm_gain, y, self.inner, P,
                          self.parts, self.eps)
        return rt.linear(y, self.w_o)


class GeneralDelta:
    captures_prompts = True      # sequences, slots and counts are read on the device only

    @staticmethod
    def _sizes(params: Mapping):
        H, d, rank = int(params["num_heads"]), int(params["head_dim"]), int(params["decay_rank"])
        if H <= 0 or not 0 < d <= 512 or rank <= 0:
            raise ConfigError(f"general_delta: {H} heads, head_dim {d} (at most 512), decay_rank {rank}")
        return H, d, rank

    @classmethod
    def _in_rows(cls, params: Mapping):
        H, d, _ = cls._sizes(params)
        return [("r_proj.weight", H * d), ("k_proj.weight", H * d), ("v_proj.weight", H * d),
                ("g_proj.weight", H * d), ("a_proj.weight", H * d)]

    @classmethod
    def tensors(cls, params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        H, d, rank = cls._sizes(params)
        out = {name: TensorDecl((n, hidden)) for name, n in cls._in_rows(params)}
        out.update({
            "a_proj.bias": TensorDecl((H * d,), init="norm"),
            "w1.weight": TensorDecl((rank, hidden)),
            "w2.weight": TensorDecl((H * d, rank)),
            "w0": TensorDecl((H * d,), init="norm"),
            "norm.weight": TensorDecl((H * d,), init="norm"),
            "o_proj.weight": TensorDecl((hidden, H * d)),
        })
        return out

    @classmethod
    def resident(cls, params: Mapping, hidden: int) -> Dict[str, Resident]:
        H, d, rank = cls._sizes(params)
        pieces, n_in = _pieces(cls._in_rows(params))
        f32 = torch.float32
        return {
            "in_proj.weight": Resident((n_in, hidden), pieces=pieces),
            "w1.weight": Resident((rank, hidden), pieces=(Piece("w1.weight"),)),
            "w2.weight": Resident((H * d, rank), pieces=(Piece("w2.weight"),)),
            "a_proj.bias": Resident((H * d,), f32, (Piece("a_proj.bias"),)),
            "w0": Resident((H * d,), f32, (Piece("w0"),)),
            "norm.gain": Resident((H * d,), f32, (Piece("norm.weight"),)),
            "o_proj.weight": Resident((hidden, H * d), pieces=(Piece("o_proj.weight"),)),
        }

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.H, self.d, self.rank = self._sizes(params)
        self.eps = float(params["norm_eps"])
        self.w_in = rt.cast_matrix(weights["in_proj.weight"])
        self.w1, self.w2 = rt.cast_matrix(weights["w1.weight"]), rt.cast_matrix(weights["w2.weight"])
        self.w_o = rt.cast_matrix(weights["o_proj.weight"])
        self.a_bias, self.w0 = weights["a_proj.bias"], weights["w0"]
        self.norm_gain = weights["norm.gain"]

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(state=StateNeed((_round4(self.H * self.d * self.d),)))

    def forward(self, x: torch.Tensor, ctx, entry: int, cache_entry: int,
                owns_cache: bool) -> torch.Tensor:
        if not owns_cache:
            raise ValueError("general_delta: a recurrent state cannot be lent to another run")
        rt, H, d = self.rt, self.H, self.d
        R, n = x.shape[0], self.H * self.d
        state = ctx.state(cache_entry)
        proj = rt.linear(x, self.w_in)
        low = rt.linear(x, self.w1)
        rt.flush()
        native.activate(low, low, native.ACT_TANH)
        decay_in = rt.linear(low, self.w2)
        rt.flush()
        prep = torch.empty((R, H, 6, d), dtype=torch.float32, device=x.device)
        native.gdelta_prepare(proj, 4 * n, decay_in, self.w0, self.a_bias, prep, H, d)
        o = torch.empty((R, n), dtype=torch.float32, device=x.device)
        native.gdelta_scan(prep, state, o, ctx, H, d)
        y = torch.empty((R, n), dtype=proj.dtype, device=x.device)
        native.head_norm_gate(o, None, self.norm_gain, proj[:, 3 * n:4 * n], y, H, d, self.eps,
                              native.GATE_SIGMOID)
        return rt.linear(y, self.w_o)


register_mixer("gated_delta", GatedDeltaRule)
register_mixer("retention", Retention)
register_mixer("matrix_memory", MatrixMemory)
register_mixer("state_space", StateSpace)
register_mixer("general_delta", GeneralDelta)
