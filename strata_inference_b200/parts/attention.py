"""The attention mixer: grouped-query attention over the paged cache.

Parameters (all from the PartSpec): ``num_heads``, ``num_kv_heads``,
``head_dim`` (heads x head_dim need not equal the hidden size),
``score_scale`` (the factor on q.k), ``logit_softcap`` (0: off), ``window``
(0: every earlier key is visible; W: the last W keys, the query's own
included) and ``position`` (a PartSpec of a position encoding).

Order of operations, as in the reference (src/model/layer.rs:1113-1161,
872-984): q, k, v projections (no bias); rotation of q and k; k and v
appended to the cache at the rows' positions; scores scaled, soft-capped,
masked; softmax; weighted sum of v; output projection.

A step whose sequences all begin at position 0 (prompts) attends over the
step's own k and v rows; any other step attends over the cache.  A run that
borrows another schedule entry's cache projects q only and reads that cache.

Fast paths inside this general part (each falls back to the general kernels
when its condition does not hold, with the same result): for at most 16
bfloat16 rows, a position part that offers ``rotary()`` with half-split pairs
over the WHOLE head lets the q|k|v product rotate and store in its own
epilogue (partial rotary or interleaved pairs take the product and then the
rotate-and-store kernel); prompts take the tcgen05 attention for head sizes
64/128/256 with at most two query heads per kv head, else the mma.sync
kernel, else the general one; single rows over the cache take the
bandwidth-tuned kernel for head sizes 64/128/256 and groups of 1, 2, 4 or 8.

Optional, each off unless its parameter is given (csrc/head_prepare.cu does them between
the projection and the attention kernel, in 32-bit):

``value_dim``   width of a value head where it differs from ``head_dim``.  The packed
                rows and the cache then hold heads of max(head_dim, value_dim) rounded up
                to 16, the narrower kind filled up with zeros, so every attention kernel
                serves them; the output is narrowed again before the output product.
``bias``        q, k and v have biases (``q_proj.bias`` ...).
``qk_norm``     {"eps": e}: q and k are divided by their root mean square per head and
                multiplied by ``q_norm.weight`` / ``k_norm.weight`` (one per dimension,
                shared by the heads), before the rotation.
``value_mix``   "first": this layer's values are also what later layers mix in;
                "mix": v <- (1 - l) v + l v_first with l = ``value_mix.weight`` (one number)
                and v_first the "first" layer's values of the same token; the mixed values
                are the ones cached.
``head_gate``   each head's output is multiplied by sigmoid(g_h), g = ``g_proj.weight`` x
                (one number per head, from the mixer's input), before the output product.
``pool``        P > 0 (with a ``window``): beside the window's tokens a row sees one key and one
                value for every block of P positions (bP .. bP + P - 1) that lies wholly before
                its window (bP + P - 1 <= position - window): the means of the block's keys
                and values as the cache holds them.  Tokens and blocks share one softmax.
                The cache keeps a cell per block (``KVNeed.pool``), written by the step that
                brings the block's last position (csrc/head_prepare.cu pool_store).

``chunk``       C > 0 (without a window): a row at position p sees the positions of its own
                chunk, C floor(p / C) .. p; chunks are counted from the sequence's position 0,
                however the sequence was cut into steps.
``sink``        True: one stored number per query head (``sink``) whose exponential joins the
                softmax's denominator; it has no key and no value and is not scaled.
``borrows_cache``  True: the layer has no key and value projections (no such tensors); its
                schedule entry names the run whose cached keys (rotated) and values it reads.
``lends_cache``  True: a later run reads this layer's keys and values; in a step of prompts the
                layer leaves its packed rows for that run, which then attends over them with
                the prompt kernel instead of row by row over the cache.

A chunked mask or a sink takes these kernels: bfloat16 prompts the tcgen05 prompt kernel, to
which every chunk of a prompt is a sequence of its own (rows of one chunk see nothing of
another, so a chunk's rows are a causal prompt; the rotation has been applied by position
before) and which takes the sink in its last division; rows over the cache the decode
kernel, whose first key is the start of the row's chunk and whose joins add the sink;
everything else (32-bit, shapes those two do not take, recorded prompt steps) the general
kernel.

Worked-on heads (any of the options from ``value_dim`` to ``pool``) are rotated in half-split or neighbouring pairs,
as the position part says, and are attended to by the general kernel when a window is set.
"""

from __future__ import annotations

import os
from typing import Dict, Mapping, Optional

import torch

from ..cache.paged import CacheNeed, KVNeed
from ..config.spec import ConfigError, PartSpec
from ..kernels import native
from ..weights.arena import Piece, Resident, resident_of
from ..weights.loader import TensorDecl
from .registry import part_class, register_mixer

# warps per SM of the general attention kernel that a split of the keys aims at
_WARPS_PER_SM = 16
# SIB_PREFILL_TCGEN05=0 selects the mma.sync prompt kernel instead of the tcgen05 one
_USE_TCGEN05_PREFILL = os.environ.get("SIB_PREFILL_TCGEN05", "1") != "0"
# SIB_LATENT_MMA=0 sends the bfloat16 latent attention to the general kernel instead of the
# tensor-core one
_USE_LATENT_MMA = os.environ.get("SIB_LATENT_MMA", "1") != "0"
# SIB_LATENT_EXPAND=0: long bfloat16 prompts of the latent attention attend over the latent rows
# too, instead of over keys and values made per head (the tcgen05 prompt kernel)
_USE_LATENT_EXPAND = os.environ.get("SIB_LATENT_EXPAND", "1") != "0"


def decode_shape(units: int, longest: int, window: int, resident4: int, resident8: int,
                 block_warps=(8, 4, 2)):
    """(runs, warps) of the decode kernel for ``units`` (row, kv head) pairs whose rows see up
    to ``longest`` keys, on a device that holds ``resident4`` warps of the kernel in blocks of
    4 (or fewer) warps and ``resident8`` in blocks of 8 (``Attention._decode_shape`` says why)."""
    # (a full window does not begin at a tile's first key: it reaches into one tile more)
    tiles = -(-longest // 16) + (1 if 0 < window <= longest else 0)

    def fewest(resident: int) -> int:
        """Warps for a (row, kv head): as few tiles each as ``resident`` warps allow."""
        room = max(1, resident // units)
        each = -(-tiles // room)
        return max(1, min(room, -(-tiles // each)))

    def trimmed(runs: int, warps: int):
        """Without the blocks that whole blocks of ``warps`` warps leave no tile for."""
        each = -(-tiles // (runs * warps))
        return -(-(-(-tiles // each)) // warps), warps

    most = fewest(resident4)
    if 8 in block_warps and resident8 // units >= 8:
        wide = min(-(-fewest(resident8) // 8), resident8 // units // 8, 128)
        if wide >= 8 and 8 * wide >= 0.6 * most:
            return trimmed(wide, 8)
    room = max(1, resident4 // units)
    for warps in (w for w in block_warps if w < 8):   # wider blocks: fewer results to join
        runs = min(-(-most // warps), room // warps, 128)
        if runs >= 1 and runs * warps >= 0.9 * most:
            return trimmed(runs, warps)
    return trimmed(min(most, 128), 1)


class Attention:
    chain_safe = True      # deferred results are read by this runtime's and native's launchers only

    @property
    def captures_prompts(self) -> bool:
        """Whether a step of prompts of this part may be recorded and replayed for other
        prompts (StepContext ``from_start``): it then reads sequences, slots and counts on
        the device only.  True with a rotary position part, or one that promises the same."""
        return hasattr(self.position, "rotary") or getattr(self.position, "captures_prompts", False)

    @staticmethod
    def _extras(params: Mapping) -> bool:
        """Whether the heads are worked on between the projection and the attention."""
        return bool(params.get("bias") or params.get("qk_norm") or params.get("value_mix")
                    or params.get("head_gate") or params.get("pool")
                    or int(params.get("value_dim") or params["head_dim"]) != params["head_dim"]
                    or int(params["head_dim"]) % 16 != 0)      # (padded to the next 16)

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        nh, nkv, hd = params["num_heads"], params["num_kv_heads"], params["head_dim"]
        vd = int(params.get("value_dim") or hd)
        out = {
            "q_proj.weight": TensorDecl((nh * hd, hidden)),
            "k_proj.weight": TensorDecl((nkv * hd, hidden)),
            "v_proj.weight": TensorDecl((nkv * vd, hidden)),
            "o_proj.weight": TensorDecl((hidden, nh * vd)),
        }
        if params.get("borrows_cache"):
            if params.get("bias") or params.get("qk_norm") or params.get("value_mix") or params.get("pool"):
                raise ConfigError("attention: a layer that reads another's keys and values has no "
                                  "biases, norms, mixed values or pooled blocks of its own")
            del out["k_proj.weight"], out["v_proj.weight"]
        if params.get("sink"):
            out["sink"] = TensorDecl((nh,), init="norm")
        if params.get("bias"):
            out["q_proj.bias"] = TensorDecl((nh * hd,), init="norm")
            out["k_proj.bias"] = TensorDecl((nkv * hd,), init="norm")
            out["v_proj.bias"] = TensorDecl((nkv * vd,), init="norm")
        if params.get("qk_norm"):
            out["q_norm.weight"] = TensorDecl((hd,), init="norm")
            out["k_norm.weight"] = TensorDecl((hd,), init="norm")
        if params.get("value_mix"):
            # (the layer whose values the others mix in may store a weight too; it is not read)
            out["value_mix.weight"] = TensorDecl((), init="norm",
                                                 optional=params["value_mix"] == "first")
        if params.get("head_gate"):
            out["g_proj.weight"] = TensorDecl((nh, hidden))
        pos: PartSpec = params["position"]
        for name, decl in part_class("position", pos.kind).tensors(pos.params, hd).items():
            out["position." + name] = decl
        return out

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        """q, k and v are kept as ONE matrix (one product makes all three)."""
        nh, nkv, hd = params["num_heads"], params["num_kv_heads"], params["head_dim"]
        vd = int(params.get("value_dim") or hd)
        n_qkv = (nh + nkv) * hd + nkv * vd
        pieces = (Piece("q_proj.weight", 0), Piece("k_proj.weight", nh * hd),
                  Piece("v_proj.weight", (nh + nkv) * hd))
        if params.get("borrows_cache"):       # q alone
            n_qkv, pieces = nh * hd, pieces[:1]
        if params.get("head_gate"):       # the gates' rows behind q, k and v: one product makes all
            pieces += (Piece("g_proj.weight", n_qkv),)
        out = {
            "qkv_proj.weight": Resident((n_qkv + (nh if params.get("head_gate") else 0), hidden),
                                        pieces=pieces),
            "o_proj.weight": Resident((hidden, nh * vd), pieces=(Piece("o_proj.weight"),)),
        }
        if params.get("sink"):
            out["sink"] = Resident((nh,), torch.float32, (Piece("sink"),))
        if params.get("bias"):
            out["qkv_proj.bias"] = Resident((n_qkv,), torch.float32, (
                Piece("q_proj.bias", 0), Piece("k_proj.bias", nh * hd),
                Piece("v_proj.bias", (nh + nkv) * hd)))
        if params.get("qk_norm"):
            out["q_norm.gain"] = Resident((hd,), torch.float32, (Piece("q_norm.weight"),))
            out["k_norm.gain"] = Resident((hd,), torch.float32, (Piece("k_norm.weight"),))
        if params.get("value_mix") == "mix":
            out["value_mix.weight"] = Resident((1,), torch.float32, (Piece("value_mix.weight"),))
        pos: PartSpec = params["position"]
        cls = part_class("position", pos.kind)
        for name, res in resident_of(cls, cls.tensors(pos.params, hd), pos.params, hd).items():
            out["position." + name] = Resident(res.shape, res.dtype, tuple(
                Piece("position." + q.source, q.row_offset, q.group, q.group_stride)
                for q in res.pieces), res.offset)
        return out

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.hidden = hidden
        self.nh = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.hd = int(params["head_dim"])
        self.scale = float(params["score_scale"])
        self.softcap = float(params.get("logit_softcap") or 0.0)
        self.window = int(params.get("window") or 0)
        self.chunk = int(params.get("chunk") or 0)
        self.sink = weights.get("sink") if params.get("sink") else None
        self.borrows = bool(params.get("borrows_cache"))
        self.lends = bool(params.get("lends_cache"))
        if self.chunk < 0 or (self.chunk and (self.window or params.get("pool"))):
            raise ConfigError("attention: a chunked mask goes without a window and pooled blocks")
        if (self.chunk or self.sink is not None) and float(params.get("logit_softcap") or 0.0):
            raise ConfigError("attention: a chunked mask or a sink goes without a soft cap")
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"attention: {self.nh} heads cannot share {self.nkv} kv heads")
        self.vd = int(params.get("value_dim") or self.hd)
        self.extras = self._extras(params)
        # kw: how wide a head is in the packed rows, in the cache and for the attention kernels
        self.kw = -(-max(self.hd, self.vd) // 16) * 16 if self.extras else self.hd
        if self.kw % 16 or not 16 <= self.kw <= 512 or self.hd <= 0 or self.vd <= 0:
            raise ConfigError(f"attention: head_dim {self.hd} must be a multiple of 16 "
                              f"between 16 and 512 (any size up to 512 with worked-on heads)")
        pos: PartSpec = params["position"]
        pos_w = {k[len("position."):]: v for k, v in weights.items() if k.startswith("position.")}
        self.position = part_class("position", pos.kind)(pos.params, self.hd, pos_w, rt)
        self.pool = int(params.get("pool") or 0)
        if self.pool < 0 or (self.pool and self.window <= 0):
            raise ConfigError("attention: pooled blocks go with a window")
        self.rope_style = native.ROPE_HALF_SPLIT
        if self.extras:
            norm = params.get("qk_norm")
            self.qk_eps = float(norm["eps"]) if norm else 0.0
            self.bias = weights.get("qkv_proj.bias")
            self.q_gain, self.k_gain = weights.get("q_norm.gain"), weights.get("k_norm.gain")
            self.value_mix = params.get("value_mix") or None
            if self.value_mix not in (None, "first", "mix"):
                raise ConfigError(f"attention: value_mix {self.value_mix!r} is not 'first' or 'mix'")
            self.lam = weights.get("value_mix.weight")
            self.head_gate = bool(params.get("head_gate"))
            self.n_qkv = self.nh * self.hd if self.borrows \
                else (self.nh + self.nkv) * self.hd + self.nkv * self.vd
            rotary = self.position.rotary() if hasattr(self.position, "rotary") else None
            if rotary is None:
                raise ConfigError("attention: worked-on heads take a rotary position part (or 'none')")
            self.rope_style = rotary[2]
        self.w_qkv = rt.cast_matrix(weights["qkv_proj.weight"])
        self.w_q = self.w_qkv[: self.nh * self.hd]
        self.w_o = rt.cast_matrix(weights["o_proj.weight"])
        self._resident_warps: Optional[int] = None
        self._target_warps = _WARPS_PER_SM * rt.sm_count
        self._block_warps = tuple(int(w) for w in os.environ.get("SIB_DECODE_WARPS", "8,4,2").split(","))

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(kv=KVNeed(self.nkv, self.kw, self.window, pool=self.pool, chunk=self.chunk))

    # ------------------------------------------------------------------
    def _longest(self, ctx, capacity: int) -> int:
        longest = (min(ctx.span or capacity, capacity)) if ctx.graph_capture else ctx.max_end
        if self.chunk > 0:
            return min(longest, self.chunk)
        return min(longest, self.window) if self.window > 0 else longest

    def _splits(self, ctx, capacity: int) -> int:
        """How many runs of keys the general kernel cuts a (row, head) into, one
        warp each: as many as fill the device once, none shorter than 32 keys."""
        want = max(1, self._target_warps // max(1, ctx.n_rows * self.nh))
        return max(1, min(want, -(-self._longest(ctx, capacity) // 32), 128))

    def _decode_shape(self, ctx, capacity: int):
        """(runs, warps) for the decode kernel: each (row, kv head) is read by
        ``runs`` blocks of ``warps`` warps.  All of them should be resident at
        once (a second, partly filled wave of blocks costs more than it brings).  A warp
        walks its tiles of 16 keys one after the other, a round trip to memory each, so a
        (row, kv head) gets as many warps as give each the fewest tiles that residency
        allows, and no more than that needs: more warps only mean more partial results to
        join.  (Before, a warp took no fewer than 32 keys and all the warps that fit: with the
        rule above batch 1 went from 1.64 to 1.57 ms at context 1 024 and from 1.72 to 1.68 ms at
        8 192, batch 16 from 2.07 to 1.98 ms at context 1 024; no size measured lost, on the 9B
        and 27B shapes neither.)  Blocks of 8 warps (of which the device holds fewer warps in all) halve the
        partial results that the last block of a (row, kv head) joins: they are taken where
        that join weighs most, with few rows and therefore many runs each (measured at the
        Gemma2-2B shape, context 8 192: batch 1 1.83 -> 1.74 ms, batch 2 1.95 -> 1.84, batch 4
        2.06 -> 2.04; batch 6 and 8 are better off with blocks of 4)."""
        if self._resident_warps is None:     # what the device holds of this kernel at a time
            self._resident_warps = {w: native.attention_decode_resident_warps(self.nh, self.nkv, self.kw, w)
                                    for w in (8, 4)}
        # (a chunk that does not begin at a tile's first key reaches into one tile more, as a window does)
        edge = self.window or (self.chunk if self.chunk % 16 else 0)
        return decode_shape(max(1, ctx.n_rows * self.nkv), self._longest(ctx, capacity), edge,
                            self._resident_warps[4], self._resident_warps[8], self._block_warps)

    def _pieces_pay(self, ctx) -> bool:
        """Whether copying what the step's sequences hold (read, write, read again by the
        prompt kernel) moves less than reading it row by row does."""
        seen = float(self.window) if self.window > 0 else float("inf")
        by_row = sum(n * min(seen, st + n / 2) for st, n in zip(ctx.starts, ctx.counts))
        copied = sum(min(seen + n, st + n) for st, n in zip(ctx.starts, ctx.counts))
        return by_row > 3 * copied

    def _attend_pieces(self, qkv: torch.Tensor, out: torch.Tensor, ctx, view) -> None:
        """Attention of a step that continues sequences with many tokens each (a prompt that
        comes in pieces): the keys and values that the rows see - what the sequences held and
        what this step has just stored - are copied from the pages into a packed buffer
        whose rows are positions, the step's queries are put at their positions, and the
        prompt kernel runs over it with the rows before each piece as keys only.  (Row by row
        over the cache, as single-token steps do it, every row reads its sequence's whole
        past: 4 096 tokens in pieces of 512 took 183 ms instead of 15 ms in one piece.)"""
        rt, nh, nkv, hd = self.rt, self.nh, self.nkv, self.kw
        memo = ctx.memo.setdefault(("pieces", self.window), {})
        if not memo:
            starts, counts = ctx.starts, ctx.counts
            ends = [st + n for st, n in zip(starts, counts)]
            first = [max(0, st - self.window + 1) if self.window > 0 else 0 for st in starts]
            row0, acc = [], 0
            for e in ends:
                row0.append(acc)
                acc += e
            dev = lambda v: torch.tensor(v, dtype=torch.int32).to(qkv.device, non_blocking=True)  # noqa: E731
            memo.update(row0=row0, ends=ends, first=first, rows=acc, d_row0=dev(row0), d_ends=dev(ends),
                        d_first=dev(first), d_starts=dev(starts),
                        most=max(e - f for e, f in zip(ends, first)))
            memo["plan"] = native.attention_prefill_tc_plan(ends, nh, nkv, hd, self.window, starts)
        width = (nh + 2 * nkv) * hd
        # (one packed buffer and one output buffer a step: the layers use them in turn)
        shared = ctx.memo.setdefault(("pieces", "buffers", width, nh * hd), {})
        if not shared:
            # (zeros: a windowed layer copies only what its rows see, but the kernel's key
            # tiles reach further down and over a sequence's end into the next one's rows;
            # what is masked there must still be finite, or 0 x NaN spoils the sums)
            shared["packed"] = torch.zeros((memo["rows"], width), dtype=qkv.dtype, device=qkv.device)
            shared["whole"] = torch.empty((memo["rows"], nh * hd), dtype=qkv.dtype, device=qkv.device)
        packed, whole = shared["packed"], shared["whole"]
        native.gather_kv_rows(packed, view.k, view.v, view.page_table, ctx.seq_slot, memo["d_first"],
                              memo["d_ends"], memo["d_row0"], memo["most"], view.page_tokens,
                              view.ring_tokens, nh, nkv, hd)
        r = 0
        for row0, st, n in zip(memo["row0"], ctx.starts, ctx.counts):
            packed[row0 + st:row0 + st + n, :nh * hd].copy_(qkv[r:r + n, :nh * hd])
            r += n
        n_items, need, n_tickets = memo["plan"]
        lens = memo["ends"] if n_items else None
        if not n_items:
            need, n_tickets = native.attention_prefill_tc_split(ctx.n_seqs, max(memo["ends"]), nh, nkv, hd)
        native.attention_prefill_tc(packed, whole, memo["d_row0"], memo["d_ends"], ctx.n_seqs,
                                    max(memo["ends"]), nh, nkv, hd, self.scale, self.softcap,
                                    self.window, rt.scratch(need) if need else None,
                                    rt.tickets(n_tickets) if need else None, lens,
                                    memo["d_starts"], ctx.starts if lens else None)
        r = 0
        for row0, st, n in zip(memo["row0"], ctx.starts, ctx.counts):
            out[r:r + n].copy_(whole[row0 + st:row0 + st + n])
            r += n

    # the most chunks of a step that the prompt kernel takes as sequences
    _MOST_CHUNKS = 16384

    def _chunks(self, ctx):
        """The chunks of a step of prompts as sequences of the prompt kernel: (first rows on
        the device, lengths on the device, lengths on the host, the longest)."""
        if self.chunk <= 0:
            return ctx.seq_row0, ctx.seq_end, ctx.counts, ctx.max_count
        memo = ctx.memo.setdefault(("chunks", self.chunk), {})
        if not memo:
            row0, lens, at = [], [], 0
            for n in ctx.counts:
                for c in range(0, n, self.chunk):
                    row0.append(at + c)
                    lens.append(min(self.chunk, n - c))
                at += n
            dev = lambda v: torch.tensor(v, dtype=torch.int32).to(ctx.row_pos.device, non_blocking=True)  # noqa: E731
            memo.update(row0=dev(row0), lens=dev(lens), host=lens, most=max(lens))
        return memo["row0"], memo["lens"], memo["host"], memo["most"]

    def _attend_masked(self, qkv: torch.Tensor, out: torch.Tensor, ctx, view, owns_cache: bool,
                       cache_entry: int) -> torch.Tensor:
        """Attention with a mask of chunks and a sink per head (either may be absent)."""
        rt, nh, nkv, hd = self.rt, self.nh, self.nkv, self.kw
        R = qkv.shape[0]
        bf16 = qkv.dtype == torch.bfloat16
        full = (nh + 2 * nkv) * hd
        prompts = ctx.all_from_start and not ctx.graph_capture
        if self.lends and owns_cache and prompts:
            ctx.memo[("kv_rows", cache_entry)] = qkv
        tc = (prompts and bf16 and _USE_TCGEN05_PREFILL and self.scale > 0
              and native.attention_prefill_tc_supports(nh, nkv, hd, full)
              and (self.chunk <= 0 or sum(-(-n // self.chunk) for n in ctx.counts) <= self._MOST_CHUNKS))
        if tc and not owns_cache:
            lent = ctx.memo.get(("kv_rows", cache_entry))
            if lent is None or lent.shape != (R, full):
                tc = False
            else:           # this layer's queries beside the lender's keys and values
                packed = torch.empty((R, full), dtype=qkv.dtype, device=qkv.device)
                packed[:, :nh * hd].copy_(qkv[:, :nh * hd])
                packed[:, nh * hd:].copy_(lent[:, nh * hd:])
                qkv = packed
        if tc:
            row0, lens, host_lens, most = self._chunks(ctx)
            n_seqs = len(host_lens)
            n_items, need, n_tickets = native.attention_prefill_tc_plan(host_lens, nh, nkv, hd, 0)
            if n_items == 0:
                host_lens = None
                need, n_tickets = native.attention_prefill_tc_split(n_seqs, most, nh, nkv, hd)
            return native.attention_prefill_tc(qkv, out, row0, lens, n_seqs, most, nh, nkv, hd, self.scale,
                                               0.0, 0, rt.scratch(need) if need else None,
                                               rt.tickets(n_tickets) if need else None, host_lens,
                                               sink=self.sink)
        width = qkv.shape[1]
        cached = not (ctx.all_from_start and owns_cache)
        if cached and bf16 and native.attention_decode_supports(nh, nkv, hd, view.page_tokens):
            splits, warps = self._decode_shape(ctx, ctx.cache.max_seq_len)
            scratch = tickets = None
            if splits > 1:
                scratch = rt.scratch(native.attention_rows_scratch_bytes(R, nh, hd, splits))
                tickets = rt.tickets(R * nkv)
            return native.attention_decode(qkv, width, view.k, view.v, view.page_table, view.page_tokens,
                                           view.ring_tokens, ctx.row_pos, ctx.row_seq, ctx.seq_slot, out,
                                           scratch, tickets, nh, nkv, hd, self.scale, 0.0, 0, splits, warps,
                                           fresh=ctx.max_count if rt.early_keys else 0, chunk=self.chunk,
                                           sink=self.sink)
        # the general kernel: the step's own keys from the packed rows, earlier ones from the cache
        splits = self._splits(ctx, ctx.cache.max_seq_len) if cached else 1
        scratch = None
        if splits > 1:
            scratch = rt.scratch(native.attention_rows_scratch_bytes(R, nh, hd, splits))
        own = owns_cache and not cached
        return native.attention_rows(qkv, width, qkv[:, nh * hd:] if own else None,
                                     qkv[:, (nh + nkv) * hd:] if own else None, width,
                                     view.k if cached else None, view.v if cached else None,
                                     view.page_table if cached else None, view.page_tokens,
                                     view.ring_tokens, ctx.row_pos, ctx.row_seq, ctx.seq_slot,
                                     ctx.seq_start, ctx.seq_row0, out, scratch, nh, nkv, hd,
                                     self.scale, 0.0, 0, splits, sink=self.sink, chunk=self.chunk)

    def forward(self, x: torch.Tensor, ctx, entry: int, cache_entry: int,
                owns_cache: bool) -> torch.Tensor:
        rt, nh, hd = self.rt, self.nh, self.kw
        R = x.shape[0]
        nkv = self.nkv if owns_cache else 0
        view = ctx.kv(cache_entry)
        if self.borrows and owns_cache:
            raise ValueError("attention: a layer without key and value projections reads another "
                             "run's cache")
        if self.extras and not owns_cache and (self.pool or self.value_mix):
            raise ValueError("attention: pooled blocks and mixed values cannot read another run's cache")
        fresh = ctx.all_from_start and owns_cache
        if not fresh and view.ring_tokens > 0 and not ctx.graph_capture:
            # rows that attend over a ring must not overwrite a key that an earlier row of
            # the same step still sees (a captured step adds one position: always fine)
            room = view.ring_tokens - max(self.window, self.pool) + 1
            for start, n in zip(ctx.starts, ctx.counts):
                if n > room and start + n > view.ring_tokens:
                    raise ValueError(
                        f"a step may add at most {max(room, view.ring_tokens - start)} positions "
                        f"to a sequence of {start} whose layers keep a window of {self.window} "
                        f"in a ring of {view.ring_tokens}; got {n}")

        w_in = self.w_qkv if (owns_cache or self.borrows) else self.w_q
        rotary = self.position.rotary() if hasattr(self.position, "rotary") else None
        proj = None
        if self.extras:
            # bias, norms of q and k, rotation, mixing of values and the cache write in one
            # kernel, from the projected row to packed heads of `kw`
            proj = rt.linear(x, w_in)
            qkv = torch.empty((R, (nh + 2 * nkv) * hd), dtype=proj.dtype, device=proj.device)
            v_first = None
            if self.value_mix == "mix":
                v_first = ctx.memo.get("value_mix.first")
                if v_first is None:
                    raise ValueError("attention: values to mix in, but no earlier layer left any")
            native.head_prepare(proj, qkv, self.bias, self.q_gain, self.k_gain, self.qk_eps,
                                rotary[0], rotary[1], v_first, self.lam if v_first is not None else None,
                                ctx.row_pos, ctx.row_seq, ctx.seq_slot, ctx.seq_end,
                                view.k if owns_cache else None, view.v if owns_cache else None,
                                view.page_table if owns_cache else None, view.page_tokens,
                                view.ring_tokens, nh, nkv, self.hd, self.vd, hd, style=self.rope_style)
            if self.pool:
                native.pool_store(qkv, view, ctx, nh, nkv, hd)
            if self.value_mix == "first":
                ctx.memo["value_mix.first"] = qkv[:, (nh + nkv) * hd:]
        elif (rotary is not None and rotary[1] == hd and rotary[2] == native.ROPE_HALF_SPLIT
                and x.dtype == torch.bfloat16 and rt.fuse_rotation and 0 < R <= rt.fused_rope_max_rows
                and self.hidden % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0):
            # few rows: the product rotates q and k and writes k and v into the cache itself
            qkv = torch.empty((R, w_in.shape[0]), dtype=x.dtype, device=x.device)
            rt.linear_rope(x, w_in, qkv, row_pos=ctx.row_pos, row_seq=ctx.row_seq,
                           seq_slot=ctx.seq_slot, seq_end=ctx.seq_end, inv_freq=rotary[0],
                           k_pool=view.k if owns_cache else None,
                           v_pool=view.v if owns_cache else None,
                           page_table=view.page_table if owns_cache else None,
                           page_tokens=view.page_tokens, ring_tokens=view.ring_tokens,
                           n_heads=nh, n_kv=nkv, head_dim=hd)
        else:
            qkv = rt.linear(x, w_in)
            if rotary is not None:
                inv_freq, rot, style = rotary
            else:
                rt.flush()      # a position part of its own works on q and k with its own code
                q_view = qkv[:, : nh * hd].view(R, nh, hd)
                k_view = qkv[:, nh * hd:(nh + nkv) * hd].view(R, nkv, hd) if nkv else None
                self.position.apply(q_view, k_view, ctx)
                inv_freq, rot, style = None, 0, native.ROPE_HALF_SPLIT
            native.rope_store(qkv, ctx.row_pos, ctx.row_seq, ctx.seq_slot, ctx.seq_end, inv_freq,
                              rot, style, view.k if owns_cache else None,
                              view.v if owns_cache else None,
                              view.page_table if owns_cache else None, view.page_tokens,
                              view.ring_tokens, nh, nkv, hd)

        out = torch.empty((R, nh * hd), dtype=qkv.dtype, device=qkv.device)
        width = qkv.shape[1]
        # (prompts of up to 128 tokens: the mma.sync kernel, whose blocks of 64 rows start in a
        # fraction of the time that a tcgen05 block needs before its first tile; measured on 2 048
        # rows of the Gemma2-2B shape: 64 prompts of 32 tokens 22 against 65 us a call, 16 of 128
        # 28 against 39 us, 8 of 256 36 against 56 us the other way round)
        short = ctx.max_count <= rt.short_prompt_tokens and native.attention_prefill_supports(
            nh, self.nkv, hd)
        tc_prompt = (fresh and qkv.dtype == torch.bfloat16 and _USE_TCGEN05_PREFILL and self.scale > 0
                     and not short and native.attention_prefill_tc_supports(nh, self.nkv, hd, width)
                     and not (self.pool and self.softcap))
        if self.chunk > 0 or self.sink is not None:
            out = self._attend_masked(qkv, out, ctx, view, owns_cache, cache_entry)
        elif (self.pool or (self.extras and self.window)) and not tc_prompt:
            # blocks before the window join the softmax: the general kernel, which reads the
            # step's own keys from the packed rows, earlier ones from the cache and the blocks'
            # cells from their store
            cached = not fresh
            splits = self._splits(ctx, ctx.cache.max_seq_len) if cached else 1
            scratch = None
            if splits > 1:
                scratch = rt.scratch(native.attention_rows_scratch_bytes(R, nh, hd, splits))
            native.attention_rows(qkv, width, None if cached else qkv[:, nh * hd:],
                                  None if cached else qkv[:, (nh + nkv) * hd:], width,
                                  view.k if cached else None, view.v if cached else None,
                                  view.page_table if cached else None, view.page_tokens,
                                  view.ring_tokens, ctx.row_pos, ctx.row_seq, ctx.seq_slot,
                                  ctx.seq_start, ctx.seq_row0, out, scratch, nh, self.nkv, hd,
                                  self.scale, self.softcap, self.window, splits,
                                  cells=view if self.pool else None)
        elif tc_prompt:
            extra = None
            if self.pool:
                # the blocks before each row's window first, by the general kernel: (max, sum,
                # accumulator) per row and head, which the prompt kernel joins with its own
                extra = torch.empty((R, nh, hd + 2), dtype=torch.float32, device=qkv.device)
                native.attention_rows(qkv, width, qkv[:, nh * hd:], qkv[:, (nh + nkv) * hd:], width,
                                      None, None, None, view.page_tokens, view.ring_tokens,
                                      ctx.row_pos, ctx.row_seq, ctx.seq_slot, ctx.seq_start,
                                      ctx.seq_row0, out, extra, nh, self.nkv, hd, self.scale, 0.0,
                                      self.window, 1, cells=view, cells_only=True)
            # a launch too small for the device splits its long blocks, given the memory
            # (with the lengths known on the host, not in a recorded step, the launch is a
            # balanced list of work items)
            lens = None if ctx.graph_capture else ctx.counts
            n_items = 0
            if lens is not None:
                n_items, need, n_tickets = native.attention_prefill_tc_plan(lens, nh, self.nkv, hd,
                                                                            self.window)
            if n_items == 0:
                lens = None
                need, n_tickets = native.attention_prefill_tc_split(ctx.n_seqs, ctx.max_count, nh,
                                                                   self.nkv, hd)
            native.attention_prefill_tc(qkv, out, ctx.seq_row0, ctx.seq_end, ctx.n_seqs,
                                        ctx.max_count, nh, self.nkv, hd, self.scale, self.softcap,
                                        self.window, rt.scratch(need) if need else None,
                                        rt.tickets(n_tickets) if need else None, lens, extra=extra)
        elif fresh and qkv.dtype == torch.bfloat16 and \
                native.attention_prefill_supports(nh, self.nkv, hd):
            native.attention_prefill(qkv, out, ctx.seq_row0, ctx.seq_end, ctx.n_seqs,
                                     ctx.max_count, nh, self.nkv, hd, self.scale, self.softcap,
                                     self.window)
        elif fresh:
            k_new = qkv[:, nh * hd:]
            v_new = qkv[:, (nh + nkv) * hd:]
            native.attention_rows(qkv, width, k_new, v_new, width, None, None, None,
                                  view.page_tokens, view.ring_tokens, ctx.row_pos, ctx.row_seq,
                                  ctx.seq_slot, ctx.seq_start, ctx.seq_row0, out, None, nh,
                                  self.nkv, hd, self.scale, self.softcap, self.window, 1)
        elif (qkv.dtype == torch.bfloat16 and not ctx.graph_capture
              and ctx.max_count >= rt.piece_attention_rows and _USE_TCGEN05_PREFILL and self.scale > 0
              and native.attention_prefill_tc_supports(nh, self.nkv, hd, (nh + 2 * self.nkv) * hd)
              and self._pieces_pay(ctx)):
            self._attend_pieces(qkv, out, ctx, view)
        elif qkv.dtype == torch.bfloat16 and native.attention_decode_supports(
                nh, self.nkv, hd, view.page_tokens):
            splits, warps = self._decode_shape(ctx, ctx.cache.max_seq_len)
            scratch = tickets = None
            if splits > 1:
                scratch = rt.scratch(native.attention_rows_scratch_bytes(R, nh, hd, splits))
                tickets = rt.tickets(R * self.nkv)
            native.attention_decode(qkv, width, view.k, view.v, view.page_table, view.page_tokens,
                                    view.ring_tokens, ctx.row_pos, ctx.row_seq, ctx.seq_slot, out,
                                    scratch, tickets, nh, self.nkv, hd, self.scale, self.softcap,
                                    self.window, splits, warps,
                                    fresh=ctx.max_count if rt.early_keys else 0)
        else:
            splits = self._splits(ctx, ctx.cache.max_seq_len)
            scratch = None
            if splits > 1:
                scratch = rt.scratch(native.attention_rows_scratch_bytes(R, nh, hd, splits))
            native.attention_rows(qkv, width, None, None, width, view.k, view.v, view.page_table,
                                  view.page_tokens, view.ring_tokens, ctx.row_pos, ctx.row_seq,
                                  ctx.seq_slot, ctx.seq_start, ctx.seq_row0, out, scratch, nh,
                                  self.nkv, hd, self.scale, self.softcap, self.window, splits)
        if self.extras:
            y = torch.empty((R, nh * self.vd), dtype=out.dtype, device=out.device)
            gate = proj[:, self.n_qkv:self.n_qkv + nh] if self.head_gate else None
            out = native.head_gate(out, gate, y, nh, self.vd, hd)
        return rt.linear(out, self.w_o)


class LatentAttention:
    """Attention whose keys and values of all heads are made from one low-rank row per
    position (the latent c = rms_norm(down(x)[:rank]) * weight) and one rotated key part of
    ``rot_dim`` columns that the heads share; only these are cached.

    Parameters: ``num_heads``, ``head_dim`` (unrotated query/key columns of a head),
    ``rot_dim`` (rotated ones, behind them), ``value_dim``, ``kv_rank``, ``score_scale``,
    ``window`` (0: none), ``norm_eps``, ``position`` (a rotary part, applied to the rotated
    columns of q and to the shared key part), ``sink`` (one stored number per head whose
    exponential joins the softmax's denominator), ``head_gate`` (sigmoid(g_proj x) per head
    on the head's output), ``q_rank`` (r > 0: the queries pass a latent of their own,
    q = uq_proj (rms_norm(dq_proj x) * dq_norm.weight) with r the latent's width, instead of
    q = q_proj x; the norm is 32-bit and takes ``norm_eps``).

        q_h = [a_h | r_h] = q_proj x (per head);  k_h = [U_h c | rot(k_r)],  v_h = V_h c
        score_h(t, j) = (<a_h(t), U_h c(j)> + <rot(r_h(t)), rot(k_r(j))>) * score_scale

    The scores are taken against the cached rows themselves: <a_h, U_h c> = <U_h^T a_h, c>, so
    a query head becomes [U_h^T a_h | rot(r_h)], every head attends over the ONE row
    [c | rot(k_r)] per position, the weighted sum of the c rows comes out of the attention
    kernel, and V_h is applied to that sum (csrc/head_prepare.cu latent_prepare; bfloat16:
    csrc/attention_latent.cu, a key tile fetched once for all heads and used on the tensor
    cores for scores and sums; 32-bit: csrc/attention_rows.cu with ``values_in_keys``).  The two per-head products are batched
    library products; softmax, sink and sums are 32-bit.
    """

    captures_prompts = True      # sequences, slots and counts are read on the device only

    @staticmethod
    def _sizes(params: Mapping):
        nh, qd, rd = int(params["num_heads"]), int(params["head_dim"]), int(params.get("rot_dim") or 0)
        vd, rank = int(params["value_dim"]), int(params["kv_rank"])
        if min(nh, qd, vd, rank) <= 0 or rd < 0:
            raise ConfigError(f"latent_attention: {nh} heads of {qd} + {rd}, values of {vd}, rank {rank}")
        pad = -(-(rank + rd) // 16) * 16
        if pad > 1024:
            raise ConfigError(f"latent_attention: kv_rank + rot_dim = {rank + rd} exceeds 1024")
        return nh, qd, rd, vd, rank, pad

    @classmethod
    def tensors(cls, params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        nh, qd, rd, vd, rank, _ = cls._sizes(params)
        q_rank = int(params.get("q_rank") or 0)
        queries = {"q_proj.weight": TensorDecl((nh * (qd + rd), hidden))} if not q_rank else {
            "dq_proj.weight": TensorDecl((q_rank, hidden)),
            "dq_norm.weight": TensorDecl((q_rank,), init="norm"),
            "uq_proj.weight": TensorDecl((nh * (qd + rd), q_rank))}
        out = {
            **queries,
            "dkv_proj.weight": TensorDecl((rank + rd, hidden)),
            "dkv_norm.weight": TensorDecl((rank,), init="norm"),
            "uk_proj.weight": TensorDecl((nh * qd, rank)),
            "uv_proj.weight": TensorDecl((nh * vd, rank)),
            "o_proj.weight": TensorDecl((hidden, nh * vd)),
        }
        if params.get("sink"):
            out["sink"] = TensorDecl((nh,), init="norm")
        if params.get("head_gate"):
            out["g_proj.weight"] = TensorDecl((nh, hidden))
        return out

    @classmethod
    def resident(cls, params: Mapping, hidden: int) -> Dict[str, Resident]:
        """The query heads, the down projection and the gates as ONE matrix."""
        nh, qd, rd, vd, rank, _ = cls._sizes(params)
        q_rank = int(params.get("q_rank") or 0)
        n_q = q_rank or nh * (qd + rd)      # rows of the first piece: the queries, or their latent
        pieces = (Piece("dq_proj.weight" if q_rank else "q_proj.weight", 0), Piece("dkv_proj.weight", n_q))
        n_in = n_q + rank + rd
        if params.get("head_gate"):
            pieces += (Piece("g_proj.weight", n_in),)
            n_in += nh
        out = {
            "in_proj.weight": Resident((n_in, hidden), pieces=pieces),
            "dkv_norm.gain": Resident((rank,), torch.float32, (Piece("dkv_norm.weight"),)),
            "uk_proj.weight": Resident((nh * qd, rank), pieces=(Piece("uk_proj.weight"),)),
            "uv_proj.weight": Resident((nh * vd, rank), pieces=(Piece("uv_proj.weight"),)),
            "o_proj.weight": Resident((hidden, nh * vd), pieces=(Piece("o_proj.weight"),)),
        }
        if params.get("sink"):
            out["sink"] = Resident((nh,), torch.float32, (Piece("sink"),))
        if q_rank:
            out["dq_norm.gain"] = Resident((q_rank,), torch.float32, (Piece("dq_norm.weight"),))
            out["uq_proj.weight"] = Resident((nh * (qd + rd), q_rank), pieces=(Piece("uq_proj.weight"),))
        return out

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.nh, self.qd, self.rd, self.vd, self.rank, self.kw = self._sizes(params)
        self.q_rank = int(params.get("q_rank") or 0)
        if self.q_rank < 0:
            raise ConfigError(f"latent_attention: q_rank {self.q_rank}")
        self.q_gain = weights.get("dq_norm.gain")
        self.w_uq = rt.cast_matrix(weights["uq_proj.weight"]) if self.q_rank else None
        self.scale = float(params["score_scale"])
        self.window = int(params.get("window") or 0)
        self.eps = float(params["norm_eps"])
        pos: PartSpec = params.get("position") or PartSpec("none", {})
        position = part_class("position", pos.kind)(pos.params, max(self.rd, 2), {}, rt) \
            if self.rd else None
        self.inv_freq, self.rot = None, 0
        if position is not None:
            if not hasattr(position, "rotary"):
                raise ConfigError("latent_attention: the position part must offer rotary()")
            self.inv_freq, self.rot, style = position.rotary()
            if self.rot and style != native.ROPE_INTERLEAVED:
                raise ConfigError("latent_attention: the rotated columns are rotated in neighbouring pairs")
        self.head_gate = bool(params.get("head_gate"))
        self.n_q = self.nh * (self.qd + self.rd)
        self.w_in = rt.cast_matrix(weights["in_proj.weight"])
        self.c_gain = weights["dkv_norm.gain"]
        # per head: U_h [qd, rank] (q times it) and V_h^T [rank, vd] (the summed latents times it)
        w_uk, w_uv = rt.cast_matrix(weights["uk_proj.weight"]), rt.cast_matrix(weights["uv_proj.weight"])
        self.w_uk = w_uk.view(self.nh, self.qd, self.rank)
        self.w_uv_t = w_uv.view(self.nh, self.vd, self.rank).transpose(1, 2)
        self.w_uk_flat, self.w_uv_flat = w_uk, w_uv      # [heads * qd, rank], [heads * vd, rank]
        # the head width of the prompt kernels that holds a key (unrotated and rotated part) and a value
        self.hw = next((w for w in (64, 128, 256) if w >= max(self.qd + self.rd, self.vd)), 0)
        self.w_o = rt.cast_matrix(weights["o_proj.weight"])
        self.sink = weights.get("sink")
        self._target_warps = _WARPS_PER_SM * rt.sm_count

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(kv=KVNeed(1, self.kw, self.window, values_in_keys=True))

    def _splits(self, ctx, capacity: int) -> int:
        """Runs of keys a (row, head) is cut into: as many as fill the device once, none
        shorter than 32 keys."""
        longest = (min(ctx.span or capacity, capacity)) if ctx.graph_capture else ctx.max_end
        if self.window > 0:
            longest = min(longest, self.window)
        want = max(1, self._target_warps // max(1, ctx.n_rows * self.nh))
        return max(1, min(want, -(-longest // 32), 128))

    def _tile_splits(self, ctx, capacity: int) -> int:
        """Runs of keys a tile of the tensor-core kernel (one row's heads, 16 at a time) is
        cut into: as many as give every SM two blocks, none shorter than 64 keys."""
        longest = (min(ctx.span or capacity, capacity)) if ctx.graph_capture else ctx.max_end
        if self.window > 0:
            longest = min(longest, self.window)
        tiles = ctx.n_rows * (-(-self.nh // 16))
        want = max(1, (2 * self.rt.sm_count) // max(1, tiles))
        return max(1, min(want, -(-longest // 64), 128))

    def _project(self, x: torch.Tensor):
        """(rows that begin with the query heads, the down projection's rows where they do not
        follow the query heads or None, the gates' columns or None)."""
        rt, tail = self.rt, self.rank + self.rd
        first = rt.linear(x, self.w_in)
        rt.flush()
        if not self.q_rank:
            gate = first[:, self.n_q + tail:self.n_q + tail + self.nh] if self.head_gate else None
            return first, None, gate
        # the queries' own latent: normed in 32-bit, then up to the heads
        cq = torch.empty((x.shape[0], self.q_rank), dtype=first.dtype, device=first.device)
        native.rms_norm(first[:, :self.q_rank], self.q_gain, self.eps, cq)
        q = rt.linear(cq, self.w_uq)
        rt.flush()
        at = self.q_rank + tail
        return q, first[:, self.q_rank:at], first[:, at:at + self.nh] if self.head_gate else None

    def _attend_expanded(self, proj: torch.Tensor, down, gate, ctx, view) -> torch.Tensor:
        """Long prompts in bfloat16: the latent rows are normed, rotated and cached as ever, and
        for the step's own rows keys and values are made per head (k_h = U_h c, v_h = V_h c:
        two library products) and attended over by the tcgen05 prompt kernel, with the sink as
        one more term of its last division: a third of the operations of the scores against
        the latent, on the faster tensor-core path.  Later steps read the cached latent rows."""
        rt, nh, qd, rd, vd, rank, kw, hw = self.rt, self.nh, self.qd, self.rd, self.vd, self.rank, self.kw, self.hw
        R = proj.shape[0]
        k_rows = torch.empty((R, kw), dtype=proj.dtype, device=proj.device)
        native.latent_prepare(proj, None, None, k_rows, self.c_gain, self.eps, self.inv_freq, self.rot,
                              ctx, view.k, view.page_table, view.page_tokens, view.ring_tokens, nh, qd, rd,
                              rank, kw, down)
        c_rows = k_rows[:, :rank]
        with native.profile_region("library product (latent rows to keys and values)",
                                   (nh * (qd + vd) * rank + R * (rank + nh * (qd + vd))) * proj.element_size(),
                                   2.0 * R * nh * (qd + vd) * rank):
            k_heads = torch.matmul(c_rows, self.w_uk_flat.t())
            v_heads = torch.matmul(c_rows, self.w_uv_flat.t())
        qkv = torch.empty((R, 3 * nh * hw), dtype=proj.dtype, device=proj.device)
        native.latent_expand(proj, k_rows, k_heads, v_heads, qkv, self.inv_freq, self.rot, ctx.row_pos,
                             nh, qd, rd, vd, rank, kw, hw)
        out = torch.empty((R, nh * hw), dtype=proj.dtype, device=proj.device)
        lens = None if ctx.graph_capture else ctx.counts
        n_items = 0
        if lens is not None:
            n_items, need, n_tickets = native.attention_prefill_tc_plan(lens, nh, nh, hw, self.window)
        if n_items == 0:
            lens = None
            need, n_tickets = native.attention_prefill_tc_split(ctx.n_seqs, ctx.max_count, nh, nh, hw)
        native.attention_prefill_tc(qkv, out, ctx.seq_row0, ctx.seq_end, ctx.n_seqs, ctx.max_count, nh, nh,
                                    hw, self.scale, 0.0, self.window, rt.scratch(need) if need else None,
                                    rt.tickets(n_tickets) if need else None, lens, sink=self.sink)
        vals = torch.empty((R, nh * vd), dtype=out.dtype, device=out.device)
        native.head_gate(out, gate, vals, nh, vd, hw)
        return rt.linear(vals, self.w_o)

    def forward(self, x: torch.Tensor, ctx, entry: int, cache_entry: int,
                owns_cache: bool) -> torch.Tensor:
        if not owns_cache:
            raise ValueError("latent_attention: reading another run's cache is not built")
        rt, nh, qd, rd, rank, kw = self.rt, self.nh, self.qd, self.rd, self.rank, self.kw
        R = x.shape[0]
        view = ctx.kv(cache_entry)
        fresh = ctx.all_from_start
        if not fresh and view.ring_tokens > 0 and not ctx.graph_capture:
            room = view.ring_tokens - self.window + 1
            for start, n in zip(ctx.starts, ctx.counts):
                if n > room and start + n > view.ring_tokens:
                    raise ValueError(
                        f"a step may add at most {max(room, view.ring_tokens - start)} positions "
                        f"to a sequence of {start} whose layers keep a window of {self.window} "
                        f"in a ring of {view.ring_tokens}; got {n}")
        proj, down, gate = self._project(x)
        if (fresh and proj.dtype == torch.bfloat16 and _USE_LATENT_EXPAND and _USE_TCGEN05_PREFILL
                and self.hw and self.scale > 0 and ctx.max_count > rt.short_prompt_tokens
                and native.attention_prefill_tc_supports(nh, nh, self.hw, 3 * nh * self.hw)):
            return self._attend_expanded(proj, down, gate, ctx, view)
        # the unrotated query columns of every head into the latent's space: [heads, rows, rank]
        q_heads = proj[:, :self.n_q].view(R, nh, qd + rd)[:, :, :qd].transpose(0, 1)
        with native.profile_region("library product (queries into the latent space)",
                                   (nh * qd * rank + R * nh * (qd + rank)) * proj.element_size(),
                                   2.0 * R * nh * qd * rank):
            q_lat = torch.bmm(q_heads, self.w_uk)
        q_rows = torch.empty((R, nh * kw), dtype=proj.dtype, device=proj.device)
        k_rows = torch.empty((R, kw), dtype=proj.dtype, device=proj.device)
        native.latent_prepare(proj, q_lat, q_rows, k_rows, self.c_gain, self.eps, self.inv_freq,
                              self.rot, ctx, view.k, view.page_table, view.page_tokens,
                              view.ring_tokens, nh, qd, rd, rank, kw, down)
        out = torch.empty((R, nh * kw), dtype=proj.dtype, device=proj.device)
        tensor_cores = (proj.dtype == torch.bfloat16 and _USE_LATENT_MMA
                        and native.attention_latent_supports(nh, kw))
        if fresh and tensor_cores:
            native.attention_latent(q_rows, k_rows, None, None, view.page_tokens, view.ring_tokens, ctx,
                                    out, None, self.sink, nh, kw, self.scale, self.window, 1,
                                    rows_per_tile=max(1, 16 // nh))
        elif tensor_cores:
            splits = self._tile_splits(ctx, ctx.cache.max_seq_len)
            scratch = None
            if splits > 1:
                scratch = rt.scratch(native.attention_rows_scratch_bytes(R, nh, kw, splits))
            native.attention_latent(q_rows, None, view.k, view.page_table, view.page_tokens,
                                    view.ring_tokens, ctx, out, scratch, self.sink, nh, kw, self.scale,
                                    self.window, splits)
        elif fresh:
            native.attention_rows(q_rows, nh * kw, k_rows, k_rows, kw, None, None, None,
                                  view.page_tokens, view.ring_tokens, ctx.row_pos, ctx.row_seq,
                                  ctx.seq_slot, ctx.seq_start, ctx.seq_row0, out, None, nh, 1, kw,
                                  self.scale, 0.0, self.window, 1, sink=self.sink, values_in_keys=True)
        else:
            splits = self._splits(ctx, ctx.cache.max_seq_len)
            scratch = None
            if splits > 1:
                scratch = rt.scratch(native.attention_rows_scratch_bytes(R, nh, kw, splits))
            native.attention_rows(q_rows, nh * kw, None, None, kw, view.k, view.k, view.page_table,
                                  view.page_tokens, view.ring_tokens, ctx.row_pos, ctx.row_seq,
                                  ctx.seq_slot, ctx.seq_start, ctx.seq_row0, out, scratch, nh, 1, kw,
                                  self.scale, 0.0, self.window, splits, sink=self.sink,
                                  values_in_keys=True)
        # the heads' summed latents (gated), then V_h per head
        lat = torch.empty((R, nh * rank), dtype=out.dtype, device=out.device)
        native.head_gate(out, gate, lat, nh, rank, kw)
        with native.profile_region("library product (summed latents to values)",
                                   (nh * self.vd * rank + R * nh * (self.vd + rank)) * out.element_size(),
                                   2.0 * R * nh * self.vd * rank):
            vals = torch.bmm(lat.view(R, nh, rank).transpose(0, 1), self.w_uv_t)     # [heads, rows, vd]
            vals = vals.transpose(0, 1).reshape(R, nh * self.vd)
        return rt.linear(vals, self.w_o)


register_mixer("attention", Attention)
register_mixer("latent_attention", LatentAttention)
