"""Token embedding and the output head.

Embedding: row gather, then a multiply by ``scale`` (the 32-bit residual
stream starts here).  Reference: src/model/layer.rs:1279-1288.  With ``side_width`` S > 0
the token also picks a row of a second table ``side.weight`` ``[vocab, S]``, left for the
layers as ``ctx.memo["token_side"]`` (32-bit; parts/pair.py ``token_side`` reads its slice).

``bigram_embedding``: the token's row times ``scale`` plus a row of a second table picked
by a hash of the previous token and the token, (prev * mul_prev + token * mul_cur) mod
``buckets``; a sequence's first token takes the table's last row (number ``buckets``).  The
previous token of a step's first row is per-slot state (``state_need``), kept by the cache.
An optional ``norm`` (a PartSpec) is applied to the sum, in 32-bit.

``stream_mix`` (a "joint"): h <- W [h | x0] with one matrix of [hidden, 2 hidden], h
first: the stream mixed with another one of the same width (the embedding's output, at the
start of every pass of a model whose layers are walked several times).

Head: the product of the (final-normed) wanted rows with the output matrix,
which is the embedding table when ``tied`` (src/engine/generate.rs:1106-1110),
then ``cap * tanh(logits / cap)`` when ``logit_softcap`` > 0.  Logits are
32-bit.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import native
from ..weights.arena import Piece, Resident
from ..weights.loader import TensorDecl
from ..cache.paged import StateNeed
from ..config.spec import PartSpec
from ..weights.arena import resident_of
from .registry import part_class, register_embedding, register_head, register_joint


class TokenEmbedding:
    captures_prompts = True   # row-wise: a recorded step of prompts may be replayed for others

    @staticmethod
    def tensors(params: Mapping, hidden: int, vocab: int) -> Dict[str, TensorDecl]:
        out = {"weight": TensorDecl((vocab, hidden))}
        if int(params.get("side_width") or 0) > 0:
            out["side.weight"] = TensorDecl((vocab, int(params["side_width"])))
        return out

    @staticmethod
    def resident(params: Mapping, hidden: int, vocab: int) -> Dict[str, Resident]:
        out = {"weight": Resident((vocab, hidden), pieces=(Piece("weight"),))}
        if int(params.get("side_width") or 0) > 0:
            out["side.weight"] = Resident((vocab, int(params["side_width"])), pieces=(Piece("side.weight"),))
        return out

    def __init__(self, params: Mapping, hidden: int, vocab: int,
                 weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.hidden = hidden
        self.vocab = vocab
        self.scale = float(params.get("scale", 1.0))
        self.table = rt.cast_matrix(weights["weight"])
        self.side = rt.cast_matrix(weights["side.weight"]) if "side.weight" in weights else None

    def forward(self, ctx) -> torch.Tensor:
        """The step's rows of the 32-bit residual stream.  An embedding gets the whole
        step context: one that adds learned positions reads ``ctx.row_pos`` too."""
        tokens = ctx.tokens
        if self.side is not None:
            rows = torch.empty((tokens.numel(), self.side.shape[1]), dtype=torch.float32,
                               device=tokens.device)
            ctx.memo["token_side"] = native.embed_rows(tokens, self.side, 1.0, rows)
        h = torch.empty((tokens.numel(), self.hidden), dtype=torch.float32, device=tokens.device)
        return native.embed_rows(tokens, self.table, self.scale, h)


class BigramEmbedding:
    captures_prompts = True   # sequences and slots are read on the device only

    @staticmethod
    def _norm(params: Mapping):
        norm: Optional[PartSpec] = params.get("norm")
        return (norm, part_class("norm", norm.kind)) if norm is not None else (None, None)

    @classmethod
    def tensors(cls, params: Mapping, hidden: int, vocab: int) -> Dict[str, TensorDecl]:
        out = {"weight": TensorDecl((vocab, hidden)),
               "bigram.weight": TensorDecl((int(params["buckets"]) + 1, hidden))}
        norm, ncls = cls._norm(params)
        if norm is not None:
            out.update({"norm." + n: d for n, d in ncls.tensors(norm.params, hidden).items()})
        return out

    @classmethod
    def resident(cls, params: Mapping, hidden: int, vocab: int) -> Dict[str, Resident]:
        out = {"weight": Resident((vocab, hidden), pieces=(Piece("weight"),)),
               "bigram.weight": Resident((int(params["buckets"]) + 1, hidden),
                                         pieces=(Piece("bigram.weight"),))}
        norm, ncls = cls._norm(params)
        if norm is not None:
            for name, res in resident_of(ncls, ncls.tensors(norm.params, hidden), norm.params, hidden).items():
                out["norm." + name] = Resident(res.shape, res.dtype, tuple(
                    Piece("norm." + q.source, q.row_offset, q.group, q.group_stride)
                    for q in res.pieces), res.offset)
        return out

    def __init__(self, params: Mapping, hidden: int, vocab: int,
                 weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.hidden = hidden
        self.vocab = vocab
        self.scale = float(params.get("scale", 1.0))
        self.buckets = int(params["buckets"])
        self.mul_prev, self.mul_cur = int(params["mul_prev"]), int(params["mul_cur"])
        self.table = rt.cast_matrix(weights["weight"])
        self.bigram = rt.cast_matrix(weights["bigram.weight"])
        norm, ncls = self._norm(params)
        self.norm = None
        if norm is not None:
            self.norm = ncls(norm.params, hidden, {k[len("norm."):]: v for k, v in weights.items()
                                                   if k.startswith("norm.")}, rt)

    @staticmethod
    def state_need() -> StateNeed:
        """One token id per slot: the sequence's last token."""
        return StateNeed((1,), torch.int32)

    def forward(self, ctx) -> torch.Tensor:
        h = torch.empty((ctx.tokens.numel(), self.hidden), dtype=torch.float32, device=ctx.tokens.device)
        native.bigram_embed(ctx, self.table, self.bigram, ctx.cache.named_state("embedding"), h,
                            self.scale, self.buckets, self.mul_prev, self.mul_cur)
        if self.norm is None:
            return h
        return self.norm.forward(h, out_dtype=torch.float32)


class StreamMix:
    captures_prompts = True   # row-wise

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((hidden, 2 * hidden))}

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        return {"weight": Resident((hidden, 2 * hidden), pieces=(Piece("weight"),))}

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.hidden = hidden
        self.weight = rt.cast_matrix(weights["weight"])

    def forward(self, h: torch.Tensor, x0: torch.Tensor) -> torch.Tensor:
        """h, x0: 32-bit ``[rows, hidden]``; returns the new 32-bit stream."""
        both = torch.empty((h.shape[0], 2 * self.hidden), dtype=self.rt.dtype, device=h.device)
        native.pair_rows(h, x0, both)
        return self.rt.linear(both, self.weight, out_dtype=torch.float32)


class LMHead:
    @staticmethod
    def tensors(params: Mapping, hidden: int, vocab: int) -> Dict[str, TensorDecl]:
        # a tied head uses the embedding's table; a file that stores the head's matrix
        # all the same is accepted and that tensor is not read
        return {"weight": TensorDecl((vocab, hidden), optional=bool(params.get("tied", True)))}

    @staticmethod
    def resident(params: Mapping, hidden: int, vocab: int) -> Dict[str, Resident]:
        if params.get("tied", True):
            return {}
        return {"weight": Resident((vocab, hidden), pieces=(Piece("weight"),))}

    def __init__(self, params: Mapping, hidden: int, vocab: int,
                 weights: Mapping[str, torch.Tensor], rt, embedding: Optional[TokenEmbedding]):
        self.rt = rt
        self.cap = float(params.get("logit_softcap") or 0.0)
        if params.get("tied", True):
            if embedding is None:
                raise ValueError("a tied head needs the embedding")
            self.weight = embedding.table
        else:
            self.weight = rt.cast_matrix(weights["weight"])

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        """y[n, hidden] in the activation type -> logits[n, vocab] in 32-bit."""
        epi = native.EPI_SOFTCAP if self.cap > 0 else native.EPI_NONE
        return self.rt.linear(y, self.weight, out_dtype=torch.float32, epilogue=epi, cap=self.cap)


register_embedding("token_embedding", TokenEmbedding)
register_embedding("bigram_embedding", BigramEmbedding)
register_joint("stream_mix", StreamMix)
register_head("lm_head", LMHead)
