"""Block arrangements: how norms, mixer, feed-forward and the residual stream
are put together.

``sandwich`` (norm before and after each sub-layer; the post norm comes
before the add, as in src/model/layer.rs:1101-1192):

    h += post_mixer(mixer(pre_mixer(h)))
    h += post_feed_forward(feed_forward(pre_feed_forward(h)))

``pre_norm`` is the same arrangement without the two post norms.  ``residual_scale`` m (a
block parameter, 1 unless a layer names it): what a sub-layer adds is multiplied by m,
h += m * post(sublayer(pre(h))); the Dynamic Tanh residual kernel and the unfused steps take
it.  A layer without a
feed-forward (``feed_forward`` None) has the first line only.  A site whose norm is the
``identity`` norm passes the stream's rows on as they are, which gives the arrangement
that norms a sub-layer's output only: h += post(sublayer(h)).  The
residual stream h is kept and summed in 32-bit.  When the norms around an
add are RMS norms the block runs "norm of the sub-layer's output, add, norm
for the next sub-layer" as one kernel (csrc/norm.cu add_rms_norm), reaching
over to the next block's first norm when the model passes it; Dynamic Tanh norms around an
add are fused in the same way (add_dyt_norm).

``parallel`` (one norm, both sub-layers read its output, one add):

    n = pre_mixer(h);   h += mixer(n) + feed_forward(n)

A block may carry a *tail* (a registered "tail" part, such as ``token_side``): it runs behind
the sub-layers on the stream itself, and its output passes an RMS norm with the tail's own
weight before it is added: y = tail(h); h += y / rms(y) * tail.gain.  That norm, the add and
the next block's first norm are one launch of the residual kernel.
"""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config.spec import ConfigError
from ..kernels import native
from .registry import register_block


def _fusable(norm) -> bool:
    return norm is None or getattr(norm, "fusable_rms", False)


def _fusable_dyt(norm) -> bool:
    return norm is None or getattr(norm, "fusable_dyt", False)


class SandwichBlock:
    norm_sites = ("pre_mixer", "post_mixer", "pre_feed_forward", "post_feed_forward")
    required_sites = ("pre_mixer", "pre_feed_forward")

    def __init__(self, mixer, feed_forward, norms: Mapping[str, object], rt,
                 residual_scale: float = 1.0):
        self.residual_scale = float(residual_scale)
        for site in self.required_sites:
            if norms.get(site) is None and (feed_forward is not None or site == "pre_mixer"):
                raise ConfigError(f"block: the '{site}' norm is required")
        self.mixer = mixer
        self.feed_forward = feed_forward       # None: the layer is its mixer alone
        self.pre_mixer = norms["pre_mixer"]
        self.post_mixer = norms.get("post_mixer")
        self.pre_ff = norms.get("pre_feed_forward")
        self.post_ff = norms.get("post_feed_forward")
        self.rt = rt

    @property
    def first_norm(self):
        return self.pre_mixer

    @property
    def chain_safe(self) -> bool:
        """Whether this block may run while few-row steps are deferred into a chain
        (parts/base.py Runtime.chaining): its mixer and feed-forward promise to touch
        deferred results through the runtime and ``kernels.native`` only, and its norms are
        the kind the residual kernel applies."""
        norms = (self.pre_mixer, self.post_mixer, self.pre_ff, self.post_ff)
        return (self.residual_scale == 1.0 and getattr(self.mixer, "chain_safe", False)
                and getattr(self.feed_forward, "chain_safe", False)
                and all(_fusable(n) and (n is None or n.gain is not None) for n in norms))

    @property
    def captures_prompts(self) -> bool:
        """Whether a recorded step of prompts of this block may be replayed for other prompts:
        its mixer and feed-forward promise to read sequences, slots and counts on the
        device only (the block itself and the norms work row by row)."""
        return (getattr(self.mixer, "captures_prompts", False)
                and (self.feed_forward is None
                     or getattr(self.feed_forward, "captures_prompts", False)))

    def _add_then_norm(self, y: torch.Tensor, post, h: torch.Tensor, nxt) -> Optional[torch.Tensor]:
        """h += residual_scale * post(y) (or y); returns nxt(h) if nxt is given."""
        if _fusable(post) and _fusable(nxt) and self.residual_scale == 1.0:
            out = torch.empty_like(y) if nxt is not None else None
            self.rt.add_rms_norm(y, post.gain if post is not None else None,
                                 post.eps if post is not None else 0.0, h,
                                 nxt.gain if nxt is not None else None,
                                 nxt.eps if nxt is not None else 0.0, out)
            return out
        if _fusable_dyt(post) and _fusable_dyt(nxt):
            # Dynamic Tanh on both sides of the add: the same step as one element-wise kernel
            self.rt.flush()
            out = torch.empty_like(y) if nxt is not None else None
            native.add_dyt_norm(y, post.triple if post is not None else None, h,
                                nxt.triple if nxt is not None else None, out, self.residual_scale)
            return out
        self.rt.flush()         # the steps below read y and h outside the chain
        if post is not None:
            y = post.forward(y, out_dtype=torch.float32)
        h.add_(y.to(torch.float32), alpha=self.residual_scale)
        return nxt.forward(h, out_dtype=self.rt.dtype) if nxt is not None else None

    def forward(self, h: torch.Tensor, normed: Optional[torch.Tensor], ctx, entry: int,
                cache_entry: int, owns_cache: bool, next_norm=None) -> Optional[torch.Tensor]:
        if normed is None:
            self.rt.flush()
            normed = self.pre_mixer.forward(h, out_dtype=self.rt.dtype)
        a = self.mixer.forward(normed, ctx, entry, cache_entry, owns_cache)
        if self.feed_forward is None:
            return self._add_then_norm(a, self.post_mixer, h, next_norm)
        n2 = self._add_then_norm(a, self.post_mixer, h, self.pre_ff)
        f = self.feed_forward.forward(n2, ctx)
        return self._add_then_norm(f, self.post_ff, h, next_norm)


class PreNormBlock(SandwichBlock):
    norm_sites = ("pre_mixer", "pre_feed_forward")


register_block("sandwich", SandwichBlock)
register_block("pre_norm", PreNormBlock)


class ParallelBlock:
    norm_sites = ("pre_mixer",)

    def __init__(self, mixer, feed_forward, norms: Mapping[str, object], rt, tail=None):
        if norms.get("pre_mixer") is None:
            raise ConfigError("block: the 'pre_mixer' norm is required")
        self.mixer = mixer
        self.feed_forward = feed_forward       # None: the layer is its mixer alone
        self.pre_mixer = norms["pre_mixer"]
        self.tail = tail
        self.rt = rt

    @property
    def first_norm(self):
        return self.pre_mixer

    chain_safe = False

    @property
    def captures_prompts(self) -> bool:
        return all(p is None or getattr(p, "captures_prompts", False)
                   for p in (self.mixer, self.feed_forward, self.tail)) and self.mixer is not None

    def _add(self, y: torch.Tensor, post, h: torch.Tensor, nxt, want_rows: bool = False):
        """h += y (normed by ``post``'s gain if given); returns nxt(h), or h's rows as
        activations when ``want_rows``, or None."""
        out = torch.empty_like(y) if (nxt is not None or want_rows) else None
        if _fusable(nxt):
            self.rt.add_rms_norm(y, post.gain if post is not None else None,
                                 post.eps if post is not None else 0.0, h,
                                 nxt.gain if nxt is not None else None,
                                 nxt.eps if nxt is not None else 0.0, out)
            return out
        self.rt.add_rms_norm(y, post.gain if post is not None else None,
                             post.eps if post is not None else 0.0, h, None, 0.0, None)
        return nxt.forward(h, out_dtype=self.rt.dtype)

    def forward(self, h: torch.Tensor, normed: Optional[torch.Tensor], ctx, entry: int,
                cache_entry: int, owns_cache: bool, next_norm=None) -> Optional[torch.Tensor]:
        if normed is None:
            self.rt.flush()
            normed = self.pre_mixer.forward(h, out_dtype=self.rt.dtype)
        a = self.mixer.forward(normed, ctx, entry, cache_entry, owns_cache)
        f = self.feed_forward.forward(normed, ctx) if self.feed_forward is not None else None
        if self.tail is None:
            if f is not None:
                self._add(a, None, h, None)
                return self._add(f, None, h, next_norm)
            return self._add(a, None, h, next_norm)
        # the sums go into the 32-bit stream; the tail reads the stream's rows as activations
        if f is not None:
            self._add(a, None, h, None)
            x = self._add(f, None, h, None, want_rows=True)
        else:
            x = self._add(a, None, h, None, want_rows=True)
        y = self.tail.forward(x, ctx)
        return self._add(y, self.tail, h, next_norm)


register_block("parallel", ParallelBlock)
