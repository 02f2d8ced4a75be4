"""Small Gegorax configurations for the tests, random weights for them, and the comparison with
the plain model (tests/plain_gegorax.py)."""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

import plain_gegorax as plain


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit=2.0, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def parallel(heads, kv_heads, dim, vdim, window, pool, s_heads, s_vdim, state, groups=1, conv=4,
             norm_groups=1, scale=0.2, rot_dims=None, base=10000.0, mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": window, "pool": pool},
            "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}}
    right = {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "conv": conv,
             "norm_groups": norm_groups}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def delta(heads, dim, mlp=None, rank=None):
    mixer = {"heads": heads, "dim": dim}
    if rank:
        mixer["decay_rank"] = rank
    return {"type": "general_delta", "mixer": mixer, "mlp": mlp}


def model(width, vocab, layers, side=8, eps=1e-5):
    cfg = {"architecture": "Gegorax", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": list(layers)}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


# one layer of each kind alone, with each feed-forward and with none
ALONE = {
    "parallel": model(64, 150, [parallel(4, 2, 16, 24, 20, 4, 4, 8, 16, groups=2, norm_groups=2)]),
    "parallel_dense": model(64, 150, [parallel(2, 1, 32, 16, 33, 8, 2, 16, 8, mlp=dense(96))], side=0),
    "delta": model(64, 150, [delta(2, 16)]),
    "delta_moe": model(64, 150, [delta(4, 8, mlp=moe(6, 2, 24, 1.5, shared=(40, 1.0)), rank=8)]),
    "delta_moe_bare": model(64, 150, [delta(1, 32, mlp=moe(5, 1, 16, 3.0))], side=0),
}

# both kinds of layers and of feed-forwards; windows shorter and longer than a page of 64 positions,
# blocks that divide the window, that do not, and one as long as the window
MIXED = model(64, 200, [
    parallel(4, 2, 16, 24, 40, 8, 4, 8, 16, groups=2, norm_groups=2, mlp=dense(96)),
    delta(2, 16, mlp=moe(8, 3, 24, 2.0, shared=(48, 1.5))),
    delta(4, 8, mlp=dense(64), rank=12),
    parallel(2, 2, 16, 16, 70, 12, 2, 16, 8, conv=3, rot_dims=8, scale=0.15, mlp=moe(4, 2, 32, 1.0)),
    parallel(3, 1, 16, 32, 16, 16, 3, 8, 24, conv=2, mlp=None),
], side=8)

# sizes that are no multiples of 16, 8 or 4; one head; one expert a row; blocks of one position;
# a window of one; a convolution of one tap; groups and parts as many as heads
ODD = model(72, 131, [
    parallel(3, 3, 10, 14, 33, 5, 3, 6, 7, groups=3, conv=1, norm_groups=3, rot_dims=4, mlp=dense(50)),
    delta(1, 20, mlp=moe(3, 1, 9, 0.7, shared=(11, 2.5)), rank=5),
    parallel(1, 1, 6, 5, 1, 1, 1, 9, 5, conv=5, scale=0.5),
    delta(3, 6, mlp=moe(7, 7, 10, 1.2), rank=3),
    parallel(2, 1, 12, 20, 7, 3, 4, 5, 10, groups=1, norm_groups=2, mlp=moe(2, 2, 6, 4.0, shared=(4, 0.5))),
], side=5, eps=1e-6)

# a width and a vocabulary that are multiples of 2 only; no token side
NARROW = model(100, 77, [
    delta(2, 12, mlp=dense(30), rank=4),
    parallel(2, 1, 12, 20, 50, 10, 2, 10, 6, conv=4, mlp=moe(4, 2, 14, 2.0, shared=(6, 1.0))),
], side=0)

# wide heads: the widest states and keys
WIDE = model(128, 300, [
    parallel(4, 2, 64, 128, 100, 32, 4, 64, 128, groups=2, norm_groups=4, scale=0.09, base=500000.0, mlp=dense(128)),
    delta(2, 128, mlp=moe(4, 2, 64, 2.0, shared=(64, 2.0)), rank=32),
    parallel(2, 1, 256, 64, 150, 64, 8, 32, 64, groups=1, rot_dims=64, scale=0.06),
], side=16)

# attention with a scale that makes the softmax pick single keys or blocks
SHARP = model(64, 200, [
    parallel(4, 2, 16, 24, 66, 8, 2, 8, 8, scale=1.5, mlp=dense(32)),
    parallel(2, 1, 16, 16, 30, 16, 2, 8, 8, scale=1.5),
], side=0)

REL_TOL = {"float32": 1e-4, "bfloat16": 4e-2}
# 32-bit: one row in a hundred may lie above the tolerance (a head whose output nearly cancels
# before it is divided by its root mean square enlarges the rounding of its inputs), none above
# five times it.  bfloat16: the typical row, the share of rows over the tolerance and every row
# loosely; the 32-bit runs (the same kernels' other instantiation) bound every row tightly.
F32_ROWS_OVER, F32_WORST = 0.01, 5.0
BF16_MEDIAN, BF16_ROWS_OVER, BF16_WORST = 2.5e-2, 0.3, 0.9


def prompts(cfg: dict, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


def random_weights(config: dict, seed: int, std: float = 0.5) -> Dict[str, torch.Tensor]:
    """Random tensors of every name the configuration asks for, rounded to bfloat16 values."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]
    side = (config.get("token_side") or {}).get("dim", 0)

    def mat(o, i, s=1.0):
        return torch.randn((o, i), generator=g) * (s * std / math.sqrt(i))

    def vec(n, s=0.3, at=0.0):
        return torch.randn((n,), generator=g) * s + at

    out: Dict[str, torch.Tensor] = {"embed": torch.randn((config["vocab"], W), generator=g)}
    if side:
        out["side.embed"] = torch.randn((config["vocab"], side * len(config["layers"])), generator=g)
    for i, layer in enumerate(config["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        out[f"l{i}.norm1"] = vec(W, 0.3, 1.0)
        if layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            out[pre + "left.q"], out[pre + "left.k"] = mat(H * D, W, 2.0), mat(G * D, W, 2.0)
            out[pre + "left.v"], out[pre + "left.o"] = mat(G * V, W, 2.0), mat(W, H * V, 2.0)
            out[pre + "left.q.norm"], out[pre + "left.k.norm"] = vec(D, 0.3, 1.0), vec(D, 0.3, 1.0)
            SH, P, N, SG = b["heads"], b["vdim"], b["state"], b["groups"]
            inner, ch = SH * P, SH * P + 2 * SG * N
            out[pre + "right.in"] = mat(inner + ch + SH, W, 2.0)
            out[pre + "right.conv"] = torch.randn((ch, b["conv"]), generator=g) * 0.6
            out[pre + "right.conv.b"] = vec(ch, 0.2)
            out[pre + "right.dt_bias"], out[pre + "right.A_log"] = vec(SH, 0.7, -1.0), vec(SH, 0.7, -0.5)
            out[pre + "right.D"], out[pre + "right.norm"] = vec(SH, 0.5, 0.5), vec(inner, 0.3, 1.0)
            out[pre + "right.o"] = mat(W, inner, 2.0)
            out[pre + "left.out"], out[pre + "right.out"] = vec(W, 0.3, 1.0), vec(W, 0.3, 1.0)
        else:
            H, D = m["heads"], m["dim"]
            rank = m.get("decay_rank", 16)
            for n in "rkvga":
                out[pre + n] = mat(H * D, W, 2.0)
            out[pre + "a.b"], out[pre + "w0"] = vec(H * D, 0.5), vec(H * D, 1.0, 0.5)
            out[pre + "w1"], out[pre + "w2"] = mat(rank, W, 2.0), mat(H * D, rank, 3.0)
            out[pre + "norm"], out[pre + "o"] = vec(H * D, 0.3, 1.0), mat(W, H * D, 2.0)
        mlp = layer.get("mlp")
        if mlp and mlp["kind"] == "dense":
            out[f"l{i}.mlp.up"], out[f"l{i}.mlp.down"] = mat(mlp["ff"], W, 2.0), mat(W, mlp["ff"], 2.0)
        elif mlp:
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            out[f"l{i}.mlp.router"], out[f"l{i}.mlp.router.b"] = mat(E, W, 4.0), vec(E, 0.5)
            names = [f"e{e}" for e in range(E)] + (["shared"] if mlp.get("shared") else [])
            for n in names:
                f = mlp["shared"]["ff"] if n == "shared" else F
                out[f"l{i}.mlp.{n}.gate"], out[f"l{i}.mlp.{n}.up"] = mat(f, W, 3.0), mat(f, W, 3.0)
                out[f"l{i}.mlp.{n}.down"] = mat(W, f, 2.0)
        if side:
            out[f"l{i}.side.gate"], out[f"l{i}.side.proj"] = mat(side, W, 2.0), mat(W, side, 2.0)
            out[f"l{i}.side.norm"] = vec(W, 0.2, 0.5)
    out["final.norm"] = vec(W, 0.3, 1.0)
    out["head"] = mat(config["vocab"], W, 3.0)
    return {n: t.to(torch.bfloat16).to(torch.float32) for n, t in out.items()}


def plain_logits(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    w = {n: t.to(torch.float64).numpy() for n, t in weights.items()}
    return torch.from_numpy(np.ascontiguousarray(plain.logits(cfg, w, list(tokens))))


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str) -> None:
    """Rows of logits against the plain model's: the largest difference as a fraction of the
    largest plain logit of the compared rows."""
    got = got.detach().to("cpu", torch.float64)
    ref = ref.to(torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = ref.abs().max().item()
    diff = (got - ref).abs().amax(dim=-1)
    bad = (diff > REL_TOL[dtype] * scale).nonzero()
    text = (f"{what}: max |diff| {diff.max().item():.3e}, median {diff.median().item():.3e}, "
            f"{bad.numel()} of {got.shape[0]} rows over {REL_TOL[dtype]:.0e} x max|ref| {scale:.3e}"
            + (f"; first of them row {int(bad[0])}" if bad.numel() else ""))
    if dtype == "float32":
        assert bad.numel() <= int(F32_ROWS_OVER * got.shape[0] + 0.99), text
        assert diff.max().item() <= F32_WORST * REL_TOL[dtype] * scale, text
    elif got.shape[0] < 8:
        assert diff.max().item() <= BF16_WORST * scale, text
    else:
        assert diff.median().item() <= BF16_MEDIAN * scale, text
        assert bad.numel() <= max(1, BF16_ROWS_OVER * got.shape[0]), text
        assert diff.max().item() <= BF16_WORST * scale, text


def rows_that_differ(a: torch.Tensor, b: torch.Tensor, factor: float = 100.0) -> int:
    """How many rows of two plain results differ by more than ``factor`` times the 32-bit
    tolerance: what a test needs to be able to tell the two apart."""
    scale = a.abs().max().item()
    return int(((a - b).abs().amax(dim=-1) > factor * REL_TOL["float32"] * scale).sum())


# ---- blocks that carry a row's weight ----------------------------------------------------------
# One layer, so that a key is a function of its token alone; few rotated columns, so that the
# mean key of a block of equal tokens is (nearly) that token's key; queries made by the keys'
# matrix, so that a row's score is largest for keys of its own token.  In ``asking_prompt``
# every block repeats one token of its own, and now and then a row carries the token of an
# earlier block that has just come into sight as a block or is about to: whether that block
# is seen decides where the row's weight goes.

def blocks_model(window, pool, heads=2, dim=16, vdim=24, rot_dims=2, scale=0.3):
    return model(64, 260, [parallel(heads, heads, dim, vdim, window, pool, 2, 8, 8, scale=scale,
                                    rot_dims=rot_dims)], side=0)


BLOCKS = {
    "blocks_in_window": blocks_model(20, 8),
    "block_longer_than_window": blocks_model(10, 24, heads=1),
    "blocks_astride_pages": blocks_model(70, 12, dim=8, vdim=8),
    "blocks_of_four": blocks_model(9, 4),          # more than 64 blocks: a second page of cells
    "blocks_of_one": blocks_model(5, 1),
}
# heads of 64 and of 128 (values wider than keys): bfloat16 prompts take the tensor cores
BLOCKS_TC = {
    "blocks_heads_of_64": blocks_model(20, 8, dim=64, vdim=64, scale=0.1),
    "blocks_values_of_128": blocks_model(70, 12, heads=1, dim=64, vdim=128, scale=0.1),
}


def tie_queries_to_keys(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = dict(weights)
    out["l0.mix.left.q"] = weights["l0.mix.left.k"].clone()
    out["l0.mix.left.q.norm"] = weights["l0.mix.left.k.norm"].clone()
    return out


def asking_prompt(cfg: dict, length: int, seed: int) -> List[int]:
    """Rows at which a block has just come into sight often carry that block's token; rows one
    before often carry the token of the block that comes next (and must get nothing of it)."""
    mask = cfg["layers"][0]["mixer"]["left"]["mask"]
    window, pool = mask["size"], mask["pool"]
    g = torch.Generator().manual_seed(seed)
    own = lambda b: 3 + b % (cfg["vocab"] - 3)  # noqa: E731
    toks = []
    for i in range(length):
        behind = i - window + 1                        # positions that have left the window
        newest = behind // pool - 1                    # the last block that row i sees
        ask = newest >= 0 and torch.rand((), generator=g).item() < 0.6
        if ask and behind % pool == 0:
            toks.append(own(newest))
        elif ask and behind % pool == pool - 1:
            toks.append(own(newest + 1))
        else:
            toks.append(own(i // pool))
    return toks


def shifted_blocks(shift: int):
    """The plain attention with every row's blocks taken as if the row stood ``shift`` positions
    further on (0: as the design says; None: no blocks at all): what a kernel that is one
    position off, or that forgets the blocks, would compute."""
    def attention(q, k, v, scale, window, pool):
        T, H, _ = q.shape
        G = k.shape[1]
        out = np.zeros((T, H, v.shape[2]))
        for i in range(T):
            first = max(0, i - window + 1)
            blocks = 0 if shift is None else max(0, min((i + shift - window + 1) // pool, (i + 1) // pool))
            for h in range(H):
                kv = h // (H // G)
                keys = [k[b * pool:(b + 1) * pool, kv].mean(0) for b in range(blocks)] + list(k[first:i + 1, kv])
                vals = [v[b * pool:(b + 1) * pool, kv].mean(0) for b in range(blocks)] + list(v[first:i + 1, kv])
                s = np.array(keys) @ q[i, h] * scale
                p = np.exp(s - s.max())
                out[i, h] = (p / p.sum()) @ np.array(vals)
        return out
    return attention
