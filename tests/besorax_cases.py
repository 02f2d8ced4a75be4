"""Small Besorax configurations for the tests, random weights for them, and the comparison with
the plain model (tests/plain_besorax.py)."""

from __future__ import annotations

import copy
import math
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

import plain_besorax as plain


def dense(ff, limit=2.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, shared=0):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def attention(heads, kv_heads, dim, vdim, chunk, scale=0.2, rot_dims=None, base=10000.0, mlp=None, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims != 0:
        mixer["rot"] = {"base": base, "dims": dim if rot_dims is None else rot_dims}
    if chunk:
        mixer["mask"] = {"size": chunk}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale=0.2, base=10000.0, mlp=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": scale, "rot": {"base": base, "dims": rot_dim}}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def lightning(heads, dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def model(width, vocab, layers, eps=1e-5, scale=1.5, mult=0.6):
    return {"architecture": "Besorax", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": scale}, "residual_mult": mult, "layers": list(layers)}


# one mechanism at a time
ALONE = {
    "attention": model(64, 200, [attention(4, 2, 16, 16, 24)]),
    "attention_values": model(64, 200, [attention(4, 4, 16, 24, 40, rot_dims=8, mlp=dense(48))]),
    "attention_open": model(64, 200, [attention(3, 1, 32, 32, 0, rot_dims=0, mlp=dense(40, 0.7))]),
    "lender": model(64, 200, [attention(4, 2, 16, 16, 30, rot_dims=6), attention(4, 2, 16, 16, 30, rot_dims=6, kv_from=0)]),
    "latent": model(64, 200, [latent(4, 16, 8, 24, 32, 40)]),
    "latent_ff": model(64, 200, [latent(2, 32, 16, 16, 48, 24, mlp=moe(4, 2, 24, shared=16))]),
    "lightning": model(64, 200, [lightning(4, 16, 24, [0.9, 0.97, 0.99, 0.999])]),
    "lightning_ff": model(64, 200, [lightning(2, 32, 16, [0.95, 1.0], mlp=dense(56))]),
    "experts": model(64, 200, [lightning(2, 16, 16, [0.9, 0.99], mlp=moe(6, 3, 20))]),
    "experts_shared": model(64, 200, [attention(2, 2, 16, 16, 50, mlp=moe(5, 1, 12, shared=28))], mult=1.0),
}

# every mixer and feed-forward; chunks shorter and longer than a page of 64; the lender is not the layer
# before the borrower and lends twice; values wider and narrower than keys
MIXED = model(64, 200, [
    attention(4, 2, 16, 16, 40, rot_dims=8, mlp=dense(96)),
    lightning(4, 16, 24, [0.8, 0.95, 0.99, 0.999], mlp=moe(6, 2, 24, shared=32)),
    attention(4, 2, 16, 16, 40, rot_dims=8, kv_from=0, mlp=moe(4, 1, 32)),
    latent(3, 16, 8, 24, 32, 40, mlp=moe(8, 2, 16, shared=16)),
    attention(2, 1, 32, 48, 100, scale=0.15, mlp=dense(48, 1.0)),
    attention(4, 2, 16, 16, 70, rot_dims=8, kv_from=0),
])

# sizes that are no multiples of 16, 8 or 4; one head; a top as large as the number of experts
ODD = model(72, 131, [
    attention(3, 3, 10, 14, 7, rot_dims=6, mlp=moe(3, 3, 10)),
    latent(3, 10, 6, 14, 21, 13, mlp=dense(100, 4.0)),
    lightning(1, 20, 7, [0.99], mlp=moe(7, 2, 9, shared=5)),
    attention(3, 3, 10, 14, 33, rot_dims=6, kv_from=0, mlp=dense(36)),
    latent(1, 7, 2, 5, 9, 3, scale=0.5),
    lightning(3, 6, 9, [0.5, 0.9, 0.999]),
], eps=1e-6, scale=0.8, mult=1.0)

# wide heads and latents, heads of 128 and 256, a chunk of one position and one longer than any request
WIDE = model(128, 300, [
    attention(8, 2, 128, 128, 1, rot_dims=64, base=500000.0, scale=0.09, mlp=dense(128)),
    latent(4, 64, 32, 64, 192, 96, scale=0.09, base=500000.0, mlp=moe(4, 2, 64, shared=64)),
    lightning(2, 128, 64, [0.99, 0.999]),
    attention(2, 1, 256, 256, 5000, rot_dims=64, scale=0.06, mlp=moe(3, 1, 40)),
    attention(8, 2, 128, 128, 128, rot_dims=64, base=500000.0, scale=0.09, kv_from=0),
    latent(8, 128, 64, 128, 448, 128, scale=0.06),
], mult=0.4)

# attention with a scale that makes the softmax pick a few keys among those inside the chunk
SHARP = model(64, 200, [
    attention(4, 2, 16, 16, 100, scale=1.5, rot_dims=4),
    attention(4, 2, 16, 16, 100, scale=1.5, rot_dims=4, kv_from=0, mlp=dense(64)),
    attention(2, 2, 16, 24, 66, scale=1.2),
])

REL_TOL = {"float32": 1e-4, "bfloat16": 4e-2}
# 32-bit: a row in which the lightning heads' outputs nearly cancel before they are divided by their
# root mean square shows the 32-bit rounding of its inputs enlarged; one row in a hundred may lie above
# the tolerance, none above five times it.
F32_ROWS_OVER, F32_WORST = 0.01, 5.0
# bfloat16: a router's close call sends a row to another expert, and a lightning row that nearly cancels
# turns rounding into an error of any size: the bfloat16 runs bound the typical row, the share of rows
# over the tolerance and every row loosely, the 32-bit runs (the same kernels' other instantiation)
# every row tightly.
BF16_MEDIAN, BF16_ROWS_OVER, BF16_WORST = 2.5e-2, 0.3, 0.9


def prompts(cfg: dict, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


def random_weights(config: dict, seed: int, std: float = 0.5) -> Dict[str, torch.Tensor]:
    """Random tensors of every name the configuration asks for, rounded to bfloat16 values."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]

    def mat(o, i, s=1.0):
        return torch.randn((o, i), generator=g) * (s * std / math.sqrt(i))

    def vec(n, s=0.3, at=0.0):
        return torch.randn((n,), generator=g) * s + at

    out: Dict[str, torch.Tensor] = {}

    def norm(name):
        out[name], out[name + ".b"] = vec(W, 0.3, 1.0), vec(W, 0.1)
        out[name + ".alpha"] = (torch.rand((), generator=g) * 0.5 + 0.25)

    out["embed"] = torch.randn((config["vocab"], W), generator=g)
    for i, layer in enumerate(config["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        norm(f"l{i}.norm1")
        H, D, V = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            G = m.get("kv_heads") or H
            out[pre + "q"] = mat(H * D, W, 2.0)
            if m.get("kv_from") is None:
                out[pre + "k"], out[pre + "v"] = mat(G * D, W, 2.0), mat(G * V, W, 2.0)
            out[pre + "sink"] = vec(H, 1.0)
            out[pre + "o"] = mat(W, H * V, 2.0)
        elif layer["type"] == "latent_attention":
            R, rank, qr = m["rot_dim"], m["kv_rank"], m["q_rank"]
            out[pre + "dq"], out[pre + "dq.norm"] = mat(qr, W, 2.0), vec(qr, 0.3, 1.0)
            out[pre + "uq"] = mat(H * (D + R), qr, 2.0)
            out[pre + "dkv"], out[pre + "dkv.norm"] = mat(rank + R, W, 2.0), vec(rank, 0.3, 1.0)
            out[pre + "uk"], out[pre + "uv"] = mat(H * D, rank, 2.0), mat(H * V, rank, 2.0)
            out[pre + "sink"] = vec(H, 1.0)
            out[pre + "o"] = mat(W, H * V, 2.0)
        else:
            out[pre + "q"], out[pre + "k"] = mat(H * D, W, 2.0), mat(H * D, W, 2.0)
            out[pre + "v"], out[pre + "g"] = mat(H * V, W, 2.0), mat(H * V, W, 2.0)
            out[pre + "norm"] = vec(H * V, 0.3, 1.0)
            out[pre + "o"] = mat(W, H * V, 2.0)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        norm(f"l{i}.norm2")
        pre = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            out[pre + "gate"], out[pre + "up"], out[pre + "down"] = mat(F, W, 3.0), mat(F, W, 3.0), mat(W, F, 2.0)
            continue
        E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
        out[pre + "router"] = mat(E, W, 3.0)
        for e in range(E):
            out[pre + f"e{e}.up"], out[pre + f"e{e}.down"] = mat(F, W, 3.0), mat(W, F, 3.0)
        if mlp.get("shared"):
            S = mlp["shared"]["ff"]
            out[pre + "shared.up"], out[pre + "shared.down"] = mat(S, W, 3.0), mat(W, S, 2.0)
    norm("final.norm")
    out["head"] = mat(config["vocab"], W, 3.0)
    return {n: t.to(torch.bfloat16).to(torch.float32) for n, t in out.items()}


def plain_logits(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(plain.logits(cfg, weights, list(tokens))))


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


def changed(cfg: dict, edit) -> dict:
    other = copy.deepcopy(cfg)
    edit(other)
    return other


def decisive_routers(weights: Dict[str, torch.Tensor], factor: float = 6.0) -> Dict[str, torch.Tensor]:
    """The same weights with every router's matrix enlarged: the scores lie far apart, so that a
    bfloat16 run chooses the experts the plain model chooses."""
    return {n: (t * factor).to(torch.bfloat16).to(torch.float32) if n.endswith(".router") else t
            for n, t in weights.items()}


def random_model(seed: int) -> dict:
    """A configuration drawn from the design's whole range: any order of the three mixers, borrowers
    behind any lender, grouped and ungrouped heads of the fast kernels' widths and of others, values
    wider and narrower than keys, chunks of any length or none, every kind of feed-forward or none."""
    import random
    r = random.Random(seed)
    width, vocab = r.choice([64, 96, 128, 100, 36]), r.randrange(90, 300)

    def mlp():
        kind = r.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return dense(r.choice([24, 40, 100, 128]), r.choice([0.8, 2.5, 6.0]))
        experts = r.randrange(2, 10)
        return moe(experts, r.randrange(1, min(experts, 4) + 1), r.choice([8, 24, 40]), r.choice([0, 0, 16, 36]))
    layers, lenders = [], []
    for i in range(r.randrange(3, 7)):
        kind = r.choice(["attention", "attention", "latent", "lightning"])
        if kind == "attention" and lenders and r.random() < 0.7:
            j = r.choice(lenders)
            m = layers[j]["mixer"]
            layers.append(attention(m["heads"], m["kv_heads"], m["dim"], m["vdim"], r.choice([0, 5, 16, 37, 64, 100]),
                                    scale=r.choice([0.1, 0.3]), rot_dims=m["rot"]["dims"] if m.get("rot") else 0,
                                    base=m["rot"]["base"] if m.get("rot") else 10000.0, mlp=mlp(), kv_from=j))
        elif kind == "attention":
            kv = r.choice([1, 2, 4])
            heads = kv * r.choice([1, 2, 4])
            dim = r.choice([16, 32, 64, 64, 128, 24])
            vdim = r.choice([dim, dim, dim, 16, 48, 128])
            lenders.append(i)
            layers.append(attention(heads, kv, dim, vdim, r.choice([0, 5, 16, 37, 64, 100]), scale=r.choice([0.1, 0.3]),
                                    rot_dims=r.choice([0, 2, dim // 2, dim]), base=r.choice([10000.0, 500000.0]), mlp=mlp()))
        elif kind == "latent":
            layers.append(latent(r.randrange(1, 5), r.choice([8, 16, 32, 64]), r.choice([4, 8, 16, 32]), r.choice([8, 16, 40]),
                                 r.choice([8, 24, 48, 100]), r.choice([8, 20, 64]), scale=r.choice([0.1, 0.3]), mlp=mlp()))
        else:
            heads = r.randrange(1, 5)
            layers.append(lightning(heads, r.choice([8, 16, 32, 64]), r.choice([8, 16, 24, 64]),
                                    [r.choice([0.5, 0.9, 0.97, 0.999, 1.0]) for _ in range(heads)], mlp=mlp()))
    return model(width, vocab, layers, eps=r.choice([1e-5, 1e-6]), scale=r.choice([0.5, 1.0, 2.0]), mult=r.choice([0.3, 0.5, 1.0]))
