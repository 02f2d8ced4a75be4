"""A plain, slow Besorax in 64-bit numpy: one function per mechanism, whole sequences only.

Nothing here is shared with the package: no cache, no state, no steps, no kernels.  A
sequence is worked on as a whole, every position from the sequence's first token, so that
what the package does with pages, slots, lent caches and recorded steps has something
independent to be compared with.

Notation: n tokens, width W; x[t] is row t.  Weights are stored [out, in] and applied as
W x.  ``w`` of a function: the tensors of that part by their short names.
"""

from __future__ import annotations

import math

import numpy as np


def f64(t) -> np.ndarray:
    """A stored tensor (torch or numpy, any type) as 64-bit numpy."""
    if hasattr(t, "detach"):
        t = t.detach().to("cpu").double().numpy()
    return np.asarray(t, dtype=np.float64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu_erf(z):
    """The exact gelu: z Phi(z) with the normal distribution's Phi."""
    return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))


def dynamic_tanh(x, w, b, alpha):
    """Element by element: tanh(alpha x) w + b.  No mean, no variance."""
    return np.tanh(float(alpha) * x) * w + b


def unit_rms(x, eps):
    """Rows of the last axis divided by their root mean square (eps inside the root)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rotate_pairs(x, positions, dims, base):
    """Rotary positions on the first ``dims`` entries of the last axis of x[n, heads, d]:
    entry 2i is paired with entry 2i + 1; the pair's angle at position p is
    p * base^(-2i/dims).  What lies behind ``dims`` passes unchanged."""
    y = x.copy()
    p = np.asarray(positions, dtype=np.float64)
    for i in range(dims // 2):
        ang = p * base ** (-2.0 * i / dims)
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        y[..., 2 * i] = u * c - v * s
        y[..., 2 * i + 1] = v * c + u * s
    return y


def softmax_with_sink(scores, sink):
    """Weights of the keys when the denominator also holds e^sink (a term with no key and
    no value).  ``sink`` None: the plain softmax."""
    top = max(scores.max(), sink) if sink is not None else scores.max()
    e = np.exp(scores - top)
    return e / (e.sum() + (np.exp(sink - top) if sink is not None else 0.0))


def visible_from(t, chunk):
    """The first position that position t sees: the start of t's chunk (chunks are counted
    from the sequence's position 0), or 0 without chunks."""
    return (t // chunk) * chunk if chunk else 0


def rotated_keys_values(h, w, m):
    """The keys (rotated) and values of an attention layer that has projections of its own:
    k[n, G, dim], v[n, G, vdim]."""
    n = h.shape[0]
    G, d, vd = m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    k = (h @ w["k"].T).reshape(n, G, d)
    v = (h @ w["v"].T).reshape(n, G, vd)
    if m.get("rot"):
        k = rotate_pairs(k, np.arange(n), m["rot"]["dims"], m["rot"]["base"])
    return k, v


def chunked_attention(h, w, m, lent=None):
    """h[n, W] -> ([n, W], (k, v)).  Grouped heads, neighbouring-pair rotation of the first
    rot.dims entries of q and k, scores times ``scale``, a position sees the earlier
    positions of its own chunk of mask.size (all earlier ones without a mask), a sink per
    head.  ``lent``: the (k, v) of the layer whose keys and values this one uses."""
    n = h.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    G = m.get("kv_heads") or H
    chunk = m["mask"]["size"] if m.get("mask") else 0
    q = (h @ w["q"].T).reshape(n, H, d)
    if m.get("rot"):
        q = rotate_pairs(q, np.arange(n), m["rot"]["dims"], m["rot"]["base"])
    k, v = lent if lent is not None else rotated_keys_values(h, w, m)
    sink = w.get("sink")
    out = np.zeros((n, H, vd))
    for t in range(n):
        lo = visible_from(t, chunk)
        for a in range(H):
            g = a // (H // G)
            s = (k[lo:t + 1, g] @ q[t, a]) * m["scale"]
            p = softmax_with_sink(s, None if sink is None else float(sink[a]))
            out[t, a] = p @ v[lo:t + 1, g]
    return out.reshape(n, H * vd) @ w["o"].T, (k, v)


def latent_attention(h, w, m, eps):
    """h[n, W] -> [n, W].  Queries through a normed latent of their own; keys and values of
    every head from ONE normed latent per position and one rotated key part that the heads
    share; causal; a sink per head."""
    n = h.shape[0]
    H, d, r, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(n)
    cq = unit_rms(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).reshape(n, H, d + r)
    down = h @ w["dkv"].T
    c = unit_rms(down[:, :rank], eps) * w["dkv.norm"]
    dims, base = m["rot"]["dims"], m["rot"]["base"]
    k_rot = rotate_pairs(down[:, None, rank:], pos, dims, base)[:, 0]
    q_rot = rotate_pairs(q[:, :, d:], pos, dims, base)
    k = (c @ w["uk"].T).reshape(n, H, d)
    v = (c @ w["uv"].T).reshape(n, H, vd)
    sink = w.get("sink")
    out = np.zeros((n, H, vd))
    for t in range(n):
        for a in range(H):
            s = (k[:t + 1, a] @ q[t, a, :d] + k_rot[:t + 1] @ q_rot[t, a]) * m["scale"]
            p = softmax_with_sink(s, None if sink is None else float(sink[a]))
            out[t, a] = p @ v[:t + 1, a]
    return out.reshape(n, H * vd) @ w["o"].T


def lightning(h, w, m, eps):
    """h[n, W] -> [n, W].  Per head a matrix S[dim, vdim] from zero: S <- decay_h S + k v^T,
    o = S^T q, with q, k, v = silu of their projections and nothing else on them; the heads
    side by side are divided by ONE root mean square, times the weight, times
    sigmoid(W_g h)."""
    n = h.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w["q"].T).reshape(n, H, d)
    k = silu(h @ w["k"].T).reshape(n, H, d)
    v = silu(h @ w["v"].T).reshape(n, H, vd)
    out = np.zeros((n, H, vd))
    for a in range(H):
        S = np.zeros((d, vd))
        for t in range(n):
            S = float(m["decay"][a]) * S + np.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    y = unit_rms(out.reshape(n, H * vd), eps) * w["norm"] * sigmoid(h @ w["g"].T)
    return y @ w["o"].T


def clipped_gated_ff(h, w, limit, alpha=1.702):
    """g = min(W_gate h, limit), u = clamp(W_up h, +-limit); W_down (g sigmoid(alpha g) (u + 1))."""
    g = np.minimum(h @ w["gate"].T, limit)
    u = np.clip(h @ w["up"].T, -limit, limit)
    return (g * sigmoid(alpha * g) * (u + 1.0)) @ w["down"].T


def small_ff(h, up, down):
    """An expert: W_down gelu(W_up h), the exact gelu, no biases."""
    return gelu_erf(h @ up.T) @ down.T


def routed_ff(h, w, mlp):
    """Scores sigmoid(W_router h); a row's ``top`` largest choose its experts (ties: the lower
    index); a chosen expert is fed the row TIMES its score, and the experts' outputs are
    summed as they are; a shared expert, if any, is fed the row itself."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = sigmoid(h @ w["router"].T)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in np.argsort(-s[t], kind="stable")[:top]:
            out[t] += small_ff(s[t, e] * h[t], w[f"e{e}.up"], w[f"e{e}.down"])
    if mlp.get("shared"):
        out += small_ff(h, w["shared.up"], w["shared.down"])
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: f64(v) for k, v in weights.items() if k.startswith(prefix)}


def _norm(x, weights, name):
    return dynamic_tanh(x, f64(weights[name]), f64(weights[name + ".b"]), float(f64(weights[name + ".alpha"])))


def layer_streams(config, weights, tokens):
    """The residual stream after every layer, [layers, n, W]."""
    eps, mult = config["norm"]["eps"], config["residual_mult"]
    x = f64(weights["embed"])[np.asarray(tokens, dtype=np.int64)] * config["embedding"]["scale"]
    kept, out = {}, []
    for i, layer in enumerate(config["layers"]):
        m, w = layer["mixer"], sub(weights, f"l{i}.mix.")
        h = _norm(x, weights, f"l{i}.norm1")
        if layer["type"] == "attention":
            y, kept[i] = chunked_attention(h, w, m, kept[m["kv_from"]] if m.get("kv_from") is not None else None)
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, w, m, eps)
        elif layer["type"] == "lightning":
            y = lightning(h, w, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * y
        mlp = layer.get("mlp")
        if mlp:
            h = _norm(x, weights, f"l{i}.norm2")
            fw = sub(weights, f"l{i}.mlp.")
            y = clipped_gated_ff(h, fw, mlp["limit"]) if mlp["kind"] == "dense" else routed_ff(h, fw, mlp)
            x = x + mult * y
        out.append(x.copy())
    return np.stack(out)


def logits(config, weights, tokens):
    """Logits of every position, [n, vocab]."""
    x = layer_streams(config, weights, tokens)[-1]
    return _norm(x, weights, "final.norm") @ f64(weights["head"]).T
