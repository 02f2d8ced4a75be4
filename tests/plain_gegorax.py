"""A plain, slow Gegorax in 64-bit numpy: one function per mechanism, whole sequences only.

It shares nothing with the package: it reads the config.json dictionary itself, takes the
stored tensors by their stored names and walks a sequence from its first token.  The tests
compare the package's logits with ``logits(config, weights, tokens)``.

Notation: x is the residual stream [T, W]; a linear weight is stored [out, in] and applied
as x @ w.T; positions count from 0.
"""

import math

import numpy as np


def rms(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x, base, dims):
    """x [T, heads, dim]: neighbouring pairs (2i, 2i+1) of the first ``dims`` columns turned
    by the angle position * base^(-2i/dims)."""
    T = x.shape[0]
    out = x.copy()
    i = np.arange(dims // 2)
    ang = np.arange(T)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]      # [T, dims/2]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = even * c - odd * s
    out[..., 1:dims:2] = odd * c + even * s
    return out


def pooled_window_attention(q, k, v, scale, window, pool):
    """q [T, H, d], k [T, G, d], v [T, G, e].  Token i sees the tokens j with 0 <= i - j <
    window and, for every block of ``pool`` tokens that ends at or before i - window, the
    mean key and the mean value of the block; one softmax over both kinds."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for i in range(T):
        first = max(0, i - window + 1) if window else 0
        blocks = 0
        if window and pool:
            blocks = max(0, (i - window + 1) // pool)
        for h in range(H):
            g = h // (H // G)
            keys = [k[b * pool:(b + 1) * pool, g].mean(0) for b in range(blocks)] + list(k[first:i + 1, g])
            vals = [v[b * pool:(b + 1) * pool, g].mean(0) for b in range(blocks)] + list(v[first:i + 1, g])
            s = np.array(keys) @ q[i, h] * scale
            p = np.exp(s - s.max())
            out[i, h] = (p / p.sum()) @ np.array(vals)
    return out


def window_attention_mixer(h, w, m, eps):
    """The softmax half of the parallel mixer; ``w`` maps 'q', 'k', 'v', 'q.norm', 'k.norm', 'o'."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, G, d)
    v = (h @ w["v"].T).reshape(T, G, e)
    q = rms(q, eps) * w["q.norm"]
    k = rms(k, eps) * w["k.norm"]
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, rot["base"], rot["dims"])
        k = rotate_pairs(k, rot["base"], rot["dims"])
    mask = m.get("mask") or {}
    o = pooled_window_attention(q, k, v, m["scale"], mask.get("size", 0), mask.get("pool", 0))
    return o.reshape(T, H * e) @ w["o"].T


def causal_conv(x, taps_w, bias):
    """x [T, C]; taps_w [C, taps], the last column the token's own; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), x])
    y = np.zeros((T, C))
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j]
    return y + bias


def state_space_mixer(h, w, m, eps):
    """The state-space half: ``w`` maps 'in', 'conv', 'conv.b', 'dt_bias', 'A_log', 'D',
    'norm', 'o'."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w["in"].T
    z = proj[:, :inner]
    xbc = silu(causal_conv(proj[:, inner:2 * inner + 2 * G * N], w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(proj[:, 2 * inner + 2 * G * N:] + w["dt_bias"])         # [T, H]
    keep = np.exp(-np.exp(w["A_log"]) * dt)
    S = np.zeros((H, N, P))
    y = np.zeros((T, H, P))
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = keep[t, hd] * S[hd] + dt[t, hd] * np.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + w["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


def parallel_mixer(h, w, m, eps):
    """Half the sum of the two halves' outputs, each normed over the width first."""
    left = {n[len("left."):]: t for n, t in w.items() if n.startswith("left.")}
    right = {n[len("right."):]: t for n, t in w.items() if n.startswith("right.")}
    a = window_attention_mixer(h, left, m["left"], eps)
    b = state_space_mixer(h, right, m["right"], eps)
    return 0.5 * (rms(a, eps) * left["out"] + rms(b, eps) * right["out"])


def general_delta_mixer(h, w, m, eps):
    """The generalized delta rule: per head S <- diag(w) S - (a u)(u^T S) + k v^T, o = S^T r."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = (h @ w["r"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, H, d)
    v = (h @ w["v"].T).reshape(T, H, d)
    decay = np.exp(-math.exp(-0.5) * sigmoid(np.tanh(h @ w["w1"].T) @ w["w2"].T + w["w0"])).reshape(T, H, d)
    a = sigmoid(h @ w["a"].T + w["a.b"]).reshape(T, H, d)
    u = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    S = np.zeros((H, d, d))
    o = np.zeros((T, H, d))
    for t in range(T):
        for hd in range(H):
            old = S[hd]
            S[hd] = decay[t, hd][:, None] * old - np.outer(a[t, hd] * u[t, hd], u[t, hd] @ old) \
                + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ r[t, hd]
    o = rms(o, eps).reshape(T, H * d) * w["norm"] * sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def dense_ff(h, w):
    return np.maximum(h @ w["up"].T, 0.0) ** 2 @ w["down"].T


def expert(h, gate, up, down, limit):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def routed_ff(h, w, mlp):
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w["router"].T + w["router.b"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = np.argsort(-z[t], kind="stable")[:top]
        p = np.exp(z[t, chosen] - z[t, chosen].max())
        p /= p.sum()
        for e, pe in zip(chosen, p):
            out[t] += pe * expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"],
                                  mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out += expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], mlp["shared"]["limit"])
    return out


def token_side(x, tokens, table, w, i, dim, eps):
    """What layer i adds from the token itself: a slice of the token's row of a second table,
    gated by the stream, projected up and normed."""
    e = table[tokens, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ w["gate"].T) * e) @ w["proj"].T
    return rms(y, eps) * w["norm"]


def sub(weights, prefix):
    return {n[len(prefix):]: np.asarray(t, dtype=np.float64) for n, t in weights.items() if n.startswith(prefix)}


def layer_streams(config, weights, tokens):
    """The residual stream after every layer, [layers, T, W], and the logits [T, vocab]."""
    eps = config["norm"]["eps"]
    tokens = np.asarray(tokens)
    x = np.asarray(weights["embed"], dtype=np.float64)[tokens]
    side = config.get("token_side")
    streams = []
    for i, layer in enumerate(config["layers"]):
        w = sub(weights, f"l{i}.")
        h = rms(x, eps) * w["norm1"]
        if layer["type"] == "parallel":
            y = parallel_mixer(h, sub(w, "mix."), layer["mixer"], eps)
        elif layer["type"] == "general_delta":
            y = general_delta_mixer(h, sub(w, "mix."), layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp:
            y = y + (dense_ff(h, sub(w, "mlp.")) if mlp["kind"] == "dense" else routed_ff(h, sub(w, "mlp."), mlp))
        x = x + y
        if side:
            x = x + token_side(x, tokens, np.asarray(weights["side.embed"], dtype=np.float64),
                               sub(w, "side."), i, side["dim"], eps)
        streams.append(x.copy())
    out = rms(x, eps) * np.asarray(weights["final.norm"], dtype=np.float64)
    return np.array(streams), out @ np.asarray(weights["head"], dtype=np.float64).T


def logits(config, weights, tokens):
    return layer_streams(config, weights, tokens)[1]
