"""Gegorax without a device: the configuration and its parts, the tensor table, and the plain
model's mechanisms against closed forms of their own."""

from __future__ import annotations

import copy
import math

import numpy as np
import pytest

import plain_gegorax as plain
from gegorax_cases import ALONE, MIXED, NARROW, ODD, WIDE, delta, dense, model, moe, parallel, random_weights

from strata_inference_b200.config.gegorax import gegorax_sizes
from strata_inference_b200.config.registry import spec_from_config
from strata_inference_b200.config.spec import ConfigError
from strata_inference_b200.engine.model import expected_tensors


def test_every_size_and_constant_comes_from_the_configuration():
    _, spec = spec_from_config(MIXED)
    assert [l.block for l in spec.layers] == ["parallel"] * 5
    pair = spec.layers[3].mixer
    assert pair.kind == "side_by_side"
    left, right = pair["left"], pair["right"]
    assert left.kind == "attention" and left["window"] == 70 and left["pool"] == 12
    assert left["num_heads"] == 2 and left["num_kv_heads"] == 2 and left["value_dim"] == 16
    assert left["score_scale"] == 0.15 and left["position"].kind == "rope_interleaved"
    assert left["position"]["rotary_dim"] == 8 and left["position"]["theta"] == 10000.0
    assert right.kind == "state_space" and right["conv_taps"] == 3 and right["state_dim"] == 8
    d = spec.layers[2].mixer
    assert d.kind == "general_delta" and d["num_heads"] == 4 and d["head_dim"] == 8 and d["decay_rank"] == 12
    ff = spec.layers[1].feed_forward
    assert ff.kind == "routed_experts" and ff["experts"] == 8 and ff["top"] == 3 and ff["limit"] == 2.0
    assert ff["shared"] == {"intermediate_size": 48, "limit": 1.5}
    assert spec.layers[3].feed_forward["shared"] is None and spec.layers[4].feed_forward is None
    assert spec.layers[0].feed_forward.kind == "mlp" and spec.layers[0].feed_forward["activation"] == "relu_squared"
    assert spec.layers[2].tail.kind == "token_side" and spec.layers[2].tail["index"] == 2
    assert spec.embedding["side_width"] == 8 * 5
    _, bare = spec_from_config(NARROW)
    assert bare.layers[0].tail is None and bare.embedding["side_width"] == 0


def test_decay_width_comes_from_the_stored_tensor():
    cfg = model(64, 150, [delta(2, 16), parallel(2, 1, 8, 8, 9, 3, 2, 8, 8), delta(2, 16)])
    sized = gegorax_sizes(cfg, {"l0.mix.w1": (24, 64), "l2.mix.w1": (5, 64)})
    _, spec = spec_from_config(sized)
    assert [spec.layers[i].mixer["decay_rank"] for i in (0, 2)] == [24, 5]
    assert "decay_rank" not in cfg["layers"][0]["mixer"]            # the given dictionary is left alone


def test_tensor_table_matches_the_random_weights():
    for cfg in list(ALONE.values()) + [MIXED, ODD, NARROW, WIDE]:
        _, spec = spec_from_config(cfg)
        exp = expected_tensors(spec)
        w = random_weights(cfg, seed=1)
        assert {n for n, d in exp.items() if not d.optional} == set(w)
        for n, t in w.items():
            assert tuple(exp[n].shape) == tuple(t.shape), n


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][1]["mixer"].pop("dim"), "dim"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_errors_name_the_key(edit, text):
    cfg = copy.deepcopy(MIXED)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        spec_from_config(cfg)
    assert text in str(e.value)


def test_plain_pooled_window_sees_tokens_then_blocks_then_nothing():
    """Values are one-hot per position, so a row's output shows its weights.  Window 4, blocks of
    3: row 9 sees tokens 6..9 and blocks 0 (0..2) and 1 (3..5); row 8 sees tokens 5..8 and block
    0 only, and positions 3 and 4 not at all."""
    T, d = 12, 4
    rng = np.random.default_rng(0)
    q, k = rng.normal(size=(T, 1, d)), rng.normal(size=(T, 1, d))
    v = np.eye(T)[:, None, :]
    out = plain.pooled_window_attention(q, k, v, 0.7, 4, 3)[:, 0]
    seen = out > 0
    assert seen[9].tolist() == [True] * 6 + [True] * 4 + [False, False]
    assert seen[8].tolist() == [True] * 3 + [False, False] + [True] * 4 + [False] * 3
    assert seen[3].tolist() == [True] * 4 + [False] * 8 and seen[6].tolist() == [True] * 7 + [False] * 5
    assert np.allclose(out.sum(-1), 1.0)
    # a block's three positions share the block's weight equally, and that weight is the
    # softmax term of the mean key
    assert np.allclose(out[9, 0], out[9, 1]) and np.allclose(out[9, 3], out[9, 5])
    s = np.array([k[0:3, 0].mean(0) @ q[9, 0], k[3:6, 0].mean(0) @ q[9, 0]] + [k[j, 0] @ q[9, 0] for j in range(6, 10)]) * 0.7
    p = np.exp(s - s.max())
    p /= p.sum()
    assert np.allclose(out[9, :3].sum(), p[0]) and np.allclose(out[9, 6:10], p[2:])


def test_plain_rotation_of_neighbouring_pairs():
    x = np.zeros((3, 1, 6))
    x[:, 0, 0] = 1.0
    x[:, 0, 4] = 2.0
    y = plain.rotate_pairs(x, 100.0, 4)
    assert np.allclose(y[2, 0, :2], [math.cos(2.0), math.sin(2.0)]) and np.allclose(y[:, 0, 4], 2.0)
    a, b = np.random.default_rng(1).normal(size=(2, 8))

    def at(vec, pos):
        rows = np.zeros((pos + 1, 1, 8))
        rows[pos, 0] = vec
        return plain.rotate_pairs(rows, 50.0, 6)[pos, 0]
    assert np.allclose(at(a, 105)[6:], a[6:]) and np.allclose((at(a, 105) ** 2).sum(), (a ** 2).sum())
    # the product of two rotated vectors depends on the distance of their positions only
    assert abs((at(a, 9) * at(b, 4)).sum() - (at(a, 105) * at(b, 100)).sum()) < 1e-9


def test_plain_state_space_is_the_decayed_sum_over_the_past():
    """y_t = sum_{s <= t} (prod_{s < r <= t} keep_r) dt_s <C_t, B_s> x_s + D x_t."""
    rng = np.random.default_rng(2)
    T, W = 9, 12
    m = {"heads": 2, "vdim": 3, "state": 4, "groups": 1, "conv": 3, "norm_groups": 2}
    inner, ch = 6, 6 + 8
    w = {"in": rng.normal(size=(inner + ch + 2, W)) * 0.4, "conv": rng.normal(size=(ch, 3)),
         "conv.b": rng.normal(size=ch) * 0.1, "dt_bias": rng.normal(size=2), "A_log": rng.normal(size=2),
         "D": rng.normal(size=2), "norm": rng.normal(size=inner), "o": rng.normal(size=(W, inner))}
    h = rng.normal(size=(T, W))
    proj = h @ w["in"].T
    raw = proj[:, inner:inner + ch]
    conv = np.zeros((T, ch))
    for t in range(T):
        for j in range(3):
            if t - 2 + j >= 0:
                conv[t] += raw[t - 2 + j] * w["conv"][:, j]
    xbc = plain.silu(conv + w["conv.b"])
    x, B, C = xbc[:, :6].reshape(T, 2, 3), xbc[:, 6:10], xbc[:, 10:]
    dt = np.log1p(np.exp(proj[:, -2:] + w["dt_bias"]))
    keep = np.exp(-np.exp(w["A_log"]) * dt)
    y = np.zeros((T, 2, 3))
    for a in range(2):
        for t in range(T):
            for s in range(t + 1):
                y[t, a] += np.prod(keep[s + 1:t + 1, a]) * dt[s, a] * (C[t] @ B[s]) * x[s, a]
            y[t, a] += w["D"][a] * x[t, a]
    y = y.reshape(T, 6) * plain.silu(proj[:, :6])
    y = np.concatenate([plain.rms(y[:, :3], 1e-5), plain.rms(y[:, 3:], 1e-5)], axis=1) * w["norm"]
    assert np.allclose(plain.state_space_mixer(h, w, m, 1e-5), y @ w["o"].T, atol=1e-10)


def test_plain_delta_rule_without_removal_is_a_decayed_sum_and_with_it_forgets_a_repeated_key():
    rng = np.random.default_rng(3)
    T, W, H, d = 7, 10, 2, 4
    m = {"heads": H, "dim": d}
    w = {n: rng.normal(size=(H * d, W)) * 0.5 for n in "rkvga"}
    w.update({"w1": rng.normal(size=(3, W)), "w2": rng.normal(size=(H * d, 3)), "w0": rng.normal(size=H * d),
              "a.b": np.full(H * d, -80.0), "norm": rng.normal(size=H * d), "o": rng.normal(size=(W, H * d))})
    h = rng.normal(size=(T, W))
    r, k, v = ((h @ w[n].T).reshape(T, H, d) for n in "rkv")
    dec = np.exp(-math.exp(-0.5) / (1 + np.exp(-(np.tanh(h @ w["w1"].T) @ w["w2"].T + w["w0"])))).reshape(T, H, d)
    assert (dec > math.exp(-math.exp(-0.5))).all() and (dec < 1).all()
    o = np.zeros((T, H, d))
    for a in range(H):
        for t in range(T):
            for s in range(t + 1):
                o[t, a] += ((r[t, a] * np.prod(dec[s + 1:t + 1, a], axis=0)) @ k[s, a]) * v[s, a]
    ref = (plain.rms(o, 1e-5).reshape(T, -1) * w["norm"] / (1 + np.exp(-(h @ w["g"].T)))) @ w["o"].T
    assert np.allclose(plain.general_delta_mixer(h, w, m, 1e-5), ref, atol=1e-9)
    # removal rate 1 and no decay: a key that comes again replaces what it stored before
    S = np.zeros((d, d))
    key, u = np.array([2.0, 0, 0, 0]), np.array([1.0, 0, 0, 0])
    for val in (np.arange(4.0), np.ones(4)):
        S = S - np.outer(u, u @ S) + np.outer(key, val)
    assert np.allclose(S[0], 2 * np.ones(4))


def test_plain_experts_router_and_token_side():
    rng = np.random.default_rng(4)
    W = 6
    mlp = moe(4, 2, 5, 1.0, shared=(3, 0.5))
    w = {"router": np.zeros((4, W)), "router.b": np.array([0.0, 3.0, 1.0, 3.0 - math.log(3.0)])}
    for n in ["e0", "e1", "e2", "e3", "shared"]:
        f = 3 if n == "shared" else 5
        w.update({f"{n}.gate": rng.normal(size=(f, W)), f"{n}.up": rng.normal(size=(f, W)),
                  f"{n}.down": rng.normal(size=(W, f))})
    h = rng.normal(size=(2, W)) * 3
    one = lambda n, lim: plain.expert(h, w[n + ".gate"], w[n + ".up"], w[n + ".down"], lim)  # noqa: E731
    ref = 0.75 * one("e1", 1.0) + 0.25 * one("e3", 1.0) + one("shared", 0.5)
    assert np.allclose(plain.routed_ff(h, w, mlp), ref)
    g, u = np.array([[5.0, -5.0, 0.3]]), np.array([[9.0, -9.0, 0.2]])
    y = plain.expert(np.ones((1, 1)), g.T, u.T, np.eye(3), 2.0)[0]
    gg = np.array([2.0, -5.0, 0.3])
    assert np.allclose(y, gg / (1 + np.exp(-1.702 * gg)) * (np.array([2.0, -2.0, 0.2]) + 1))
    # the token side: layer i reads columns [i dim, (i + 1) dim) of the token's row
    table = np.arange(3 * 4, dtype=float).reshape(3, 4)
    ws = {"gate": rng.normal(size=(2, W)), "proj": rng.normal(size=(W, 2)), "norm": rng.normal(size=W)}
    x = rng.normal(size=(2, W))
    y = (plain.gelu_tanh(x @ ws["gate"].T) * table[[2, 0], 2:4]) @ ws["proj"].T
    assert np.allclose(plain.token_side(x, [2, 0], table, ws, 1, 2, 1e-6), plain.rms(y, 1e-6) * ws["norm"])
    assert abs(plain.gelu_tanh(np.array([1.0]))[0] - 0.8411919906) < 1e-9


def test_plain_layer_adds_both_sublayers_of_one_normed_input():
    cfg = model(16, 20, [parallel(2, 1, 4, 4, 5, 2, 2, 4, 4, mlp=dense(8))], side=0)
    w = {n: t.double().numpy() for n, t in random_weights(cfg, seed=5).items()}
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    streams, _ = plain.layer_streams(cfg, w, toks)
    x = w["embed"][toks]
    h = plain.rms(x, cfg["norm"]["eps"]) * w["l0.norm1"]
    mix = plain.parallel_mixer(h, plain.sub(w, "l0.mix."), cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    assert np.allclose(streams[0], x + mix + plain.dense_ff(h, plain.sub(w, "l0.mlp.")))
