"""Besorax on the CPU: the configuration and its layout as parts, and the plain model's own
mechanisms (tests/plain_besorax.py) against closed forms."""

from __future__ import annotations

import copy
import math

import numpy as np
import pytest

import plain_besorax as plain
from besorax_cases import ALONE, MIXED, ODD, WIDE, attention, dense, latent, lightning, model, moe, random_weights

from strata_inference_b200.config.registry import spec_from_config
from strata_inference_b200.config.spec import ConfigError
from strata_inference_b200.engine.model import expected_tensors


def test_every_size_and_constant_comes_from_the_configuration():
    typed, spec = spec_from_config(MIXED)
    assert spec.architecture == "Besorax" and spec.hidden_size == 64 and spec.vocab_size == 200
    assert spec.embedding.params["scale"] == 1.5
    assert [e.cache_of for e in spec.schedule] == [None, None, 0, None, None, 0]
    first, borrower = spec.layers[0], spec.layers[5]
    assert first.block == "pre_norm" and first.block_params["residual_scale"] == 0.6
    assert first.mixer.kind == "attention" and first.mixer["chunk"] == 40 and first.mixer["window"] == 0
    assert first.mixer["sink"] and not first.mixer["borrows_cache"]
    assert first.mixer["position"].kind == "rope_interleaved" and first.mixer["position"]["rotary_dim"] == 8
    assert borrower.mixer["borrows_cache"] and borrower.mixer["chunk"] == 70 and borrower.feed_forward is None
    assert first.feed_forward.kind == "clipped_gated_mlp" and first.feed_forward["limit"] == 2.5
    light = spec.layers[1]
    assert light.mixer.kind == "retention" and light.mixer["decay"] == (0.8, 0.95, 0.99, 0.999)
    assert (light.mixer["activation"], light.mixer["norm"], light.mixer["gate"]) == ("silu", "joint", "sigmoid")
    ff = light.feed_forward
    assert ff.kind == "routed_experts" and (ff["experts"], ff["top"], ff["intermediate_size"]) == (6, 2, 24)
    assert (ff["form"], ff["score"], ff["shared"]["intermediate_size"]) == ("plain_gelu", "sigmoid", 32)
    lat = spec.layers[3].mixer
    assert lat.kind == "latent_attention" and (lat["kv_rank"], lat["q_rank"], lat["rot_dim"]) == (32, 40, 8)
    assert lat["sink"] and not lat["head_gate"] and lat["window"] == 0
    assert spec.layers[4].mixer["value_dim"] == 48 and spec.layers[4].mixer["score_scale"] == 0.15
    assert spec.final_norm.kind == "dynamic_tanh" and not spec.head["tied"]


@pytest.mark.parametrize("cfg", [MIXED, ODD, WIDE] + [ALONE[k] for k in sorted(ALONE)])
def test_tensor_table_matches_the_random_weights(cfg):
    _, spec = spec_from_config(cfg)
    table = expected_tensors(spec)
    w = random_weights(cfg, seed=1)
    needed = {n for n, d in table.items() if not d.optional}
    assert needed == set(w), (sorted(needed - set(w)), sorted(set(w) - needed))
    for n in needed:
        assert tuple(table[n].shape) == tuple(w[n].shape), n
    # a layer that reads another's keys and values has no key and value tensors
    for i, layer in enumerate(cfg["layers"]):
        if layer["mixer"].get("kv_from") is not None:
            assert f"l{i}.mix.k" not in table and f"l{i}.mix.v" not in table and f"l{i}.mix.q" in table


def _edit(path, value):
    def edit(c):
        d = c
        for k in path[:-1]:
            d = d[k]
        if value is None:
            d.pop(path[-1])
        else:
            d[path[-1]] = value
    return edit


@pytest.mark.parametrize("edit, text", [
    (_edit(["residual_mult"], None), "residual_mult"),
    (_edit(["embedding"], None), "embedding"),
    (_edit(["layers", 0, "type"], "windowed"), "layers[0].'type'"),
    (_edit(["layers", 0, "mixer", "scale"], -1.0), "layers[0].mixer.'scale'"),
    (_edit(["layers", 0, "mixer", "kv_heads"], 3), "kv_heads"),
    (_edit(["layers", 0, "mixer", "rot", "dims"], 7), "layers[0].mixer.rot"),
    (_edit(["layers", 0, "mlp", "limit"], None), "layers[0].mlp.'limit'"),
    (_edit(["layers", 1, "mixer", "decay"], [0.5]), "layers[1].mixer.'decay'"),
    (_edit(["layers", 1, "mlp", "router", "top"], 9), "'top' exceeds 'experts'"),
    (_edit(["layers", 2, "mixer", "kv_from"], 1), "kv_from"),
    (_edit(["layers", 2, "mixer", "kv_from"], 5), "kv_from"),
    (_edit(["layers", 2, "mixer", "dim"], 32), "'dim' differs"),
    (_edit(["layers", 3, "mixer", "q_rank"], None), "layers[3].mixer.'q_rank'"),
    (_edit(["layers", 3, "mlp", "kind"], "sparse"), "layers[3].mlp.'kind'"),
])
def test_configuration_errors_name_the_key(edit, text):
    cfg = copy.deepcopy(MIXED)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        spec_from_config(cfg)
    assert text in str(e.value), str(e.value)


def test_plain_lightning_is_the_decayed_sum_over_the_past():
    """o_t = sum_{j <= t} decay^(t - j) (q_t . k_j) v_j on the SiLU of the projections, then one
    root mean square over all heads, the weight and the sigmoid gate."""
    rng = np.random.default_rng(0)
    n, W, H, d, vd = 9, 12, 2, 4, 3
    h = rng.normal(size=(n, W))
    w = {k: rng.normal(size=s) for k, s in (("q", (H * d, W)), ("k", (H * d, W)), ("v", (H * vd, W)), ("g", (H * vd, W)),
                                             ("norm", (H * vd,)), ("o", (W, H * vd)))}
    m = {"heads": H, "dim": d, "vdim": vd, "decay": [0.5, 1.0]}
    q, k, v = (plain.silu(h @ w[x].T) for x in "qkv")
    o = np.zeros((n, H, vd))
    for a in range(H):
        for t in range(n):
            for j in range(t + 1):
                o[t, a] += m["decay"][a] ** (t - j) * (q[t, a * d:(a + 1) * d] @ k[j, a * d:(a + 1) * d]) * v[j, a * vd:(a + 1) * vd]
    flat = o.reshape(n, H * vd)
    want = flat / np.sqrt((flat ** 2).mean(-1, keepdims=True) + 1e-5) * w["norm"] / (1 + np.exp(-(h @ w["g"].T))) @ w["o"].T
    assert np.allclose(plain.lightning(h, w, m, 1e-5), want, rtol=1e-10, atol=1e-12)


def test_plain_rotation_of_neighbouring_pairs():
    rng = np.random.default_rng(1)
    x = rng.normal(size=(5, 2, 10))
    y = plain.rotate_pairs(x, [0, 1, 2, 50, 1000], 6, 100.0)
    assert np.array_equal(y[0], x[0]) and np.array_equal(y[..., 6:], x[..., 6:])
    # lengths of pairs are kept; a pair turns by position * base^(-2i/dims)
    for i in range(3):
        assert np.allclose(np.hypot(y[..., 2 * i], y[..., 2 * i + 1]), np.hypot(x[..., 2 * i], x[..., 2 * i + 1]))
        turn = np.arctan2(y[3, 0, 2 * i + 1], y[3, 0, 2 * i]) - np.arctan2(x[3, 0, 2 * i + 1], x[3, 0, 2 * i])
        assert abs(math.remainder(turn - 50 * 100.0 ** (-2 * i / 6), 2 * math.pi)) < 1e-9
    # scores depend on the distance of two positions only
    a, b = rng.normal(size=(1, 1, 6)), rng.normal(size=(1, 1, 6))
    s = [(plain.rotate_pairs(a, [p], 6, 100.0) * plain.rotate_pairs(b, [p - 3], 6, 100.0)).sum() for p in (3, 40)]
    assert abs(s[0] - s[1]) < 1e-9


def test_plain_chunks_and_the_sink():
    assert [plain.visible_from(t, 4) for t in range(9)] == [0, 0, 0, 0, 4, 4, 4, 4, 8]
    assert [plain.visible_from(t, 0) for t in (0, 5, 900)] == [0, 0, 0]
    s = np.array([0.3, -1.0, 2.0])
    p = plain.softmax_with_sink(s, 1.5)
    e = np.exp(s)
    assert np.allclose(p, e / (e.sum() + math.exp(1.5))) and p.sum() < 1.0
    assert np.allclose(plain.softmax_with_sink(s, None).sum(), 1.0)
    # a position at the start of its chunk sees itself alone; with a huge sink it gets nothing
    rng = np.random.default_rng(2)
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 0.5, "mask": {"size": 3}}
    w = {"q": rng.normal(size=(8, 6)), "k": rng.normal(size=(4, 6)), "v": rng.normal(size=(3, 6)),
         "o": np.eye(6), "sink": np.array([-50.0, 50.0])}
    h = rng.normal(size=(7, 6))
    y, (k, v) = plain.chunked_attention(h, w, m)
    for t in (0, 3, 6):
        assert np.allclose(y[t, :3], v[t, 0]) and np.allclose(y[t, 3:], 0.0, atol=1e-12)
    # a borrower reads the keys and values it is handed, through its own chunks
    m2 = dict(m, mask={"size": 7})
    y2, _ = plain.chunked_attention(h, {"q": w["q"], "o": w["o"], "sink": w["sink"]}, m2, lent=(k, v))
    assert np.allclose(y2[0], y[0]) and not np.allclose(y2[3, :3], y[3, :3])


def test_plain_latent_attention_against_keys_made_per_head():
    rng = np.random.default_rng(3)
    n, W = 6, 10
    m = {"heads": 2, "dim": 3, "rot_dim": 2, "vdim": 4, "kv_rank": 5, "q_rank": 7, "scale": 0.4,
         "rot": {"dims": 2, "base": 10.0}}
    w = {"dq": rng.normal(size=(7, W)), "dq.norm": rng.normal(size=7), "uq": rng.normal(size=(10, 7)),
         "dkv": rng.normal(size=(7, W)), "dkv.norm": rng.normal(size=5), "uk": rng.normal(size=(6, 5)),
         "uv": rng.normal(size=(8, 5)), "sink": np.array([0.2, -0.3]), "o": rng.normal(size=(W, 8))}
    h = rng.normal(size=(n, W))
    got = plain.latent_attention(h, w, m, 1e-5)
    # the last position by hand
    cq = h @ w["dq"].T
    cq = cq / np.sqrt((cq ** 2).mean(-1, keepdims=True) + 1e-5) * w["dq.norm"]
    q = (cq @ w["uq"].T).reshape(n, 2, 5)
    down = h @ w["dkv"].T
    c = down[:, :5] / np.sqrt((down[:, :5] ** 2).mean(-1, keepdims=True) + 1e-5) * w["dkv.norm"]

    def turn(x, p):
        ang = p * 1.0
        return np.array([x[0] * math.cos(ang) - x[1] * math.sin(ang), x[1] * math.cos(ang) + x[0] * math.sin(ang)])
    t = n - 1
    out = []
    for a in range(2):
        s = np.array([(w["uk"][3 * a:3 * a + 3] @ c[j]) @ q[t, a, :3] + turn(down[j, 5:], j) @ turn(q[t, a, 3:], t)
                      for j in range(n)]) * 0.4
        e = np.exp(s)
        p = e / (e.sum() + math.exp(w["sink"][a]))
        out.append(sum(p[j] * (w["uv"][4 * a:4 * a + 4] @ c[j]) for j in range(n)))
    assert np.allclose(got[t], np.concatenate(out) @ w["o"].T)


def test_plain_feed_forwards():
    rng = np.random.default_rng(4)
    h = rng.normal(size=(5, 6)) * 3
    w = {"gate": rng.normal(size=(4, 6)), "up": rng.normal(size=(4, 6)), "down": rng.normal(size=(6, 4))}
    g, u = np.minimum(h @ w["gate"].T, 1.5), np.clip(h @ w["up"].T, -1.5, 1.5)
    assert (h @ w["gate"].T).max() > 1.5 and (h @ w["up"].T).min() < -1.5
    assert np.allclose(plain.clipped_gated_ff(h, w, 1.5), (g / (1 + np.exp(-1.702 * g)) * (u + 1)) @ w["down"].T)
    assert abs(plain.gelu_erf(np.array([1.0]))[0] - 0.8413447460685429) < 1e-12
    # experts: the largest sigmoid scores choose; the score multiplies the expert's INPUT
    mlp = {"router": {"experts": 3, "top": 2}, "shared": {"ff": 2}}
    ew = {"router": np.array([[1.0, 0, 0, 0, 0, 0], [0, 1.0, 0, 0, 0, 0], [0, 0, 1.0, 0, 0, 0]]),
          "shared.up": rng.normal(size=(2, 6)), "shared.down": rng.normal(size=(6, 2))}
    for e in range(3):
        ew[f"e{e}.up"], ew[f"e{e}.down"] = rng.normal(size=(4, 6)), rng.normal(size=(6, 4))
    x = np.array([[2.0, -1.0, 0.5, 0.3, 0.1, -0.2]])
    s = 1 / (1 + np.exp(-x[0, :3]))
    want = (plain.small_ff(s[0] * x[0], ew["e0.up"], ew["e0.down"]) + plain.small_ff(s[2] * x[0], ew["e2.up"], ew["e2.down"])
            + plain.small_ff(x[0], ew["shared.up"], ew["shared.down"]))
    assert np.allclose(plain.routed_ff(x, ew, mlp)[0], want)
    on_output = s[0] * plain.small_ff(x[0], ew["e0.up"], ew["e0.down"]) + s[2] * plain.small_ff(x[0], ew["e2.up"], ew["e2.down"])
    assert not np.allclose(want - plain.small_ff(x[0], ew["shared.up"], ew["shared.down"]), on_output)


def test_plain_layer_scales_what_it_adds():
    cfg = model(16, 20, [lightning(1, 4, 4, [0.9], mlp=dense(8))], mult=0.25)
    w = random_weights(cfg, seed=5)
    toks = [1, 2, 3]
    x0 = plain.f64(w["embed"])[toks] * 1.5
    h = plain.dynamic_tanh(x0, plain.f64(w["l0.norm1"]), plain.f64(w["l0.norm1.b"]), float(w["l0.norm1.alpha"]))
    x1 = x0 + 0.25 * plain.lightning(h, plain.sub(w, "l0.mix."), cfg["layers"][0]["mixer"], 1e-5)
    h = plain.dynamic_tanh(x1, plain.f64(w["l0.norm2"]), plain.f64(w["l0.norm2.b"]), float(w["l0.norm2.alpha"]))
    x2 = x1 + 0.25 * plain.clipped_gated_ff(h, plain.sub(w, "l0.mlp."), 2.5)
    assert np.allclose(plain.layer_streams(cfg, w, toks)[0], x2)


def test_sizes_that_the_configuration_omits_come_from_the_tensors():
    """A folder's config.json may leave a size to the tensors' shapes: the completed configuration is
    the full one; a size that is given stays as given."""
    from strata_inference_b200.config.besorax import besorax_sizes
    for cfg in (MIXED, ODD):
        shapes = {n: tuple(t.shape) for n, t in random_weights(cfg, seed=1).items()}
        bare = copy.deepcopy(cfg)
        del bare["vocab"], bare["width"]
        for layer in bare["layers"]:
            m = layer["mixer"]
            for key in ("dim", "vdim", "kv_heads", "q_rank", "kv_rank", "rot_dim"):
                m.pop(key, None)
            if layer["mlp"]:
                layer["mlp"].pop("ff", None)
                layer["mlp"].get("router", {}).pop("experts", None)
                layer["mlp"].get("expert", {}).pop("ff", None)
                if layer["mlp"].get("shared"):
                    layer["mlp"]["shared"].pop("ff")
        full = besorax_sizes(bare, shapes)
        assert spec_from_config(full)[1] == spec_from_config(cfg)[1]
        assert spec_from_config(bare, shapes)[1] == spec_from_config(cfg)[1]
        assert besorax_sizes(cfg, shapes) == cfg
