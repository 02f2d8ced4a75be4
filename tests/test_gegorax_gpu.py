"""Gegorax through the engine against the plain model (tests/plain_gegorax.py): each layer kind
alone, prompts against token-by-token steps, portions, unequal batches, slots and pages used
again, the window's edges and blocks that have just come into sight or are about to (as a
prompt, in portions and token by token), the first tokens of a sequence, long decoding, odd,
narrow and wide sizes, recorded steps, the mechanisms' kernels alone, greedy generation, the
command line and trace replay."""

from __future__ import annotations

import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_gegorax as plain
from gegorax_cases import (ALONE, BLOCKS, BLOCKS_TC, MIXED, NARROW, ODD, SHARP, WIDE, assert_close, asking_prompt,
                           plain_logits, prompts, random_weights, rows_that_differ, shifted_blocks,
                           tie_queries_to_keys)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_engine(cfg, weights, dtype, **kw):
    from strata_inference_b200.config.registry import spec_from_config
    from strata_inference_b200.engine.engine import Engine
    _, spec = spec_from_config(cfg)
    kw.setdefault("max_tokens", 2048)
    kw.setdefault("max_seq_len", 1024)
    return Engine(spec, weights, dtype=dtype, **kw)


def all_rows(n):
    return list(range(n))


def run_whole(eng, tokens):
    s = eng.new_sequence()
    out = eng.step([(s, tokens)], [all_rows(len(tokens))])
    eng.end_sequence(s)
    return out


def run_portions(eng, tokens, sizes):
    """The prompt cut into steps of the given sizes, and what is left into steps of 48."""
    s, at, rows = eng.new_sequence(), 0, []
    for n in list(sizes) + [48] * (len(tokens) // 48 + 1):
        part = tokens[at:at + n]
        if not part:
            break
        rows.append(eng.step([(s, part)], [all_rows(len(part))]))
        at += len(part)
    eng.end_sequence(s)
    return torch.cat(rows)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_layer_kind_alone(name, dtype):
    cfg = ALONE[name]
    w = random_weights(cfg, seed=11)
    eng = make_engine(cfg, w, dtype)
    for toks in prompts(cfg, [1, 2, 5, 90], seed=3):
        assert_close(run_whole(eng, toks), plain_logits(cfg, w, toks), dtype, f"{name}, {len(toks)} tokens")
    toks = prompts(cfg, [95], seed=4)[0]
    assert_close(run_portions(eng, toks, [3, 1, 1, 2, 50] + [1] * 8), plain_logits(cfg, w, toks), dtype,
                 f"{name} in portions and single tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_then_long_decoding(dtype):
    """A prompt in one step, then 260 single-token steps (over page borders, past every window
    and many blocks; the token steps are recorded at the second and replayed from the third),
    and token by token from the very first token."""
    cfg = MIXED
    w = random_weights(cfg, seed=5)
    eng = make_engine(cfg, w, dtype)
    toks = prompts(cfg, [300], seed=6)[0]
    ref = plain_logits(cfg, w, toks)
    assert_close(run_portions(eng, toks, [40] + [1] * 260), ref, dtype, "prompt of 40, then token by token")
    assert_close(run_portions(eng, toks[:60], [1] * 45 + [15]), ref[:60], dtype, "token by token from the first token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [[2, 2, 2, 2], [64, 25], [63, 2, 24], [1, 24, 3, 23], [17, 17, 17, 17, 17],
                                   [7, 8, 9, 16, 1, 15, 24], [39, 1, 1, 7, 1, 1, 20], [15, 1, 1, 52, 1, 1, 11, 1]])
def test_portions(sizes, dtype):
    """(the mixed model's windows are 40, 70 and 16 with blocks of 8, 12 and 16; the last two
    lists cut at the windows' edges and where a block's last position arrives; the one before
    them around the scans' chunks of 8)"""
    cfg = MIXED
    w = random_weights(cfg, seed=7)
    eng = make_engine(cfg, w, dtype)
    toks = prompts(cfg, [150], seed=8)[0]
    assert_close(run_portions(eng, toks, sizes + [20] * 8), plain_logits(cfg, w, toks), dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_against_each_alone(dtype):
    """Prompts of 1 to 130 tokens in one step, then single-token steps together; the
    shorter requests end earlier and a new one takes a freed slot later."""
    cfg = MIXED
    w = random_weights(cfg, seed=9)
    eng = make_engine(cfg, w, dtype)
    reqs = prompts(cfg, [21, 22, 100, 160, 35], seed=10)
    first = [1, 2, 70, 130, 5]
    refs = [plain_logits(cfg, w, t) for t in reqs]
    live = [0, 1, 2, 3]
    slots = {i: eng.new_sequence() for i in live}
    out = eng.step([(slots[i], reqs[i][:first[i]]) for i in live], [all_rows(first[i]) for i in live])
    at = 0
    for i in live:
        assert_close(out[at:at + first[i]], refs[i][:first[i]], dtype, f"batched prompt {i}")
        at += first[i]
    pos = {i: first[i] for i in live}
    step = 0
    while live:
        if step == 25:                         # the latecomer starts alone, then decodes with the rest
            slots[4] = eng.new_sequence()
            got = eng.step([(slots[4], reqs[4][:first[4]])], [all_rows(first[4])])
            assert_close(got, refs[4][:first[4]], dtype, "late prompt")
            pos[4] = first[4]
            live.append(4)
        out = eng.step([(slots[i], [reqs[i][pos[i]]]) for i in live], [[0]] * len(live))
        for k, i in enumerate(live):
            assert_close(out[k:k + 1], refs[i][pos[i]:pos[i] + 1], dtype, f"request {i}, token {pos[i]}")
            pos[i] += 1
        for i in list(live):
            if pos[i] == len(reqs[i]):
                eng.end_sequence(slots[i])
                live.remove(i)
        step += 1
    assert step > 25


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(dtype):
    """A slot that is given back and taken again starts from nothing: matrices, the
    convolution's last inputs, keys, blocks' cells and pages of the request before leave no
    trace; with few pages they are all used again."""
    cfg = MIXED
    w = random_weights(cfg, seed=12)
    eng = make_engine(cfg, w, dtype, max_tokens=256, max_seq_len=256, max_slots=2)
    a, b, c = prompts(cfg, [100, 90, 120], seed=13)
    ra, rb, rc = (plain_logits(cfg, w, t) for t in (a, b, c))
    sa = eng.new_sequence()
    assert_close(eng.step([(sa, a[:70])], [all_rows(70)]), ra[:70], dtype, "a, first part")
    sb = eng.new_sequence()
    assert_close(eng.step([(sb, b[:50])], [all_rows(50)]), rb[:50], dtype, "b, first part")
    assert_close(eng.step([(sa, a[70:])], [all_rows(30)]), ra[70:], dtype, "a, second part")
    eng.end_sequence(sa)
    sc = eng.new_sequence()
    assert sc == sa
    assert_close(eng.step([(sc, c[:110])], [all_rows(110)]), rc[:110], dtype, "c in a's slot and pages")
    out = eng.step([(sb, [b[50]]), (sc, [c[110]])], [[0], [0]])
    assert_close(out, torch.stack([rb[50], rc[110]]), dtype, "b and c together")
    assert_close(eng.step([(sb, b[51:])], [all_rows(39)]), rb[51:], dtype, "b, the rest")
    eng.end_sequence(sb)
    eng.end_sequence(sc)
    assert_close(run_whole(eng, a), ra, dtype, "a once more")
    assert eng.cache.pages_in_use() == 0


def changed(cfg, edit):
    other = copy.deepcopy(cfg)
    edit(other)
    return other


def test_window_edges_with_a_sharp_softmax():
    """With a large scale the softmax puts most of a row's weight on single keys, wherever in
    the window they lie.  The plain model with a window one shorter or one longer gives other
    logits in most rows behind the windows (checked first: the test can tell them apart); the
    engine agrees with the right one as a prompt, in portions around page borders and the
    windows' edges, token by token, and as two requests of unequal length."""
    cfg, dtype = SHARP, "float32"
    w = random_weights(cfg, seed=14)
    toks = prompts(cfg, [330], seed=15)[0]
    ref = plain_logits(cfg, w, toks)

    def window(delta):
        def edit(c):
            for layer in c["layers"]:
                layer["mixer"]["left"]["mask"]["size"] += delta
        return edit
    for delta in (-1, 1):
        other = plain_logits(changed(cfg, window(delta)), w, toks)
        assert rows_that_differ(ref[100:], other[100:], 20.0) > 100, f"a window off by {delta} would not show"
    eng = make_engine(cfg, w, dtype)
    assert_close(run_whole(eng, toks), ref, dtype, "whole prompt")
    assert_close(run_portions(eng, toks, [64, 64, 64, 64]), ref, dtype, "portions of one page")
    assert_close(run_portions(eng, toks, [63, 2, 63, 1, 1, 20, 66, 60]), ref, dtype, "portions around page borders")
    assert_close(run_portions(eng, toks, [29, 1, 1, 34, 1, 1, 1, 90, 60, 60]), ref, dtype, "portions around the windows' edges")
    assert_close(run_portions(eng, toks, [200] + [1] * 130), ref, dtype, "single tokens past both windows")
    assert_close(run_portions(eng, toks[:120], [20] + [1] * 100), ref[:120], dtype, "single tokens over both edges")
    a, b = toks[:250], prompts(cfg, [180], seed=16)[0]
    rb = plain_logits(cfg, w, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([(sa, a[:200]), (sb, b[:100])], [all_rows(200), all_rows(100)])
    assert_close(out, torch.cat([ref[:200], rb[:100]]), dtype, "two prompts")
    for k in range(50):
        out = eng.step([(sa, [a[200 + k]]), (sb, [b[100 + k]])], [[0], [0]])
        assert_close(out, torch.stack([ref[200 + k], rb[100 + k]]), dtype, f"two requests, token {k}")


@pytest.mark.parametrize("name", sorted(BLOCKS))
def test_blocks_that_have_just_come_into_sight_and_blocks_about_to(name, monkeypatch):
    """One layer whose queries are made by the keys' matrix, and a prompt whose blocks repeat
    one token each: a row that carries an earlier block's token puts much of its weight on
    that block's cell if it sees it.  The plain model that takes a row's blocks one position
    early or late, or leaves them out, gives other logits (checked first); the engine agrees
    with the right one as a prompt, in portions that end at, before and after a block's last
    position, token by token over many blocks, and as two unequal requests."""
    cfg, dtype = BLOCKS[name], "float32"
    w = tie_queries_to_keys(random_weights(cfg, seed=14))
    mask = cfg["layers"][0]["mixer"]["left"]["mask"]
    window, pool = mask["size"], mask["pool"]
    toks = asking_prompt(cfg, 330, seed=15)
    ref = plain_logits(cfg, w, toks)
    for shift, least in ((-1, 8), (1, 8), (None, 200)):
        monkeypatch.setattr(plain, "pooled_window_attention", shifted_blocks(shift))
        assert rows_that_differ(ref, plain_logits(cfg, w, toks), 20.0) > least, f"blocks shifted by {shift} would not show"
        monkeypatch.undo()
    eng = make_engine(cfg, w, dtype)
    assert_close(run_whole(eng, toks), ref, dtype, "whole prompt")
    edge = window + 2 * pool - 1          # the row at which block 1 comes into sight
    cuts = [[edge - 1, 1, 1, 1], [edge, pool, pool - 1, 1, pool + 1], [pool - 1, 1, 1, pool - 1, 2, 64, 2, 62],
            [window, pool, 2, 2, 2, 2, 100]]
    for sizes in cuts:
        sizes = [n for n in sizes if n > 0]
        assert_close(run_portions(eng, toks, sizes + [50] * 8), ref, dtype, f"portions {sizes}")
    assert_close(run_portions(eng, toks, [window + pool - 2] + [1] * 150), ref, dtype, "single tokens over many blocks")
    assert_close(run_portions(eng, toks[:140], [1] * 140), ref[:140], dtype, "token by token from the first token")
    b = asking_prompt(cfg, 200, seed=16)
    rb = plain_logits(cfg, w, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([(sa, toks[:150]), (sb, b[:37])], [all_rows(150), all_rows(37)])
    assert_close(out, torch.cat([ref[:150], rb[:37]]), dtype, "two prompts")
    for k in range(100):
        out = eng.step([(sa, [toks[150 + k]]), (sb, [b[37 + k]])], [[0], [0]])
        assert_close(out, torch.stack([ref[150 + k], rb[37 + k]]), dtype, f"two requests, token {k}")
    # bfloat16: the same prompt whole and token by token
    eng = make_engine(cfg, w, "bfloat16")
    assert_close(run_whole(eng, toks), ref, "bfloat16", "whole prompt, bfloat16")
    assert_close(run_portions(eng, toks[:200], [window + pool - 2] + [1] * 120), ref[:200], "bfloat16", "single tokens, bfloat16")


def test_first_tokens_of_a_sequence():
    """Before the start the convolution reads zeros and the matrices are zero, also in a slot
    that held another request: the first tokens one by one, in pairs, and alone."""
    cfg, dtype = MIXED, "float32"
    w = random_weights(cfg, seed=24)
    toks = prompts(cfg, [40], seed=25)[0]
    ref = plain_logits(cfg, w, toks)
    eng = make_engine(cfg, w, dtype, max_slots=1)
    assert_close(run_portions(eng, toks, [1, 1, 1, 2, 2, 5]), ref, dtype, "first tokens one by one")
    assert_close(run_portions(eng, toks[::-1], [3, 1]), plain_logits(cfg, w, toks[::-1]), dtype, "the slot again")
    assert_close(run_whole(eng, toks[:1]), ref[:1], dtype, "one token alone")
    assert_close(run_portions(eng, toks, [2, 2, 2]), ref, dtype, "pairs")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd", "wide", "narrow"])
def test_other_sizes(name, dtype):
    cfg = {"odd": ODD, "wide": WIDE, "narrow": NARROW}[name]
    w = random_weights(cfg, seed=16)
    eng = make_engine(cfg, w, dtype)
    a, b = prompts(cfg, [230, 37], seed=17)
    ra, rb = plain_logits(cfg, w, a), plain_logits(cfg, w, b)
    assert_close(run_whole(eng, a), ra, dtype, f"{name}: whole prompt")
    assert_close(run_portions(eng, a, [2, 60, 30] + [1] * 20 + [70] + [1] * 30), ra, dtype, f"{name}: portions and tokens")
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([(sa, a[:130]), (sb, b[:30])], [[0, 129], [29]])
    assert_close(out, torch.stack([ra[0], ra[129], rb[29]]), dtype, f"{name}: two prompts")
    for k in range(7):
        out = eng.step([(sa, [a[130 + k]]), (sb, [b[30 + k]])], [[0], [0]])
        assert_close(out, torch.stack([ra[130 + k], rb[30 + k]]), dtype, f"{name}: tokens {k}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_recorded_prompt_steps(dtype):
    """Prompt steps of one shape: launched, recorded, then replayed for other prompts (also
    shorter ones, filled up with rows that belong to no sequence)."""
    cfg = MIXED
    w = random_weights(cfg, seed=18)
    eng = make_engine(cfg, w, dtype)
    for n, seed in ((60, 1), (64, 2), (50, 3), (33, 4), (64, 5)):
        toks = prompts(cfg, [n], seed=seed)[0]
        s = eng.new_sequence()
        out = eng.step([(s, toks)], [[0, n - 1]])
        eng.end_sequence(s)
        ref = plain_logits(cfg, w, toks)
        assert_close(out, torch.stack([ref[0], ref[n - 1]]), dtype, f"prompt of {n}")
    assert any(g.graph is not None for g in eng._prompt_graphs.values())


@pytest.mark.parametrize("dtype", DTYPES)
def test_many_rows_take_the_sorted_experts_and_few_the_streamed_ones(dtype):
    """A prompt of more rows than the pair-streaming path takes and the same tokens in small
    portions choose the same experts and agree with the plain model; so does a batch of 40
    single tokens (sorted) against each alone (streamed)."""
    cfg = ALONE["delta_moe"]
    w = random_weights(cfg, seed=31)
    eng = make_engine(cfg, w, dtype, max_slots=48)
    toks = prompts(cfg, [120], seed=32)[0]
    ref = plain_logits(cfg, w, toks)
    assert_close(run_whole(eng, toks), ref, dtype, "120 rows at once")
    assert_close(run_portions(eng, toks, [5] * 24), ref, dtype, "portions of 5")
    reqs = prompts(cfg, [3] * 40, seed=33)
    slots = [eng.new_sequence() for _ in reqs]
    out = eng.step([(s, t[:2]) for s, t in zip(slots, reqs)], [[1]] * 40)
    refs = [plain_logits(cfg, w, t) for t in reqs]
    assert_close(out, torch.stack([r[1] for r in refs]), dtype, "40 prompts of two")
    out = eng.step([(s, t[2:]) for s, t in zip(slots, reqs)], [[0]] * 40)
    assert_close(out, torch.stack([r[2] for r in refs]), dtype, "40 single tokens")


def test_states_that_hardly_decay_remember_the_first_tokens():
    """A_log and w0 lowered so that the matrices keep what they hold over hundreds of tokens:
    another first token changes the logits 250 positions on (checked on the plain model), and
    the engine agrees as a prompt, in portions and after 200 single tokens."""
    dtype = "float32"
    for name, lowered in (("parallel", "l0.mix.right.A_log"), ("delta", "l0.mix.w0")):
        cfg = ALONE[name]
        w = random_weights(cfg, seed=41)
        w[lowered] = w[lowered] - 7.0
        toks = prompts(cfg, [260], seed=42)[0]
        ref = plain_logits(cfg, w, toks)
        other = plain_logits(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
        assert rows_that_differ(ref[250:], other[250:], 5.0) == 10, f"{name}: the first token would not show"
        eng = make_engine(cfg, w, dtype)
        assert_close(run_whole(eng, toks), ref, dtype, f"{name}: whole prompt")
        assert_close(run_portions(eng, toks, [7, 2, 50] + [1] * 200), ref, dtype, f"{name}: portions and tokens")


# ---- the mechanisms' kernels alone ---------------------------------------------------------

def _dev(t, dtype=torch.float32):
    return t.to(dtype).cuda()


@pytest.mark.parametrize("experts, top", [(8, 3), (5, 1), (7, 7), (64, 8), (33, 32), (2, 2)])
def test_router_choice_alone(experts, top):
    """The largest logits in order, ties to the lower index, weights a softmax over the chosen
    ones alone; logits that are equal everywhere choose the first experts evenly."""
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(experts * 100 + top)
    rows = 50
    z = torch.randn((rows, experts), generator=g)
    z[4, :] = 0.5
    if experts > 2:
        z[5, 1] = z[5, 2] = z[5].max() + 1.0
    bias = torch.randn(experts, generator=g)
    ids = torch.empty((rows, top), dtype=torch.int32, device="cuda")
    p = torch.empty((rows, top), dtype=torch.float32, device="cuda")
    for b in (None, bias):
        native.router_topk(z.cuda(), None if b is None else b.cuda(), ids, p)
        zb = z if b is None else z + b           # (32-bit sums, as the kernel makes them)
        for r in range(rows):
            order = sorted(range(experts), key=lambda e: (-zb[r, e].item(), e))[:top]
            assert ids[r].tolist() == order, f"row {r}"
            want = torch.softmax(zb[r, order].double(), dim=0)
            assert (p[r].cpu().double() - want).abs().max().item() < 1e-6
    native.router_topk(z.cuda(), None, ids, p)
    assert ids[4].tolist() == list(range(top)) and (p[4].cpu() - 1.0 / top).abs().max().item() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows, width, ff, experts, top", [(1, 64, 24, 6, 2), (8, 72, 9, 3, 1), (20, 128, 64, 16, 4),
                                                          (3, 100, 14, 4, 4), (2, 64, 32, 16, 3), (5, 256, 40, 64, 4),
                                                          (64, 128, 48, 8, 2), (12, 100, 14, 16, 4),
                                                          (9, 72, 9, 6, 1), (40, 136, 20, 5, 3)])
def test_streamed_experts_alone(rows, width, ff, experts, top, dtype):
    """(pair by pair while the pairs are fewer than half the experts, expert by expert beyond)"""
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(rows + width)
    rnd = lambda *s: (torch.randn(s, generator=g) * 0.5).to(torch.bfloat16).float()  # noqa: E731
    x, gate, up, down = rnd(rows, width) * 2, rnd(experts, ff, width), rnd(experts, ff, width), rnd(experts, width, ff)
    base = rnd(rows, width)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).to(torch.int32)
    p = torch.softmax(torch.randn((rows, top), generator=g), dim=1)
    limit = 0.8
    ref = base.double().numpy().copy()
    for r in range(rows):
        for k in range(top):
            e = int(ids[r, k])
            ref[r] += p[r, k].item() * plain.expert(x[r:r + 1].double().numpy(), gate[e].double().numpy(),
                                                    up[e].double().numpy(), down[e].double().numpy(), limit)[0]
    out = torch.empty((rows, width), dtype=dtype, device="cuda")
    native.routed_rows(_dev(x, dtype), _dev(torch.cat([gate, up], dim=1), dtype), _dev(down, dtype), ids.cuda(),
                       p.cuda(), _dev(base, dtype), out, limit, 1.702)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(out.float().cpu().double().numpy() - ref).max() <= tol * np.abs(ref).max()
    # the activation alone, also with a weight per row
    gu = torch.cat([rnd(rows, ff) * 4, rnd(rows, ff) * 4], dim=1)
    y = torch.empty((rows, ff), dtype=dtype, device="cuda")
    native.expert_activate(_dev(gu, dtype), y, p[:, 0].contiguous().cuda(), limit, 1.702)
    gg, uu = gu[:, :ff].double().clamp(max=limit), gu[:, ff:].double().clamp(-limit, limit)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1) * p[:, :1].double()
    assert (y.float().cpu().double() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [64, 100, 1032])
def test_pair_norm_and_token_gate_alone(width, dtype):
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(width)
    rows = 37
    a, b = (torch.randn((rows, width), generator=g) * s for s in (3.0, 0.01))
    a, b = a.to(dtype).float(), b.to(dtype).float()
    wa, wb = torch.randn(width, generator=g), torch.randn(width, generator=g)
    y = native.pair_norm_mean(_dev(a, dtype), _dev(b, dtype), wa.cuda(), wb.cuda(),
                              torch.empty((rows, width), dtype=dtype, device="cuda"), 1e-6)
    ref = 0.5 * (plain.rms(a.double().numpy(), 1e-6) * wa.double().numpy() + plain.rms(b.double().numpy(), 1e-6) * wb.double().numpy())
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert np.abs(y.float().cpu().double().numpy() - ref).max() <= tol * np.abs(ref).max()
    dim = 5 if width == 100 else 8
    t = (torch.randn((rows, dim), generator=g) * 2).to(dtype).float()
    e = torch.randn((rows, 4 * dim), generator=g)
    out = native.gelu_gate_rows(_dev(t, dtype), e.cuda(), 2 * dim, torch.empty((rows, dim), dtype=dtype, device="cuda"))
    want = plain.gelu_tanh(t.double().numpy()) * e[:, 2 * dim:3 * dim].double().numpy()
    assert np.abs(out.float().cpu().double().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())


def write_model(path, cfg, weights):
    from strata_inference_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {n: t.to(torch.bfloat16) for n, t in weights.items()})
    return path


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_generation_engine(tmp_path, dtype):
    """Unequal prompts through generate(): every chosen token is the plain model's best (or
    within rounding of it) given the run's own history."""
    from strata_inference_b200 import GenerationConfig, GenerationEngine, SamplingConfig
    cfg = MIXED
    w = random_weights(cfg, seed=19)
    model_dir = write_model(str(tmp_path / "model"), cfg, w)
    engine = GenerationEngine.from_dir(model_dir, dtype=dtype, max_tokens=1024, ctx=256)
    reqs = prompts(cfg, [3, 40, 75], seed=20)
    outs = engine.generate(reqs, GenerationConfig(max_tokens=24, sampling=SamplingConfig(temperature=0.0)))
    tol = {"float32": 1e-4, "bfloat16": 0.15}[dtype]
    for prompt, out in zip(reqs, outs):
        assert len(out.token_ids) == 24 and out.stop_reason == "max_tokens"
        logits = plain_logits(cfg, w, list(prompt) + list(out.token_ids))
        for k, tok in enumerate(out.token_ids):
            row = logits[len(prompt) + k - 1]
            gap = (row.max() - row[tok]).item()
            assert gap <= tol * row.abs().max().item(), f"token {k} ({tok}) lies {gap:.3e} below the best"


def test_trace_replay_of_a_model_folder(tmp_path):
    """(the folder's decay path is 5 wide and 3 wide, which only its tensors say)"""
    cfg, dtype = ODD, "float32"
    w = random_weights(cfg, seed=21)
    stored = copy.deepcopy(cfg)
    for layer in stored["layers"]:
        layer["mixer"].pop("decay_rank", None)
    model_dir = write_model(str(tmp_path / "model"), stored, w)
    a, b = prompts(cfg, [80, 30], seed=22)
    ra, rb = plain_logits(cfg, w, a), plain_logits(cfg, w, b)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]},
                                     {"id": "b", "tokens": b[:20], "want": []}], "end": []}]
    for k in range(10):
        steps.append({"step": k + 1, "entries": [{"id": "a", "tokens": [a[70 + k]], "want": [0]},
                                                 {"id": "b", "tokens": [b[20 + k]], "want": [0] if k % 2 else []}],
                      "end": ["a", "b"] if k == 9 else []})
    out = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
                        "--dtype", dtype, "--out", out, "--max-tokens", "256"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {k}" for k in range(11)]
    V = cfg["vocab"]

    def read(step):
        return torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, V).copy())
    assert_close(read(0), torch.stack([ra[0], ra[69]]), dtype, "prompts")
    for k in range(10):
        want = [ra[70 + k]] + ([rb[20 + k]] if k % 2 else [])
        assert_close(read(k + 1), torch.stack(want), dtype, f"step {k + 1}")


def test_command_line_generates_from_a_model_folder(tmp_path):
    cfg = ALONE["delta_moe"]
    w = random_weights(cfg, seed=23)
    model_dir = write_model(str(tmp_path / "model"), cfg, w)
    prompt = prompts(cfg, [9], seed=24)[0]
    p = subprocess.run([sys.executable, "-m", "strata_inference_b200.cli", "-m", model_dir, "--token-ids",
                        ",".join(map(str, prompt)), "-n", "6", "--temp", "0", "--output-format", "json",
                        "--dtype", "float32"], capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-2000:]
    out = json.loads(p.stdout)
    tokens = out["output_token_ids"]
    assert len(tokens) == 6 and out["stop_reason"] == "max_tokens"
    logits = plain_logits(cfg, w, list(prompt) + list(tokens))
    for k, tok in enumerate(tokens):
        row = logits[len(prompt) + k - 1]
        assert (row.max() - row[tok]).item() <= 1e-4 * row.abs().max().item()


@pytest.mark.parametrize("heads, kv, hd, window, pool, lens", [(2, 2, 64, 40, 8, [300, 70, 9]), (4, 2, 128, 130, 16, [520, 200]),
                                                               (2, 1, 256, 17, 5, [150]), (2, 2, 64, 8, 24, [260, 131])])
def test_prompt_kernel_joins_the_blocks_before_the_window(heads, kv, hd, window, pool, lens):
    """The tensor cores' prompt kernel over the window, joined with the general kernel's sums
    over the blocks before it, against a 64-bit softmax over both: scores spread widely, so a
    block often carries a row; the general kernel alone over the same rows and cells as well."""
    from types import SimpleNamespace
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(heads * 1000 + hd + window)
    scale = 3.0 / math.sqrt(hd)
    cpt, per_seq = 16, 4                      # cells a page, pages of cells a sequence
    n_seqs = len(lens)
    order = torch.randperm(n_seqs * per_seq, generator=g).view(n_seqs, per_seq)
    cell_k = torch.zeros((n_seqs * per_seq, kv, cpt, hd), dtype=torch.bfloat16)
    cell_v = torch.zeros_like(cell_k)
    rows, refs, with_blocks = [], [], 0
    for b, T in enumerate(lens):
        q = torch.randn((T, heads, hd), generator=g).to(torch.bfloat16)
        k = torch.randn((T, kv, hd), generator=g).to(torch.bfloat16)
        v = torch.randn((T, kv, hd), generator=g).to(torch.bfloat16)
        nb = T // pool
        ck = k[:nb * pool].float().view(nb, pool, kv, hd).mean(1).to(torch.bfloat16)
        cv = v[:nb * pool].float().view(nb, pool, kv, hd).mean(1).to(torch.bfloat16)
        for c in range(nb):
            cell_k[order[b, c // cpt], :, c % cpt] = ck[c]
            cell_v[order[b, c // cpt], :, c % cpt] = cv[c]
        ref = torch.zeros((T, heads, hd), dtype=torch.float64)
        for i in range(T):
            lo, seen = max(0, i - window + 1), max(0, (i - window + 1) // pool)
            with_blocks += seen > 0
            for h in range(heads):
                kk = torch.cat([ck[:seen, h // (heads // kv)], k[lo:i + 1, h // (heads // kv)]]).double()
                vv = torch.cat([cv[:seen, h // (heads // kv)], v[lo:i + 1, h // (heads // kv)]]).double()
                ref[i, h] = torch.softmax(kk @ q[i, h].double() * scale, dim=0) @ vv
        refs.append(ref.view(T, -1))
        rows.append(torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1))
    assert with_blocks > sum(lens) // 2
    packed, ref = torch.cat(rows).contiguous().cuda(), torch.cat(refs)
    R, width = packed.shape
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    row0 = [sum(lens[:b]) for b in range(n_seqs)]
    cells = SimpleNamespace(cell_k=cell_k.cuda(), cell_v=cell_v.cuda(), cell_table=order.to(torch.int32).cuda(),
                            need=SimpleNamespace(pool=pool), cell_page_tokens=cpt)
    pos, seq = i32([i for T in lens for i in range(T)]), i32([b for b, T in enumerate(lens) for _ in range(T)])
    slot, start = i32(list(range(n_seqs))), i32([0] * n_seqs)

    def general(out, scratch, only):
        return native.attention_rows(packed, width, packed[:, heads * hd:], packed[:, (heads + kv) * hd:], width,
                                     None, None, None, 64, 0, pos, seq, slot, start, i32(row0), out, scratch,
                                     heads, kv, hd, scale, 0.0, window, 1, cells=cells, cells_only=only)
    out = general(torch.empty((R, heads * hd), dtype=torch.bfloat16, device="cuda"), None, False)
    err = (out.cpu().double() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item(), f"general kernel: {err:.3e}"
    extra = torch.full((R, heads, hd + 2), float("nan"), dtype=torch.float32, device="cuda")
    general(out, extra, True)
    assert torch.isfinite(extra[:, :, 1:]).all()
    out = torch.full((R, heads * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.attention_prefill_tc(packed, out, i32(row0), i32(lens), n_seqs, max(lens), heads, kv, hd, scale, 0.0,
                                window, extra=extra)
    assert native.attention_prefill_tc_error() == 0
    err = (out.cpu().double() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item(), f"prompt kernel with the blocks joined: {err:.3e}"
    n_items, need, n_tickets = native.attention_prefill_tc_plan(lens, heads, kv, hd, window)
    if n_items:
        out.fill_(float("nan"))
        native.attention_prefill_tc(packed, out, i32(row0), i32(lens), n_seqs, max(lens), heads, kv, hd, scale, 0.0,
                                    window, torch.empty(max(need, 16), dtype=torch.uint8, device="cuda"),
                                    torch.zeros(max(n_tickets, 1), dtype=torch.int32, device="cuda"), lens, extra=extra)
        assert native.attention_prefill_tc_error() == 0
        err = (out.cpu().double() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item(), f"as a list of work: {err:.3e}"


@pytest.mark.parametrize("name", sorted(BLOCKS_TC))
def test_long_prompts_on_the_tensor_cores_and_through_the_general_kernel_agree(name):
    from strata_inference_b200.parts import attention
    cfg = BLOCKS_TC[name]
    w = tie_queries_to_keys(random_weights(cfg, seed=41))
    a, b = asking_prompt(cfg, 300, seed=42), asking_prompt(cfg, 190, seed=43)
    ref = torch.cat([plain_logits(cfg, w, a), plain_logits(cfg, w, b)])
    got = {}
    for tc in (True, False):
        attention._USE_TCGEN05_PREFILL = tc
        try:
            eng = make_engine(cfg, w, "bfloat16")
            sa, sb = eng.new_sequence(), eng.new_sequence()
            got[tc] = eng.step([(sa, a), (sb, b)], [all_rows(300), all_rows(190)]).cpu().double()
        finally:
            attention._USE_TCGEN05_PREFILL = True
        assert_close(got[tc], ref, "bfloat16", f"{name}, tensor cores: {tc}")
    diff = (got[True] - got[False]).abs().amax(-1) / ref.abs().max()
    assert diff.median().item() <= 1.5e-2 and (diff > 4e-2).float().mean().item() <= 0.1, \
        f"median {diff.median().item():.3e}, worst {diff.max().item():.3e}"
