"""Besorax through the engine against the plain model (tests/plain_besorax.py): each mechanism
alone, prompts against token-by-token steps, portions, unequal batches, slots and pages used
again, the chunks' edges, the sink and keys far back with a softmax that picks single keys, a
layer that reads another's keys and values, the first tokens of a sequence, long decoding,
odd and wide sizes, the kernels alone, greedy generation and trace replay."""

from __future__ import annotations

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_besorax as plain
from besorax_cases import (ALONE, MIXED, ODD, SHARP, WIDE, assert_close, attention, changed, decisive_routers, dense,
                           lightning, model, moe, plain_logits, prompts, random_model, random_weights, rows_that_differ)

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
    """The prompt cut into steps of the given sizes (the last takes the rest)."""
    s, at, rows = eng.new_sequence(), 0, []
    for n in list(sizes) + [len(tokens)]:
        part = tokens[at:at + n]
        if not part:
            break
        rows.append(eng.step([(s, part)], [all_rows(len(part))]))
        at += len(part)
    eng.end_sequence(s)
    return torch.cat(rows)


def weights_for(cfg, seed, dtype):
    """(bfloat16 runs get routers whose scores lie far apart: a close call would send a row to
    another expert than the plain model's)"""
    w = random_weights(cfg, seed=seed)
    return decisive_routers(w) if dtype == "bfloat16" else w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(name, dtype):
    cfg = ALONE[name]
    w = weights_for(cfg, 11, dtype)
    eng = make_engine(cfg, w, dtype)
    for toks in prompts(cfg, [1, 2, 5, 90], seed=3):
        assert_close(run_whole(eng, toks), plain_logits(cfg, w, toks), dtype, f"{name}, {len(toks)} tokens")
    toks = prompts(cfg, [95], seed=4)[0]
    assert_close(run_portions(eng, toks, [3, 1, 1, 2, 50] + [1] * 8), plain_logits(cfg, w, toks), dtype,
                 f"{name} in portions and single tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_then_long_decoding(dtype):
    """A prompt in one step, then 260 single-token steps (over page borders and through several
    chunks of every size; the token steps are recorded at the second and replayed from the
    third), and token by token from the very first token."""
    cfg = MIXED
    w = weights_for(cfg, 5, dtype)
    eng = make_engine(cfg, w, dtype)
    toks = prompts(cfg, [300], seed=6)[0]
    ref = plain_logits(cfg, w, toks)
    assert_close(run_portions(eng, toks, [40] + [1] * 260), ref, dtype, "prompt of 40, then token by token")
    assert_close(run_portions(eng, toks[:50], [1] * 30 + [20]), ref[:50], dtype, "token by token from the first token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [[2, 2, 2, 2], [64, 25], [63, 2, 24], [1, 24, 3, 23], [17, 17, 17, 17, 17],
                                   [7, 8, 9, 16, 1, 15, 24], [39, 1, 1, 23, 2], [40, 40, 20, 39, 2]])
def test_portions(sizes, dtype):
    """(the chunks of the mixed model are 40, 100 and 70 positions; the last two lists cut at the
    first one's edges, the one before them around the scan's chunks of 8)"""
    cfg = MIXED
    w = weights_for(cfg, 7, dtype)
    eng = make_engine(cfg, w, dtype)
    toks = prompts(cfg, [150], seed=8)[0]
    assert_close(run_portions(eng, toks, sizes + [20] * 8), plain_logits(cfg, w, toks), dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_against_each_alone(dtype):
    """Prompts of 1 to 130 tokens in one step, then single-token steps together; the
    shorter requests end earlier and a new one takes a freed slot later."""
    cfg = MIXED
    w = weights_for(cfg, 9, dtype)
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
    """A slot that is given back and taken again starts from nothing: state and pages of the
    request before leave no trace; with few pages they are all used again."""
    cfg = MIXED
    w = weights_for(cfg, 12, dtype)
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


def test_chunk_edges_sinks_and_far_keys_with_a_sharp_softmax():
    """With a large scale the softmax puts most of a row's weight on single keys, wherever in
    the chunk they lie.  The plain model with chunks one shorter or one longer gives other
    logits in most rows (that is checked first: the test can tell them apart); the engine
    agrees with the right one as a prompt, in portions around page borders and the chunks'
    edges, token by token, and as two requests whose chunks begin in different rows."""
    cfg, dtype = SHARP, "float32"
    w = random_weights(cfg, seed=14)
    toks = prompts(cfg, [330], seed=15)[0]
    ref = plain_logits(cfg, w, toks)

    def chunk(delta):
        def edit(c):
            for layer in c["layers"]:
                layer["mixer"]["mask"]["size"] += delta
        return edit
    for delta in (-1, 1):
        other = plain_logits(changed(cfg, chunk(delta)), w, toks)
        assert rows_that_differ(ref[66:], other[66:], 20.0) > 150, f"chunks off by {delta} would not show"
    eng = make_engine(cfg, w, dtype)
    assert_close(run_whole(eng, toks), ref, dtype, "whole prompt")
    assert_close(run_portions(eng, toks, [64, 64, 64, 64]), ref, dtype, "portions of one page")
    assert_close(run_portions(eng, toks, [63, 2, 63, 1, 1, 20, 66, 60]), ref, dtype, "portions around page borders")
    assert_close(run_portions(eng, toks, [66, 34, 32, 66, 1, 1, 63, 1, 1, 34]), ref, dtype, "portions at the chunks' edges")
    assert_close(run_portions(eng, toks, [65, 2, 32, 2, 97, 2]), ref, dtype, "portions across the chunks' edges")
    assert_close(run_portions(eng, toks, [60] + [1] * 270), ref, dtype, "single tokens through several chunks")
    a, b = toks[:250], prompts(cfg, [180], seed=16)[0]
    rb = plain_logits(cfg, w, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([(sa, a[:195]), (sb, b[:98])], [all_rows(195), all_rows(98)])
    assert_close(out, torch.cat([ref[:195], rb[:98]]), dtype, "two prompts")
    for k in range(50):
        out = eng.step([(sa, [a[195 + k]]), (sb, [b[98 + k]])], [[0], [0]])
        assert_close(out, torch.stack([ref[195 + k], rb[98 + k]]), dtype, f"two requests, token {k}")


def _asking_model(chunk):
    """One attention layer, one head, no rotation, whose query and key matrices are the same
    and large: a token's strongest key is the last earlier occurrence of the same token."""
    return model(32, 50, [attention(1, 1, 16, 16, chunk, scale=4.0, rot_dims=0)], scale=1.0, mult=1.0)


def _asking_weights(cfg, seed):
    w = random_weights(cfg, seed)
    w["l0.mix.k"] = w["l0.mix.q"].clone()
    w["l0.mix.sink"] = w["l0.mix.sink"] - 20.0
    return w


@pytest.mark.parametrize("mode", ["prompt", "tokens"])
def test_a_key_just_inside_and_just_outside_a_chunk(mode):
    """A token asks for its own earlier occurrence.  When that lies at the first position of
    the asking row's chunk it is seen; one position earlier, at the last position of the chunk
    before, it is not; the row's logits differ widely between the two (checked on the plain
    model first), in a prompt and when the asking token is decoded alone.  Also a key hundreds of
    positions back in a chunk that is longer than that."""
    for chunk, back in ((48, 30), (48, 47), (64, 63), (400, 390)):
        cfg = _asking_model(chunk)
        w = _asking_weights(cfg, 40)
        for start in (2 * chunk, 2 * chunk - 1):          # the asked-for token's position
            n = start + back + 1
            if n > 1000:
                continue
            toks = [3 + (i % 40) for i in range(n)]
            toks[start] = toks[n - 1] = 47                  # token 47 occurs at `start` and asks at the end
            ref = plain_logits(cfg, w, toks)
            blind = list(toks)
            blind[start] = 46
            seen = start // chunk == (n - 1) // chunk
            moved = rows_that_differ(ref[-1:], plain_logits(cfg, w, blind)[-1:], 50.0)
            assert moved == (1 if seen else 0), (chunk, back, start, seen)
            eng = make_engine(cfg, w, "float32")
            got = run_whole(eng, toks) if mode == "prompt" else run_portions(eng, toks, [n - 20] + [1] * 20)
            assert_close(got, ref, "float32", f"chunk {chunk}, key {back} back at {start} ({mode})")


def test_sinks_that_take_much_of_the_weight():
    """Sinks raised by 3 take a large share of every row's weight; without them every row's
    logits are others (checked first).  Prompt, portions, tokens, and a batch; the attention
    with chunks and the latent attention."""
    for name in ("attention", "latent"):
        cfg, dtype = ALONE[name], "float32"
        w = {n: (t + 3.0 if n.endswith(".sink") else t) for n, t in random_weights(cfg, seed=26).items()}
        a, b = prompts(cfg, [200, 77], seed=27)
        ra, rb = plain_logits(cfg, w, a), plain_logits(cfg, w, b)
        no_sink = {n: (t - 30.0 if n.endswith(".sink") else t) for n, t in w.items()}
        assert rows_that_differ(ra, plain_logits(cfg, no_sink, a), 30.0) == 200, "a sink left out would not show"
        eng = make_engine(cfg, w, dtype)
        assert_close(run_whole(eng, a), ra, dtype, f"{name}: whole prompt")
        assert_close(run_portions(eng, a, [30, 2, 50] + [1] * 100), ra, dtype, f"{name}: portions and single tokens")
        sa, sb = eng.new_sequence(), eng.new_sequence()
        out = eng.step([(sa, a[:150]), (sb, b[:60])], [all_rows(150), all_rows(60)])
        assert_close(out, torch.cat([ra[:150], rb[:60]]), dtype, f"{name}: two prompts")
        for k in range(17):
            out = eng.step([(sa, [a[150 + k]]), (sb, [b[60 + k]])], [[0], [0]])
            assert_close(out, torch.stack([ra[150 + k], rb[60 + k]]), dtype, f"{name}: two requests, token {k}")


def test_lent_keys_are_the_lenders_rotated_keys():
    """The borrowing layer's logits change when the LENDER's key matrix changes, and a plain
    model that lets the borrower see every position (its own mask dropped) differs: the
    borrower reads the lender's cache through its own chunks."""
    cfg, dtype = MIXED, "float32"
    w = random_weights(cfg, seed=30)
    toks = prompts(cfg, [160], seed=31)[0]
    ref = plain_logits(cfg, w, toks)
    other = changed(cfg, lambda c: c["layers"][5]["mixer"].pop("mask"))
    assert rows_that_differ(ref[70:], plain_logits(other, w, toks)[70:], 10.0) > 60
    eng = make_engine(cfg, w, dtype)
    assert_close(run_whole(eng, toks), ref, dtype, "whole prompt")
    assert_close(run_portions(eng, toks, [69, 1, 1, 1, 38, 2] + [1] * 40), ref, dtype, "portions at the borrower's edges")


def test_first_tokens_of_a_sequence():
    cfg, dtype = MIXED, "float32"
    w = random_weights(cfg, seed=24)
    toks = prompts(cfg, [40], seed=25)[0]
    ref = plain_logits(cfg, w, toks)
    eng = make_engine(cfg, w, dtype, max_slots=1)
    assert_close(run_portions(eng, toks, [1, 1, 1, 2, 2, 5]), ref, dtype, "first tokens one by one")
    assert_close(run_portions(eng, toks[::-1], [3, 1]), plain_logits(cfg, w, toks[::-1]), dtype, "the slot again")
    assert_close(run_whole(eng, toks[:1]), ref[:1], dtype, "one token alone")


def test_a_long_memory_in_lightning_attention():
    """A head whose decay is 1 keeps what the first tokens wrote: the plain model's last rows
    change when the first token changes (checked first), and the engine agrees after 500
    tokens in portions and single-token steps."""
    cfg, dtype = model(48, 60, [lightning(2, 16, 16, [1.0, 0.9])], mult=1.0), "float32"
    w = random_weights(cfg, seed=33)
    toks = prompts(cfg, [500], seed=34)[0]
    ref = plain_logits(cfg, w, toks)
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert rows_that_differ(ref[-20:], plain_logits(cfg, w, other)[-20:], 3.0) == 20
    eng = make_engine(cfg, w, dtype)
    assert_close(run_portions(eng, toks, [200, 2, 150, 100] + [1] * 48), ref, dtype, "500 tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_other_sizes(name, dtype):
    cfg = {"odd": ODD, "wide": WIDE}[name]
    w = weights_for(cfg, 17, dtype)
    eng = make_engine(cfg, w, dtype)
    toks = prompts(cfg, [200], seed=18)[0]
    ref = plain_logits(cfg, w, toks)
    assert_close(run_whole(eng, toks), ref, dtype, f"{name}: whole prompt")
    assert_close(run_portions(eng, toks, [33, 2, 60, 64] + [1] * 41), ref, dtype, f"{name}: portions and tokens")
    a, b = toks[:150], prompts(cfg, [60], seed=19)[0]
    rb = plain_logits(cfg, w, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([(sa, a[:140]), (sb, b[:50])], [all_rows(140), all_rows(50)])
    assert_close(out, torch.cat([ref[:140], rb[:50]]), dtype, f"{name}: two prompts")
    for k in range(10):
        out = eng.step([(sa, [a[140 + k]]), (sb, [b[50 + k]])], [[0], [0]])
        assert_close(out, torch.stack([ref[140 + k], rb[50 + k]]), dtype, f"{name}: two requests, token {k}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", list(range(12)))
def test_configurations_drawn_at_random(seed, dtype):
    """Any order of layers, any lender, any of the sizes: a prompt, portions down to two tokens with
    single tokens behind them, and two unequal requests together."""
    cfg = random_model(seed)
    w = weights_for(cfg, 70 + seed, dtype)
    eng = make_engine(cfg, w, dtype)
    toks = prompts(cfg, [170], seed=seed)[0]
    ref = plain_logits(cfg, w, toks)
    assert_close(run_whole(eng, toks), ref, dtype, f"drawn model {seed}: whole prompt")
    assert_close(run_portions(eng, toks, [70, 2, 30, 18] + [1] * 50), ref, dtype, f"drawn model {seed}: portions and tokens")
    a, b = toks[:120], prompts(cfg, [60], seed=seed + 100)[0]
    rb = plain_logits(cfg, w, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([(sa, a[:101]), (sb, b[:33])], [all_rows(101), all_rows(33)])
    assert_close(out, torch.cat([ref[:101], rb[:33]]), dtype, f"drawn model {seed}: two prompts")
    for k in range(19):
        out = eng.step([(sa, [a[101 + k]]), (sb, [b[33 + k]])], [[0], [0]])
        assert_close(out, torch.stack([ref[101 + k], rb[33 + k]]), dtype, f"drawn model {seed}: two requests, token {k}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_many_rows_choose_their_experts(dtype):
    """Prompts long enough for the experts to run as batched products over sorted rows, beside the
    same rows in steps short enough to stream each pair's expert."""
    cfg = model(64, 120, [lightning(2, 16, 16, [0.9, 0.99], mlp=moe(6, 3, 24, shared=16)),
                          attention(2, 1, 16, 16, 90, mlp=moe(5, 1, 40))])
    w = weights_for(cfg, 50, dtype)
    eng = make_engine(cfg, w, dtype)
    toks = prompts(cfg, [400], seed=51)[0]
    ref = plain_logits(cfg, w, toks)
    assert_close(run_whole(eng, toks), ref, dtype, "400 rows in one step")
    assert_close(run_portions(eng, toks, [300, 33, 20, 8, 5] + [1] * 34), ref, dtype, "fewer and fewer rows")


@pytest.mark.parametrize("dtype", DTYPES)
def test_recorded_steps_of_many_rows_choose_their_experts(dtype):
    """48 requests decoded together: their single-token steps are recorded and replayed, and the
    experts of so many rows run as batched products with room for every row at every expert."""
    cfg = model(64, 120, [lightning(2, 16, 16, [0.9, 0.99], mlp=moe(6, 3, 24, shared=16)),
                          attention(2, 1, 16, 16, 20, mlp=moe(5, 1, 40))])
    w = weights_for(cfg, 52, dtype)
    eng = make_engine(cfg, w, dtype, max_tokens=4096, max_slots=48)
    reqs = prompts(cfg, [9 + (i * 7) % 23 for i in range(48)], seed=53)
    refs = [plain_logits(cfg, w, t) for t in reqs]
    slots = [eng.new_sequence() for _ in reqs]
    eng.step([(s, t[:4]) for s, t in zip(slots, reqs)], [[3]] * 48)
    for k in range(4, 9):
        out = eng.step([(s, [t[k]]) for s, t in zip(slots, reqs)], [[0]] * 48)
        assert_close(out, torch.stack([r[k] for r in refs]), dtype, f"48 requests, token {k}")


# --------------------------------------------------------------------------
# kernels alone, against plain functions


def _dev(t, dtype=torch.float32):
    return t.to("cuda", dtype).contiguous()


@pytest.mark.parametrize("rows, experts, top", [(1, 8, 1), (5, 6, 3), (40, 7, 7), (300, 33, 4)])
def test_router_scores_are_sigmoids_of_the_chosen(rows, experts, top):
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(rows)
    z = torch.randn((rows, experts), generator=g) * 2
    ids = torch.empty((rows, top), dtype=torch.int32, device="cuda")
    p = torch.empty((rows, top), dtype=torch.float32, device="cuda")
    native.router_topk(_dev(z), None, ids, p, native.SCORE_SIGMOID)
    s = plain.sigmoid(z.double().numpy())
    for r in range(rows):
        want = np.argsort(-s[r], kind="stable")[:top]
        assert ids[r].tolist() == want.tolist()
        assert np.allclose(p[r].cpu().numpy(), s[r][want], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows, width, experts, top", [(1, 64, 8, 2), (5, 100, 16, 3), (8, 256, 40, 4), (32, 72, 33, 1)])
def test_router_of_few_rows(rows, width, experts, top, dtype):
    """The router's 32-bit product and the choice in one call, with few and with many experts (the
    logits of 16 and more are made by many blocks): ids and sigmoid scores against the plain sort."""
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(rows + experts)
    x = torch.randn((rows, width), generator=g).to(dtype).float()
    w = torch.randn((experts, width), generator=g) * 0.3
    ids = torch.empty((rows, top), dtype=torch.int32, device="cuda")
    p = torch.empty((rows, top), dtype=torch.float32, device="cuda")
    native.router_rows(_dev(x, dtype), _dev(w), None, ids, p, native.SCORE_SIGMOID)
    s = plain.sigmoid(x.double().numpy() @ w.double().numpy().T)
    for r in range(rows):
        want = np.argsort(-s[r], kind="stable")[:top]
        assert ids[r].tolist() == want.tolist()
        assert np.allclose(p[r].cpu().numpy(), s[r][want], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows, width, ff, experts, top", [(1, 64, 24, 4, 1), (3, 72, 10, 5, 2), (20, 128, 97, 6, 3),
                                                          (32, 256, 64, 40, 4)])
def test_streamed_experts_without_a_gate(rows, width, ff, experts, top, dtype):
    """out = base + sum_k down_k(gelu(p_k up_k x)) against the plain expert; both layouts of the
    launch (pair by pair, expert by expert)."""
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(rows * 7 + ff)
    x = (torch.randn((rows, width), generator=g) * 0.7).to(dtype).float()
    up = (torch.randn((experts, ff, width), generator=g) / math.sqrt(width)).to(dtype).float()
    down = (torch.randn((experts, width, ff), generator=g) / math.sqrt(ff)).to(dtype).float()
    base = (torch.randn((rows, width), generator=g) * 0.3).to(dtype).float()
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).to(torch.int32)
    p = torch.rand((rows, top), generator=g) * 0.9 + 0.05
    out = torch.empty((rows, width), dtype=dtype, device="cuda")
    native.routed_rows(_dev(x, dtype), _dev(up, dtype), _dev(down, dtype), ids.cuda(), _dev(p), _dev(base, dtype), out,
                       0.0, 1.702, native.FORM_PLAIN_GELU)
    want = base.double().numpy().copy()
    for r in range(rows):
        for k in range(top):
            e = int(ids[r, k])
            want[r] += plain.small_ff(float(p[r, k]) * x[r].double().numpy(), up[e].double().numpy(), down[e].double().numpy())
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk, heads, kv, hd", [(7, 4, 2, 16), (64, 2, 2, 64), (100, 8, 2, 128), (1, 2, 1, 32)])
def test_general_attention_kernel_with_chunks_and_sinks(chunk, heads, kv, hd, dtype):
    """Rows of two sequences over their packed keys: every row sees its own chunk, and the
    sink joins the denominator."""
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(chunk)
    lens = [150, 37]
    R = sum(lens)
    qkv = (torch.randn((R, (heads + 2 * kv) * hd), generator=g) * 0.8).to(dtype).float()
    sink = torch.randn((heads,), generator=g)
    row_pos = torch.tensor([p for n in lens for p in range(n)], dtype=torch.int32)
    row_seq = torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], dtype=torch.int32)
    seq_row0 = torch.tensor([0, lens[0]], dtype=torch.int32)
    seq_start = torch.zeros(2, dtype=torch.int32)
    seq_slot = torch.tensor([0, 1], dtype=torch.int32)
    d_qkv = _dev(qkv, dtype)
    out = torch.empty((R, heads * hd), dtype=dtype, device="cuda")
    width = qkv.shape[1]
    native.attention_rows(d_qkv, width, d_qkv[:, heads * hd:], d_qkv[:, (heads + kv) * hd:], width, None, None, None,
                          64, 0, row_pos.cuda(), row_seq.cuda(), seq_slot.cuda(), seq_start.cuda(), seq_row0.cuda(),
                          out, None, heads, kv, hd, 0.3, 0.0, 0, 1, sink=_dev(sink), chunk=chunk)
    q = qkv[:, :heads * hd].double().numpy().reshape(R, heads, hd)
    k = qkv[:, heads * hd:(heads + kv) * hd].double().numpy().reshape(R, kv, hd)
    v = qkv[:, (heads + kv) * hd:].double().numpy().reshape(R, kv, hd)
    want = np.zeros((R, heads, hd))
    for r in range(R):
        t, r0 = int(row_pos[r]), int(seq_row0[int(row_seq[r])])
        lo = plain.visible_from(t, chunk)
        for a in range(heads):
            gq = a // (heads // kv)
            s = (k[r0 + lo:r0 + t + 1, gq] @ q[r, a]) * 0.3
            want[r, a] = plain.softmax_with_sink(s, float(sink[a])) @ v[r0 + lo:r0 + t + 1, gq]
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(out.float().cpu().numpy().reshape(R, heads, hd) - want).max() <= tol


def _chunked_reference(q, k, v, sink, scale, chunk):
    """q[T, H, d], k and v [T, G, d] of one sequence (bfloat16 values): rows of a 64-bit softmax
    over the row's own chunk with the sink in the denominator."""
    T, H, d = q.shape
    G = k.shape[1]
    q, k, v = (x.double().numpy() for x in (q, k, v))
    out = np.zeros((T, H, d))
    for t in range(T):
        lo = plain.visible_from(t, chunk)
        for a in range(H):
            s = (k[lo:t + 1, a // (H // G)] @ q[t, a]) * scale
            out[t, a] = plain.softmax_with_sink(s, None if sink is None else float(sink[a])) @ v[lo:t + 1, a // (H // G)]
    return out


@pytest.mark.parametrize("nh, nkv, hd, chunk, splits, warps", [
    (4, 2, 128, 96, 1, 4), (4, 2, 128, 96, 3, 4), (8, 1, 64, 40, 5, 2), (2, 2, 256, 16, 2, 8), (8, 4, 256, 100, 20, 4),
    (16, 2, 64, 7, 1, 1), (4, 4, 128, 1, 2, 4), (8, 2, 128, 1000, 40, 8), (2, 1, 128, 33, 70, 8)])
def test_decode_kernel_with_chunks_and_sinks(nh, nkv, hd, chunk, splits, warps):
    """The bfloat16 decode kernel over a paged cache whose pages lie in any order: rows at the
    first and last positions of chunks, at tile and page borders; sinks far above and far below
    the scores; every way of joining the runs."""
    from strata_inference_b200.kernels import native
    assert native.attention_decode_supports(nh, nkv, hd, 16)
    g = torch.Generator().manual_seed(nh * hd + chunk)
    T, page = 230, 16
    q = torch.randn((T, nh, hd), generator=g).to(torch.bfloat16)
    k = torch.randn((T, nkv, hd), generator=g).to(torch.bfloat16)
    v = torch.randn((T, nkv, hd), generator=g).to(torch.bfloat16)
    sink = torch.randn(nh, generator=g) * 4.0 + 1.0
    scale = 3.0 / math.sqrt(hd)
    ref = _chunked_reference(q, k, v, sink, scale, chunk)
    n_pages = -(-T // page)
    order = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    kp = torch.full((n_pages + 3, nkv, page, hd), 1e4, dtype=torch.bfloat16)      # (loud if read)
    vp = torch.full((n_pages + 3, nkv, page, hd), 1e4, dtype=torch.bfloat16)
    for t in range(T):
        kp[order[t // page], :, t % page], vp[order[t // page], :, t % page] = k[t], v[t]
    table = torch.zeros((2, n_pages), dtype=torch.int32)
    table[1] = order.to(torch.int32)
    edges = {0, 1, 15, 16, 17, T - 1}
    for c in range(0, T, max(chunk, 1)):
        edges |= {c, c + 1, c + chunk - 1, c + chunk // 2}
    rows = sorted(r for r in edges if 0 <= r < T)[:40]
    R = len(rows)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    qs = torch.stack([q[r].reshape(nh * hd) for r in rows]).contiguous().cuda()
    out = torch.empty((R, nh * hd), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(max(1, native.attention_rows_scratch_bytes(R, nh, hd, splits)), dtype=torch.uint8, device="cuda")
    tickets = torch.zeros(R * nkv, dtype=torch.int32, device="cuda")
    native.attention_decode(qs, nh * hd, kp.cuda(), vp.cuda(), table.cuda(), page, 0, i32(rows), i32([0] * R), i32([1]),
                            out, scratch, tickets, nh, nkv, hd, scale, 0.0, 0, splits, warps, chunk=chunk, sink=sink.cuda())
    assert int(tickets.abs().sum()) == 0, "the ticket counters are put back"
    got = out.float().cpu().numpy().reshape(R, nh, hd)
    for i, r in enumerate(rows):
        err = np.abs(got[i] - ref[r]).max()
        assert err <= 2e-2 * max(1.0, np.abs(ref[r]).max()), f"row at position {r}: {err:.3e}"


@pytest.mark.parametrize("heads, kv, hd, chunk, lens", [(4, 2, 128, 96, [398, 23, 97]), (4, 4, 64, 40, [200, 5, 64, 131]),
                                                        (2, 1, 256, 128, [700, 130]), (8, 4, 128, 1, [50]),
                                                        (2, 2, 128, 5000, [1500]), (6, 3, 64, 0, [300, 90])])
def test_prompt_kernel_over_chunks_with_sinks(heads, kv, hd, chunk, lens):
    """The tcgen05 prompt kernel with every chunk of a prompt as a sequence of its own and a sink
    per head, against the 64-bit softmax over the row's chunk: as a grid and as a balanced list."""
    from strata_inference_b200.kernels import native
    if not native.attention_prefill_tc_supports(heads, kv, hd, (heads + 2 * kv) * hd):
        pytest.skip("not a shape of the prompt kernel")
    g = torch.Generator().manual_seed(heads + hd + chunk)
    scale = 3.0 / math.sqrt(hd)
    sink = torch.randn(heads, generator=g) * 3.0 + 2.0
    rows, refs, row0, sizes, at = [], [], [], [], 0
    for T in lens:
        q = torch.randn((T, heads, hd), generator=g).to(torch.bfloat16)
        k, v = (torch.randn((T, kv, hd), generator=g).to(torch.bfloat16) for _ in range(2))
        refs.append(_chunked_reference(q, k, v, sink, scale, chunk))
        rows.append(torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1))
        step = chunk or T
        for c in range(0, T, step):
            row0.append(at + c)
            sizes.append(min(step, T - c))
        at += T
    packed = torch.cat(rows).contiguous().cuda()
    ref = np.concatenate(refs).reshape(sum(lens), -1)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731

    def run(scratch, tickets, host):
        out = torch.full((sum(lens), heads * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        native.attention_prefill_tc(packed, out, i32(row0), i32(sizes), len(sizes), max(sizes), heads, kv, hd, scale,
                                    0.0, 0, scratch, tickets, host, sink=sink.cuda())
        assert native.attention_prefill_tc_error() == 0
        err = np.abs(out.float().cpu().numpy() - ref).max()
        assert err <= 2e-2 * np.abs(ref).max(), f"{err:.3e} of {np.abs(ref).max():.3e}"
    run(None, None, None)
    n_items, need, n_tickets = native.attention_prefill_tc_plan(sizes, heads, kv, hd, 0)
    if n_items:
        run(torch.empty(max(need, 16), dtype=torch.uint8, device="cuda"),
            torch.zeros(max(n_tickets, 1), dtype=torch.int32, device="cuda"), sizes)


@pytest.mark.parametrize("dtype", DTYPES)
def test_heads_of_the_fast_kernels_through_the_engine(dtype):
    """Heads of 64 and 128 with two query heads a key head: bfloat16 prompts take the tcgen05
    prompt kernel chunk by chunk (the borrower over the lender's rows), single rows the decode
    kernel; portions of several rows go row by row over the cache."""
    cfg = model(96, 150, [attention(4, 2, 64, 64, 48, rot_dims=16, scale=0.3, mlp=dense(64)),
                          attention(4, 2, 64, 64, 80, rot_dims=16, scale=0.3, kv_from=0),
                          attention(2, 1, 128, 128, 0, scale=0.2),
                          attention(4, 2, 64, 64, 200, rot_dims=16, scale=0.3, kv_from=0, mlp=dense(32))])
    w = random_weights(cfg, seed=61)
    eng = make_engine(cfg, w, dtype)
    toks = prompts(cfg, [330], seed=62)[0]
    ref = plain_logits(cfg, w, toks)
    assert_close(run_whole(eng, toks), ref, dtype, "whole prompt")
    assert_close(run_portions(eng, toks, [150, 2, 40, 48] + [1] * 90), ref, dtype, "portions and single tokens")
    a, b = toks[:260], prompts(cfg, [120], seed=63)[0]
    rb = plain_logits(cfg, w, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([(sa, a[:200]), (sb, b[:47])], [all_rows(200), all_rows(47)])
    assert_close(out, torch.cat([ref[:200], rb[:47]]), dtype, "two prompts")
    for k in range(60):
        out = eng.step([(sa, [a[200 + k]]), (sb, [b[47 + k]])], [[0], [0]])
        assert_close(out, torch.stack([ref[200 + k], rb[47 + k]]), dtype, f"two requests, token {k}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows, inter", [(1, 264), (8, 264), (12, 100), (130, 264), (300, 264), (300, 100), (40, 7)])
def test_clipped_gated_feed_forward_alone(rows, inter, dtype):
    """The dense feed-forward part alone at row counts that take the weight-streaming product with
    the clipped epilogue, the library's product with the activation behind it, and the tensor-core
    product with the epilogue; widths that are and are not multiples of 8; values beyond the limit."""
    from strata_inference_b200.parts.base import Runtime, build_part
    from strata_inference_b200.parts.feed_forward import ClippedGatedMLP
    g = torch.Generator().manual_seed(rows + inter)
    hidden = 128
    stored = {"gate_proj.weight": torch.randn((inter, hidden), generator=g) * 0.25,
              "up_proj.weight": torch.randn((inter, hidden), generator=g) * 0.25,
              "down_proj.weight": torch.randn((hidden, inter), generator=g) * 0.2}
    stored = {n: t.to(torch.bfloat16) for n, t in stored.items()}
    rt = Runtime("cuda:0", dtype)
    part = build_part(ClippedGatedMLP, ({"intermediate_size": inter, "limit": 1.5, "alpha": 1.702}, hidden),
                      {n: t.cuda() for n, t in stored.items()}, rt)
    x = torch.randn((rows, hidden), generator=g).to(torch.bfloat16)
    got = part.forward(x.cuda().to(dtype), None).float().cpu().double().numpy()
    w = {n.split("_")[0]: plain.f64(t.float()) for n, t in stored.items()}
    assert (plain.f64(x.float()) @ w["gate"].T).max() > 1.5 and (plain.f64(x.float()) @ w["up"].T).min() < -1.5
    ref = plain.clipped_gated_ff(plain.f64(x.float()), w, 1.5)
    assert np.abs(got - ref).max() <= (1e-4 if dtype == torch.float32 else 2e-2) * np.abs(ref).max()


@pytest.mark.parametrize("rows, heads, vd", [(1, 1, 2048), (9, 1, 600), (5, 3, 512), (40, 1, 1000)])
def test_norm_and_gate_over_many_columns(rows, heads, vd):
    """Heads of 512 columns and more (all heads normed together count as one) take a block a
    row: x / rms(x) * w * sigmoid(gate) against the plain formula."""
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(vd)
    o = torch.randn((rows, heads * vd), generator=g) * 3
    w = torch.randn(heads * vd, generator=g)
    gate = torch.randn((rows, heads * vd + 8), generator=g).to(torch.bfloat16)
    y = torch.empty((rows, heads * vd), dtype=torch.bfloat16, device="cuda")
    native.head_norm_gate(_dev(o), None, _dev(w), gate.cuda()[:, :heads * vd], y, heads, vd, 1e-5, native.GATE_SIGMOID)
    x = o.double().numpy().reshape(rows, heads, vd)
    want = plain.unit_rms(x, 1e-5) * w.double().numpy().reshape(heads, vd) * plain.sigmoid(
        gate[:, :heads * vd].double().numpy().reshape(rows, heads, vd))
    assert np.abs(y.float().cpu().numpy().reshape(rows, heads, vd) - want).max() <= 2e-2 * np.abs(want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_add_with_a_factor(dtype):
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(1)
    a = torch.randn((9, 100), generator=g).to(dtype).float()
    h = torch.randn((9, 100), generator=g)
    w, b, al = torch.randn(100, generator=g), torch.randn(100, generator=g), torch.tensor([0.7])
    d_h = _dev(h)
    out = torch.empty((9, 100), dtype=dtype, device="cuda")
    native.add_dyt_norm(_dev(a, dtype), None, d_h, (_dev(w), _dev(b), _dev(al)), out, 0.35)
    want_h = h.double() + 0.35 * a.double()
    assert (d_h.cpu().double() - want_h).abs().max() < 1e-5
    want = torch.from_numpy(plain.dynamic_tanh(want_h.numpy(), w.double().numpy(), b.double().numpy(), 0.7))
    assert (out.cpu().double() - want).abs().max() < (1e-5 if dtype == torch.float32 else 3e-2)


# --------------------------------------------------------------------------
# the engine's own entry points


def _write_model(path, cfg, weights):
    from strata_inference_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {n: t.to(torch.bfloat16) for n, t in weights.items()})
    return path


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_generation_engine(tmp_path, dtype):
    """Several prompts through GenerationEngine.generate (its scheduler batches them): every
    chosen token is the plain model's best, or so near it that rounding decides, given the run's
    own history."""
    from strata_inference_b200 import GenerationConfig, GenerationEngine, SamplingConfig
    cfg = MIXED
    w = weights_for(cfg, 21, dtype)
    path = _write_model(str(tmp_path / "m"), cfg, w)
    engine = GenerationEngine.from_dir(path, dtype=dtype, max_tokens=1024)
    reqs = prompts(cfg, [5, 47, 90, 13], seed=22)
    outs = engine.generate(reqs, GenerationConfig(max_tokens=24, sampling=SamplingConfig(temperature=0.0)))
    tol = {"float32": 1e-4, "bfloat16": 0.15}[dtype]
    far = total = 0
    for p, o in zip(reqs, outs):
        assert len(o.token_ids) == 24 and o.stop_reason == "max_tokens"
        ref = plain_logits(cfg, w, list(p) + list(o.token_ids))
        for k, tok in enumerate(o.token_ids):
            row = ref[len(p) + k - 1]
            far += (row.max() - row[tok]).item() > tol * row.abs().max().item()
            total += 1
    # (bfloat16: a row whose router scores nearly tie goes to another expert than the plain model's)
    assert far <= (0 if dtype == "float32" else 0.04 * total), f"{far} of {total} tokens lie far below the best"


def test_trace_replay_of_a_model_folder(tmp_path):
    """bin/trace_run on a folder: prompts of unequal length in one step, then single tokens
    together, the shorter request ending first; the files hold the wanted rows' logits."""
    cfg = MIXED
    w = random_weights(cfg, seed=23)
    path = _write_model(str(tmp_path / "m"), cfg, w)
    a, b = prompts(cfg, [60, 45], seed=24)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:50], "want": [0, 39, 40, 49]},
                                     {"id": "b", "tokens": b[:42], "want": [41]}], "end": []}]
    for k in range(10):
        entries = [{"id": "a", "tokens": [a[50 + k]], "want": [0]}]
        if k < 3:
            entries.append({"id": "b", "tokens": [b[42 + k]], "want": [0] if k != 1 else []})
        steps.append({"step": k + 1, "entries": entries, "end": ["b"] if k == 2 else []})
    out_dir = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", "float32",
                           "--out", out_dir, "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {k}" for k in range(11)]
    ra, rb = plain_logits(cfg, w, a), plain_logits(cfg, w, b)
    got = torch.from_numpy(np.fromfile(os.path.join(out_dir, "0.f32"), dtype="<f4").reshape(5, -1))
    assert_close(got, torch.stack([ra[0], ra[39], ra[40], ra[49], rb[41]]), "float32", "the prompts' rows")
    for k in range(10):
        want = [ra[50 + k]] + ([rb[42 + k]] if k < 3 and k != 1 else [])
        got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{k + 1}.f32"), dtype="<f4").reshape(len(want), -1))
        assert_close(got, torch.stack(want), "float32", f"step {k + 1}")


def test_command_line_generates_from_a_model_folder(tmp_path):
    cfg = ALONE["latent_ff"]
    w = random_weights(cfg, seed=2)
    path = _write_model(str(tmp_path / "m"), cfg, w)
    prompt = prompts(cfg, [9], seed=3)[0]
    p = subprocess.run([sys.executable, "-m", "strata_inference_b200.cli", "-m", path, "--token-ids",
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
