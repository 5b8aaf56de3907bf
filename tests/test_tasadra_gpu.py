"""The Tasadra decoder in the engine against the plain implementation (tests/plain/tasadra_plain.py): whole prompts,
decoding token by token, prompts in portions, batches of unequal requests, pages and slots used again, the edges of
cells, far tokens, other sizes, generation through the entry point, and trace replay as a user runs it."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT
from plain.tasadra_plain import PlainTasadra
from replay_util import batched, whole, with_tail
from tasadra_util import (CONFIGS, assert_close, attention, config, delta, differential, layer, make_weights, rotation,
                          run_steps, write_folder)

pytestmark = pytest.mark.gpu

_plain, _logits = {}, {}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        out[name] = write_folder(str(tmp_path_factory.mktemp(f"tasadra_{name}")), cfg, make_weights(cfg, 500 + i, sharp=2.0))
    return out


def plain_logits(folder, toks):
    key = (folder, tuple(toks))
    if key not in _logits:
        if folder not in _plain:
            _plain[folder] = PlainTasadra(folder)
        _logits[key] = _plain[folder].forward(toks)
    return _logits[key]


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def engine_for(folder, dtype, max_tokens=1024, **kw):
    import turboquant_cpp_b200 as tq
    return tq.Engine(tq.load_model(folder, dtype), max_tokens=max_tokens, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_whole_prompts_decoding_and_batches_agree_with_plain(folders, name, dtype):
    cfg, folder = CONFIGS[name], folders[name]
    reqs = {"r0": tokens_for(cfg, 150, 1), "r1": tokens_for(cfg, 1, 2), "r2": tokens_for(cfg, 77, 3), "r3": tokens_for(cfg, 200, 4)}
    eng = engine_for(folder, dtype, max_tokens=64 * 12)
    try:
        modes = {}
        steps, ends = [], {}
        for rid, toks in reqs.items():                        # each alone and whole, one after another
            s, e = whole(rid, toks)
            ends.update({k + len(steps): v for k, v in e.items()})
            steps += s
        modes["whole"] = run_steps(eng, steps, ends)
        steps, ends = [], {}
        for rid, toks in reqs.items():                        # the last 80 tokens one by one (cells pass over decoded tokens)
            s, e = with_tail(rid, toks, 80)
            ends.update({k + len(steps): v for k, v in e.items()})
            steps += s
        modes["tail"] = run_steps(eng, steps, ends)
        s, e = batched(reqs, {"r0": 100, "r1": 1, "r2": 64, "r3": 129})     # unequal prompts, then decoded together
        modes["batched"] = run_steps(eng, s, e)
        eng.cache.book.check_invariants()
        assert eng.cache.book.slots.n_held == 0 and all(p.n_held == 0 for p in eng.cache.book.pools)
        for rid, toks in reqs.items():
            for mode, got in modes.items():
                assert sorted(got[rid]) == list(range(len(toks))), f"{mode} {rid}"
                assert_close(got[rid], plain_logits(folder, toks), dtype, f"{name} {mode} {rid}")
    finally:
        eng.release()


@pytest.mark.parametrize("name,sizes", [("a", (2, 3, 50, 2, 64, 9)), ("b", (70, 2, 58, 2, 65)), ("c", (17, 2, 2, 2, 40))])
def test_prompts_in_portions(folders, name, sizes):
    """A prompt cut into portions, down to two tokens, beside a request that goes on token by token: the shift's kept
    row, the convolution's kept inputs and the recurrence's state pass from portion to portion; cells are counted
    from the sequence's start, not from a portion's."""
    cfg, folder = CONFIGS[name], folders[name]
    toks, other = tokens_for(cfg, sum(sizes), 7), tokens_for(cfg, len(sizes) + 20, 8)
    for dtype in ("float32", "bfloat16"):
        eng = engine_for(folder, dtype)
        try:
            steps, at = [], 0
            for i, n in enumerate(sizes):
                step = [("p", toks[at:at + n], list(range(n)))]
                if i == 0:
                    step.append(("o", other[:21], list(range(21))))
                else:
                    step.append(("o", [other[20 + i]], [0]))
                steps.append(step)
                at += n
            got = run_steps(eng, steps, {len(steps) - 1: ["p", "o"]})
            assert_close(got["p"], plain_logits(folder, toks), dtype, f"{name} portions")
            assert_close(got["o"], plain_logits(folder, other), dtype, f"{name} beside portions")
        finally:
            eng.release()


def test_slots_and_pages_used_again_carry_nothing_over(folders):
    """A request run after others have ended gets their slot and pages; its logits are those of a fresh engine."""
    cfg, folder = CONFIGS["a"], folders["a"]
    eng = engine_for(folder, "float32", max_tokens=64 * 4, max_slots=2)
    try:
        a, b, c = tokens_for(cfg, 130, 11), tokens_for(cfg, 90, 12), tokens_for(cfg, 140, 13)
        s1, e1 = batched({"a": a, "b": b}, {"a": 100, "b": 80})
        run_steps(eng, s1, e1)
        s2, e2 = with_tail("c", c, 30)
        got = run_steps(eng, s2, e2)
        assert_close(got["c"], plain_logits(folder, c), "float32", "after reuse")
        eng.cache.book.check_invariants()
    finally:
        eng.release()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """300 tokens decoded one by one from a 3-token prompt: states and cells over many steps, graphs replayed."""
    cfg, folder = CONFIGS["b"], folders["b"]
    toks = tokens_for(cfg, 303, 21)
    eng = engine_for(folder, dtype)
    try:
        s, e = with_tail("x", toks, 300)
        got = run_steps(eng, s, e)
        assert eng.graphs is not None and eng.graphs.replays >= 290
        assert_close(got["x"], plain_logits(folder, toks), dtype, "long decoding")
    finally:
        eng.release()


VARIANTS = {
    # everything one: one head, one element a key, values of two, one tap, cells of one position
    "ones": [layer("attention", attention(heads=1, kv_heads=1, dim=2, vdim=2, rot=rotation(2, 10.0), softcap=0)),
             layer("channel_delta", delta(heads=1, kv_heads=1, dim=1, vdim=1, conv=1)),
             layer("attention_2", differential(heads=1, kv_heads=1, dim=1, vdim=1, size=1), ff=1)],
    # no rotation at all; no feed-forward anywhere
    "no_rotation": [layer("attention", attention(rot=None)), layer("attention_2", differential(size=0))],
    # whole heads rotated, frequencies stretched; nine heads on three
    "full_rotation": [layer("attention", attention(heads=9, kv_heads=3, dim=12, vdim=4, rot=rotation(12, 50.0, (16.0, 16, 4.0, 0.5))), ff=20)],
    # cells of exactly a page and of two pages; a reader with narrower cells than its source
    "page_cells": [layer("attention_2", differential(size=128), ff=16), layer("attention_2", differential(size=64, kv_from=0))],
    # sizes of the tensor-core kernels with sixteen query rows a key head, cells that are no multiple of anything
    "wide_groups": [layer("attention_2", differential(heads=8, kv_heads=1, dim=32, vdim=128, scale=0.2, size=37), ff=16),
                    layer("attention", attention(heads=16, kv_heads=1, dim=128, vdim=64, scale=0.1, rot=rotation(64, 1e4)))],
    # keys of 256 elements in the recurrence, values that no block of sixteen columns divides
    "wide_state": [layer("channel_delta", delta(heads=2, kv_heads=1, dim=256, vdim=21, conv=5), ff=16)],
    # odd sizes everywhere: width, heads, keys, feed-forward
    "odd_width": [layer("attention", attention(heads=3, kv_heads=1, dim=10, vdim=6, rot=rotation(6, 77.0, (3.0, 20, 5.0, 1.5))), ff=11),
                  layer("channel_delta", delta(heads=3, kv_heads=1, dim=5, vdim=9, conv=6), ff=13),
                  layer("attention_2", differential(heads=5, kv_heads=5, dim=3, vdim=7, size=33), ff=7),
                  layer("attention_2", differential(heads=5, kv_heads=5, dim=3, vdim=7, size=33, kv_from=2, diff=0.6, scale=1.1))],
}


WIDTHS = {"odd_width": 37}       # a stream no 16-byte access divides


@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_other_sizes_and_options(tmp_path, variant):
    cfg = config(VARIANTS[variant], vocab=50, width=WIDTHS.get(variant, 36), mult=1.3)
    folder = write_folder(str(tmp_path / variant), cfg, make_weights(cfg, 5, sharp=2.0, decay_rank=1, gate_rank=3))
    toks = tokens_for(cfg, 200, 31)
    for dtype in ("float32", "bfloat16"):
        eng = engine_for(folder, dtype)
        try:
            s, e = with_tail("x", toks, 40)
            got = run_steps(eng, s, e)
            assert_close(got["x"], plain_logits(folder, toks), dtype, variant)
        finally:
            eng.release()


def test_a_wrong_cell_edge_a_lost_state_or_a_wrong_constant_would_show(folders, tmp_path):
    """The tests above mean something only if the plain model itself reacts to these faults: with the weights used
    here, moving a cell's edge by one token, forgetting the token before a portion, the recurrence's state, the
    values' rotation or the depth weights moves the logits by far more than the tolerance."""
    from plain import tasadra_plain as P
    cfg, folder = CONFIGS["a"], folders["a"]
    toks = tokens_for(cfg, 60, 1)
    ref = plain_logits(folder, toks)
    weights = make_weights(cfg, 500, sharp=2.0)
    spread = ref.std()
    wrong = copy.deepcopy(cfg)
    wrong["layers"][3]["mixer"]["mask"]["size"] += 1
    f2 = write_folder(str(tmp_path / "cell"), wrong, weights)
    assert np.abs(PlainTasadra(f2).forward(toks) - ref)[26:].max() > 1e-2 * spread
    # the token before a portion's first token and the states: a portion run alone differs from the portion in place
    assert np.abs(PlainTasadra(folder).forward(toks[30:])[0] - ref[30]).max() > 1e-2 * spread
    w2 = dict(weights)
    for k in list(w2):
        if k.endswith("dwa"):
            w2[k] = np.zeros_like(w2[k])
            w2[k][-1] = 1.0
    f3 = write_folder(str(tmp_path / "depth"), cfg, w2)
    assert np.abs(PlainTasadra(f3).forward(toks) - ref).max() > 1e-2 * spread
    wrong = copy.deepcopy(cfg)
    wrong["layers"][0]["mixer"]["rot"]["base"] *= 1.5        # moves the values' angles too
    f4 = write_folder(str(tmp_path / "base"), wrong, weights)
    assert np.abs(PlainTasadra(f4).forward(toks) - ref)[5:].max() > 1e-2 * spread


def test_a_far_token_reaches_through_attention_and_through_the_state(tmp_path):
    """Hundreds of tokens back: the plain logits at the end change when the first token changes, and the engine follows
    that change through pages (attention) and through the recurrence's state, in prompts and in decoding."""
    for kind, mixer in (("attention", attention(heads=2, kv_heads=1, dim=16, vdim=16, softcap=0, scale=1.0)),
                        ("channel_delta", delta(heads=2, kv_heads=2, dim=16, vdim=8, conv=2))):
        cfg = config([layer(kind, mixer, ff=16)], vocab=40, width=32, mult=1.0)
        w = make_weights(cfg, 9, sharp=1.0)
        if kind == "channel_delta":
            w["l0.mix.dt_bias"] = np.full_like(w["l0.mix.dt_bias"], -9.0)        # decays near one: the state forgets slowly
            w["l0.mix.a2"] = w["l0.mix.a2"] * 0.05
        else:
            w["l0.mix.q"] = w["l0.mix.q"] * 0.05                                  # flat weights: every far token counts
        w["l0.shift"] = np.zeros_like(w["l0.shift"])
        folder = write_folder(str(tmp_path / kind), cfg, w)
        a = tokens_for(cfg, 400, 3)
        b = [(a[0] + 7) % cfg["vocab"]] + a[1:]
        ra, rb = plain_logits(folder, a), plain_logits(folder, b)
        moved = np.abs(ra[-1] - rb[-1]).max() / ra.std()
        assert moved > 2e-4, f"{kind}: the first token does not reach the last position ({moved:.1e})"
        eng = engine_for(folder, "float32")
        try:
            for toks, ref in ((a, ra), (b, rb)):
                for sched in (whole("x", toks, keep={399}), with_tail("x", toks, 90, keep={0})):
                    got = run_steps(eng, *sched)
                    e = np.abs(got["x"][399] - ref[399]).max() / ra.std()
                    assert e < moved / 20, f"{kind}: the last position is off by {e:.1e}, the far token moves it by {moved:.1e}"
        finally:
            eng.release()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folders, dtype):
    import turboquant_cpp_b200 as tq
    cfg, folder = CONFIGS["a"], folders["a"]
    prompts = [tokens_for(cfg, n, 40 + n) for n in (1, 9, 40, 70)]
    n_new = 12
    with tq.Model(folder, temperature=0.0, max_tokens=n_new, dtype=dtype, max_batch=4, context_length=128) as m:
        outs = m.generate_batch(prompts)
        assert m.generate_batch(prompts[::-1])[::-1] == outs          # another order in the batch, slots used again
        assert [m.ask(p) for p in prompts] == outs                    # each alone
        m.engine.cache.book.check_invariants()
        assert m.engine.cache.book.slots.n_held == 0
    plain = PlainTasadra(folder)
    floor = 1e-4 if dtype == "float32" else 0.15
    for p, o in zip(prompts, outs):
        toks = list(p)
        for i, t in enumerate(o):
            l = plain.forward(toks)[-1]
            top = np.sort(l)[-2:]
            if int(np.argmax(l)) != t:
                assert top[1] - top[0] < floor * l.std(), f"token {i}: engine {t}, plain {int(np.argmax(l))}"
            toks.append(t)


def test_command_line_and_trace_replay(folders, tmp_path):
    """The generation program on a folder, and the replay program as a user runs it: steps on standard input, logits
    in files, a line per step."""
    cfg, folder = CONFIGS["c"], folders["c"]
    toks = tokens_for(cfg, 40, 77)
    env = dict(os.environ, PYTHONPATH=ROOT)
    import turboquant_cpp_b200 as tq
    quant = [sys.executable, os.path.join(ROOT, "bin", "quant")]
    common = ["-p", " ".join(map(str, toks[:9])), "-n", "5", "-T", "0", "--dtype", "float32"]
    out = subprocess.run(quant + [folder] + common, capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    with tq.Model(folder, temperature=0.0, max_tokens=5, dtype="float32") as m:
        assert [int(t) for t in out.stdout.split()] == m.ask(toks[:9])
    info = subprocess.run(quant + [folder, "--info"], capture_output=True, text=True, env=env, timeout=600)
    assert info.returncode == 0 and "Tasadra" in info.stdout
    # weights drawn at random need the inner sizes of the delta rule's low-rank pairs, which a file gives by its tensors
    given = copy.deepcopy(cfg)
    for l in given["layers"]:
        if l["type"] == "channel_delta":
            l["mixer"].update(decay_rank=3, gate_rank=5)
    json.dump(given, open(tmp_path / "cfg.json", "w"))
    runs = [subprocess.run(quant + ["--random", str(tmp_path / "cfg.json"), "--seed-weights", str(seed)] + common + ["--profile"],
                           capture_output=True, text=True, env=env, timeout=600) for seed in (3, 4)]
    assert all(x.returncode == 0 for x in runs), runs[0].stderr[-2000:] + runs[1].stderr[-2000:]
    assert any(l.startswith("[Profile ") and "matmul=" in l for l in runs[0].stderr.splitlines())
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[32:], "want": [7]}], "end": ["x"]}]
    res = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(tmp_path / "o"),
                          "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(tmp_path / "o" / "1.f32")
    ref = plain_logits(folder, toks)
    got0 = np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(2, cfg["vocab"])
    got2 = np.fromfile(tmp_path / "o" / "2.f32", dtype="<f4").reshape(1, cfg["vocab"])
    assert_close({0: got0[0], 29: got0[1], 39: got2[0]}, ref, "float32", "trace replay")
