"""The Sisepel decoder in the engine against the plain implementation (tests/plain/sisepel_plain.py): whole prompts,
decoding token by token, prompts in portions, batches of unequal requests, pages and slots used again, the edges of
windows, far tokens kept by the retention state, other sizes, generation through the entry point, and trace replay
as a user runs it."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT
from plain.sisepel_plain import PlainSisepel
from replay_util import batched, whole, with_tail
from sisepel_util import (CONFIGS, assert_close, check_against_plain, config, dense, layer, left, make_weights, moe, right,
                          rotation, run_steps, run_steps_with_routing, write_folder)

pytestmark = pytest.mark.gpu

_plain = {}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        out[name] = write_folder(str(tmp_path_factory.mktemp(f"sisepel_{name}")), cfg, make_weights(cfg, 300 + i))
    return out


def plain_model(folder):
    if folder not in _plain:
        _plain[folder] = PlainSisepel(folder)
    return _plain[folder]


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def engine_for(folder, dtype, max_tokens=1024, **kw):
    import turboquant_cpp_b200 as tq
    return tq.Engine(tq.load_model(folder, dtype), max_tokens=max_tokens, record_routing=True, **kw)


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
        modes["whole"] = run_steps_with_routing(eng, steps, ends)
        steps, ends = [], {}
        for rid, toks in reqs.items():                        # the last 80 tokens one by one (windows pass over decoded tokens)
            s, e = with_tail(rid, toks, 80)
            ends.update({k + len(steps): v for k, v in e.items()})
            steps += s
        modes["tail"] = run_steps_with_routing(eng, steps, ends)
        s, e = batched(reqs, {"r0": 100, "r1": 1, "r2": 64, "r3": 129})     # unequal prompts, then decoded together
        modes["batched"] = run_steps_with_routing(eng, s, e)
        eng.cache.book.check_invariants()
        assert eng.cache.book.slots.n_held == 0 and all(p.n_held == 0 for p in eng.cache.book.pools)
        for rid, toks in reqs.items():
            for mode, (got, routing) in modes.items():
                assert sorted(got[rid]) == list(range(len(toks))), f"{mode} {rid}"
                check_against_plain(plain_model(folder), toks, got[rid], routing[rid], dtype, f"{name} {mode} {rid}")
    finally:
        eng.release()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,sizes", [("a", [2, 3, 64, 1, 2, 7, 50, 17]), ("b", [63, 2, 2, 65, 5, 40, 16]), ("c", [5, 128, 2, 30])])
def test_prompts_in_portions(folders, name, sizes, dtype):
    """A prompt cut into portions, down to two tokens, beside a request that goes on token by token: the retention
    state and the windows carry over every cut."""
    cfg, folder = CONFIGS[name], folders[name]
    toks, other = tokens_for(cfg, sum(sizes), 7), tokens_for(cfg, len(sizes) + 20, 8)
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
        got, routing = run_steps_with_routing(eng, steps, {len(steps) - 1: ["p", "o"]})
        check_against_plain(plain_model(folder), toks, got["p"], routing["p"], dtype, f"{name} portions")
        check_against_plain(plain_model(folder), other, got["o"], routing["o"], dtype, f"{name} beside portions")
    finally:
        eng.release()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,sizes", [("a", [700]), ("b", [333, 130, 237]), ("c", [129, 571])])
def test_long_prompts_whose_recurrence_runs_in_chunks(folders, name, sizes, dtype, monkeypatch):
    """Runs long enough for the retention mixer to cut them into chunks that it scans side by side (whole, and in
    portions that go on from a kept state), beside a short request.  float32: against the plain model.  bfloat16:
    against the same engine with the cutting switched off, position by position (among 700 positions some enlarge a
    rounding beyond any bound that would still tell a fault; both paths round alike, so they stay together)."""
    from turboquant_cpp_b200.parts.retention import RetentionMixer
    cfg, folder = CONFIGS[name], folders[name]
    toks, other = tokens_for(cfg, sum(sizes), 21), tokens_for(cfg, len(sizes) + 40, 22)
    steps, at = [], 0
    for i, n in enumerate(sizes):
        step = [("p", toks[at:at + n], list(range(n)))]
        step.append(("o", other[:41], list(range(41))) if i == 0 else ("o", [other[40 + i]], [0]))
        steps.append(step)
        at += n

    def run():
        eng = engine_for(folder, dtype, max_tokens=1024)
        try:
            return run_steps_with_routing(eng, steps, {len(steps) - 1: ["p", "o"]})
        finally:
            eng.release()

    cut = []
    plan = RetentionMixer._chunks
    monkeypatch.setattr(RetentionMixer, "_chunks", lambda self, ctx: cut.append(plan(self, ctx)) or cut[-1])
    got, routing = run()
    assert any(c is not None for c in cut)                    # the runs were cut
    if dtype == "float32":
        check_against_plain(plain_model(folder), toks, got["p"], routing["p"], dtype, f"{name} long prompt")
        check_against_plain(plain_model(folder), other, got["o"], routing["o"], dtype, f"{name} beside a long prompt")
        return
    monkeypatch.setattr(RetentionMixer, "_chunks", lambda self, ctx: None)
    whole, _ = run()
    for rid in ("p", "o"):
        ref = np.stack([whole[rid][p] for p in sorted(whole[rid])])
        rows = np.stack([got[rid][p] for p in sorted(whole[rid])])
        d = rows - ref
        e = np.sqrt((d * d).mean(axis=1)) / ref.std()
        assert e.max() < 2e-2, f"{name} {rid}: position {int(e.argmax())} differs by {e.max():.3e} between the cut and the whole recurrence"


def test_slots_and_pages_used_again_carry_nothing_over(folders):
    """A request run after others have ended gets their slot (its retention state) and pages; its logits are those of
    a fresh engine."""
    cfg, folder = CONFIGS["a"], folders["a"]
    eng = engine_for(folder, "float32", max_tokens=64 * 4, max_slots=2)
    try:
        a, b, c = tokens_for(cfg, 130, 11), tokens_for(cfg, 90, 12), tokens_for(cfg, 140, 13)
        s1, e1 = batched({"a": a, "b": b}, {"a": 100, "b": 80})
        run_steps(eng, s1, e1)
        s2, e2 = with_tail("c", c, 30)
        got, routing = run_steps_with_routing(eng, s2, e2)
        check_against_plain(plain_model(folder), c, got["c"], routing["c"], "float32", "after reuse")
        eng.cache.book.check_invariants()
    finally:
        eng.release()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_gives_pages_back(folders, dtype):
    """300 tokens decoded one by one from a 3-token prompt: windows pass over decoded tokens, pages that fell out of
    every window are given back, the state is carried through every step; graphs are replayed."""
    cfg, folder = CONFIGS["b"], folders["b"]
    toks = tokens_for(cfg, 303, 21)
    eng = engine_for(folder, dtype)
    try:
        s, e = with_tail("x", toks, 300)
        got, routing = run_steps_with_routing(eng, s[:-1], {}, leave_open=True)
        live = list(eng.cache.book.live.values())
        assert len(live) == 1 and live[0].length == 302
        gaps = 0
        for g, need in enumerate(eng.cache.groups):
            held = [p is not None for p in live[0].pages[g]]
            gone = (302 + 1 - need.window) // 64 if need.window else 0
            assert held == [i >= gone for i in range(len(held))], (need, held)
            gaps += gone > 0
        assert gaps >= 2                                      # the test's model has windows that did move on
        eng.close(live[0])
        assert eng.graphs is not None and eng.graphs.replays >= 280
        check_against_plain(plain_model(folder), toks[:-1], got["x"], routing["x"], dtype, "long decoding")
    finally:
        eng.release()


ONE = dict(heads=1, kv_heads=1, dim=8, vdim=8, size=5, rot=None)       # a small left branch beside the mechanism under test
VARIANTS = {
    # one mechanism a model (the other branch, which a layer cannot be without, is as small as it gets)
    "left_alone": config([layer(left(), right(heads=1, dim=2, vdim=2, decay=(0.5,), rot=None))], side=0, logit_scale=None),
    "right_alone": config([layer(left(**ONE), right())], side=0, logit_scale=None),
    "dense_alone": config([layer(left(**ONE), right(heads=1, dim=2, vdim=2, decay=(0.5,), rot=None), dense(ff=40))], side=0, logit_scale=None),
    "experts_alone": config([layer(left(**ONE), right(heads=1, dim=2, vdim=2, decay=(0.5,), rot=None), moe(experts=12, top=4, ff=8, shared=12))], side=0, logit_scale=None),
    "token_input_alone": config([layer(left(**ONE), right(heads=1, dim=2, vdim=2, decay=(0.5,), rot=None))], side=5, logit_scale=None),
    # sizes and options
    "window_of_one": config([layer(left(size=1), right())]),
    "no_cap_no_rotation": config([layer(left(softcap=0, rot=None), right(rot=None))]),
    "wide_heads": config([layer(left(heads=2, kv_heads=1, dim=8, vdim=136, size=20), right(heads=2, dim=200, vdim=3, decay=(0.9, 0.99), rot=rotation(200, 1e4))),
                          layer(left(heads=4, kv_heads=1, dim=200, vdim=136, size=7, scale=0.05, rot=rotation(200, 777.0, (3.0, 2.0, 6.0, 30))), right(heads=1, dim=100, vdim=100, decay=(0.95,), rot=rotation(50, 60.0)))]),
    "odd_sizes": config([layer(left(heads=5, kv_heads=5, dim=7, vdim=3, size=13, rot=rotation(6, 20.0)), right(heads=3, dim=5, vdim=7, decay=(0.7, 0.8, 0.9), rot=rotation(4, 9.0)), dense(ff=5)),
                         layer(left(heads=3, kv_heads=1, dim=10, vdim=9, size=33, rot=rotation(2, 3.0)), right(heads=1, dim=33, vdim=2, decay=(0.999,), rot=rotation(32, 1e3)), moe(experts=5, top=2, ff=3, shared=7))],
                        vocab=50, width=36, side=3),
    # the same oddities with feed-forwards a few elements wider, for bfloat16 as well (a norm on the output of a
    # feed-forward three or five elements wide enlarges the rounding before it whenever those few elements are small together)
    "odd_sizes_wider": config([layer(left(heads=5, kv_heads=5, dim=7, vdim=5, size=13, rot=rotation(6, 20.0)), right(heads=3, dim=5, vdim=7, decay=(0.7, 0.8, 0.9), rot=rotation(4, 9.0)), dense(ff=21)),
                               layer(left(heads=3, kv_heads=1, dim=10, vdim=9, size=33, rot=rotation(2, 3.0)), right(heads=1, dim=33, vdim=6, decay=(0.999,), rot=rotation(32, 1e3)), moe(experts=5, top=2, ff=11, shared=13))],
                              vocab=50, width=36, side=3),
    # everything that can be one is one (a unit norm over one element, and a token input one wide, are sign functions: in float32 only, where a rounding
    # does not flip it)
    "ones": config([layer(left(heads=1, kv_heads=1, dim=2, vdim=1, size=2, rot=rotation(2, 3.0)), right(heads=1, dim=1, vdim=1, decay=(0.9,), rot=None),
                          moe(experts=1, top=1, ff=1, shared=1))], vocab=50, width=36, side=1),
    "many_experts": config([layer(left(), right(), moe(experts=72, top=6, ff=8, shared=0))]),
    "sixteen_heads_a_group": config([layer(left(heads=16, kv_heads=1, dim=32, vdim=32, scale=0.25, size=100, rot=rotation(16, 99.0)), right(heads=8, dim=16, vdim=16, decay=[0.9 + 0.01 * i for i in range(8)], rot=rotation(16, 1e4)))],
                                    width=64),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_other_sizes_and_options(tmp_path, variant, dtype):
    if variant == "ones" and dtype != "float32":
        pytest.skip("a sign function of rounded numbers")
    if variant == "odd_sizes" and dtype != "float32":
        pytest.skip("norms over three to five rounded numbers: odd_sizes_wider runs in bfloat16")
    cfg = copy.deepcopy(VARIANTS[variant])
    folder = write_folder(str(tmp_path / variant), cfg, make_weights(cfg, 5))
    toks = tokens_for(cfg, 110, 31)
    eng = engine_for(folder, dtype)
    try:
        s, e = with_tail("x", toks, 25)
        got, routing = run_steps_with_routing(eng, s, e)
        check_against_plain(plain_model(folder), toks, got["x"], routing["x"], dtype, variant)
    finally:
        eng.release()


def test_a_wrong_edge_a_missing_sink_or_a_wrong_constant_would_show(folders, tmp_path):
    """The tests above mean something only if the plain model itself reacts to these faults: with the weights used
    here, a window's edge moved by one token, a sink or a cap left out, another pairing's frequencies, a decay or the
    router's bias changed move the logits by far more than the tolerance."""
    cfg, folder = CONFIGS["a"], folders["a"]
    toks = tokens_for(cfg, 160, 1)
    ref = plain_model(folder).forward(toks)
    weights = make_weights(cfg, 300)
    spread = ref.std()

    def changed(change, new_weights=None):
        wrong = copy.deepcopy(cfg)
        change(wrong)
        f = write_folder(str(tmp_path / f"v{len(os.listdir(tmp_path))}"), wrong, new_weights or weights)
        return np.abs(PlainSisepel(f).forward(toks) - ref).max()

    assert changed(lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=25)) > 1e-2 * spread
    assert changed(lambda c: c["layers"][1]["mixer"]["left"]["mask"].update(size=8)) > 1e-2 * spread
    assert changed(lambda c: c["layers"][0]["mixer"]["left"].update(softcap=0)) > 1e-3 * spread
    assert changed(lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(factor=1.0)) > 1e-3 * spread
    assert changed(lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.9, 0.97, 0.99])) > 1e-3 * spread
    assert changed(lambda c: c["layers"][1]["mixer"]["right"]["rot"].update(dims=4)) > 1e-3 * spread
    assert changed(lambda c: None, dict(weights, **{"l0.mix.left.sink": weights["l0.mix.left.sink"] - 30.0})) > 1e-2 * spread
    assert changed(lambda c: None, dict(weights, **{"l0.mlp.router.b": np.zeros_like(weights["l0.mlp.router.b"])})) > 1e-2 * spread
    assert changed(lambda c: c.update(logit_scale=1.0)) > 1e-2 * spread
    # every layer reads its own columns of the second table
    assert changed(lambda c: None, dict(weights, **{"side.embed": np.roll(weights["side.embed"], 6, axis=1)})) > 1e-2 * spread


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_at_a_windows_edge_and_far_tokens_in_the_state(tmp_path, dtype):
    """One key carries almost all the weight of the query that matches it: it must count at distance size - 1 and not
    at distance size, in a prompt, across a page border and for decoded tokens.  And a token hundreds of positions
    back still speaks through a retention head that forgets nothing."""
    size, W = 70, 32
    cfg = config([layer(left(heads=2, kv_heads=1, dim=32, vdim=32, scale=2.0, size=size, softcap=50.0, rot=None),
                        right(heads=2, dim=8, vdim=8, decay=(1.0, 0.5), rot=None))], vocab=40, width=W, side=0)
    w = make_weights(cfg, 9)
    # token 1 is the marked key's token, token 2 the asking token: the asking token's embedding is the marked one's
    # read backwards, and the key projections are the query projections with their columns read backwards, so that
    # q(2) = k(1) (as large a score as unit vectors allow) while the two tokens' own keys and values differ
    w["l0.norm1"][:] = 1.0
    w["embed"][2] = w["embed"][1][::-1]
    w["l0.mix.left.k"][:] = w["l0.mix.left.q"][:32][:, ::-1]
    a = w["embed"][1] / np.sqrt((w["embed"][1] ** 2).mean()) / np.sqrt(W)
    u = np.random.default_rng(0).standard_normal(16)
    w["l0.mix.right.k"][:] = np.outer(u, a)               # the retention keys look along the marked token's direction only
    w["l0.mix.right.q"][:] = np.outer(u, a[::-1])
    base = np.random.default_rng(3).integers(3, 40, size=400).tolist()
    folder = write_folder(str(tmp_path / "edge"), cfg, w)
    plain = PlainSisepel(folder)
    eng = engine_for(folder, dtype)
    try:
        for key_at, ask_at, tail, lo, hi in ((100, 100 + size - 1, 10, 0.3, 9.0), (100, 100 + size, 10, 0.0, 0.05),
                                             (60, 60 + size - 1, 200, 0.3, 9.0), (60, 60 + size, 200, 0.0, 0.05),
                                             (5, 399, 10, 2e-3, 0.05)):
            toks = list(base)
            toks[key_at], toks[ask_at] = 1, 2
            ref = plain.forward(toks)
            moved = list(toks)
            moved[key_at] = 5
            # what the marked token means to the asking position: a lot inside the window, little outside it (only
            # what the state carries), and from afar still more than the comparison in float32 lets pass
            effect = np.abs(plain.forward(moved)[ask_at] - ref[ask_at]).max() / ref.std()
            assert lo <= effect <= hi, (key_at, ask_at, effect)
            s, e = with_tail("x", toks, tail)
            got = run_steps(eng, s, e)
            assert_close(got["x"], ref, dtype, f"key at {key_at}, asked at {ask_at}")
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
    plain = plain_model(folder)
    floor = 1e-4 if dtype == "float32" else 0.15
    for p, o in zip(prompts, outs):
        toks = list(p)
        for i, t in enumerate(o):
            l = plain.forward(toks)[-1]
            top = np.sort(l)[-2:]
            if int(np.argmax(l)) != t:
                assert top[1] - top[0] < floor * l.std(), f"token {i}: engine {t}, plain {int(np.argmax(l))}"
                break                                                   # after a near-tie the texts part ways
            toks.append(t)


def test_command_line_on_a_folder_and_on_random_weights(folders, tmp_path):
    """bin/quant on a folder of the design gives the entry point's greedy tokens; --info names the design; --random
    CONFIG --seed-weights N builds and runs a model of the configuration, another seed another model; --profile
    prints its buckets."""
    import turboquant_cpp_b200 as tq
    cfg, folder = CONFIGS["a"], folders["a"]
    prompts = [tokens_for(cfg, n, 60 + n) for n in (3, 21)]
    quant = [sys.executable, os.path.join(ROOT, "bin", "quant")]
    common = ["-n", "7", "-T", "0", "--dtype", "float32"]
    tok_file, cfg_file = str(tmp_path / "prompts.txt"), str(tmp_path / "cfg.json")
    open(tok_file, "w").write("\n".join(" ".join(map(str, q)) for q in prompts) + "\n")
    json.dump(cfg, open(cfg_file, "w"))
    r = subprocess.run(quant + [folder] + common + ["--tokens-file", tok_file], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    with tq.Model(folder, temperature=0.0, max_tokens=7, dtype="float32") as m:
        want = m.generate_batch(prompts)
    assert [[int(t) for t in l.split()] for l in r.stdout.strip().splitlines()] == want
    info = subprocess.run(quant + [folder, "--info"], capture_output=True, text=True, timeout=600)
    assert info.returncode == 0 and "Sisepel" in info.stdout
    runs = [subprocess.run(quant + ["--random", cfg_file, "--seed-weights", str(seed)] + common + ["--tokens-file", tok_file, "--profile"],
                           capture_output=True, text=True, timeout=600) for seed in (3, 4)]
    assert all(x.returncode == 0 for x in runs), runs[0].stderr + runs[1].stderr
    assert len(runs[0].stdout.strip().splitlines()) == 2 and runs[0].stdout != runs[1].stdout
    assert any(l.startswith("[Profile ") and "matmul=" in l for l in runs[0].stderr.splitlines())


def test_trace_replay_as_a_user_runs_it(folders, tmp_path):
    cfg, folder = CONFIGS["c"], folders["c"]
    reqs = {"a": tokens_for(cfg, 45, 50), "b": tokens_for(cfg, 140, 51), "c": tokens_for(cfg, 1, 52)}
    s, e = batched(reqs, {"a": 13, "b": 100, "c": 1})
    lines = [json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in step], "end": e.get(i, [])})
             for i, step in enumerate(s)]
    out_dir = str(tmp_path / "out")
    need = sum(len(t) for t in reqs.values())                 # padding not counted
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out_dir, "--max-tokens", str(need)], input="\n".join(lines) + "\n", capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(s))]
    got, pos = {}, {}
    for i, step in enumerate(s):
        a = np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        row = 0
        for rid, toks, want in step:
            for w in want:
                got.setdefault(rid, {})[pos.get(rid, 0) + w] = a[row]
                row += 1
            pos[rid] = pos.get(rid, 0) + len(toks)
    for rid, toks in reqs.items():
        assert_close(got[rid], plain_model(folder).forward(toks), "float32", f"replay {rid}")
