"""The kernels behind the Sisepel parts, each alone against the plain functions (tests/plain/sisepel_plain.py): the
cache write with rotation and unit norm, the attention kernels with a cap on the scores and a learned sink (a marked
key just inside and just outside the window, in a prompt and for single tokens, over scattered pages), the retention
recurrence with its state carried over portions in slots that held other values, the unit norm with the gate behind
it, the mean of two normed branches, the gated slice of a token table, the router's bias and the scaled logits."""
import math
import os

import numpy as np
import pytest
import torch

from plain import sisepel_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV).contiguous()


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device=DEV)


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rel(got, want):
    return np.abs(host(got) - want).max() / max(1e-30, np.abs(want).max())


def frequencies(rot):
    return None if not rot or not rot["dims"] else dev(P.frequencies(rot))


def scattered_cache(T, G, dr, dtype, rng, extra_pages=3):
    """More pages than the sequence needs, a large value where nothing is written, pages visited in a shuffled order."""
    n = -(-T // 64)
    cache = torch.full((n + extra_pages, 1, G, 64, dr), 1e30, dtype=dtype, device=DEV)
    table = torch.tensor(rng.permutation(n + extra_pages)[:n].reshape(1, n), dtype=torch.int32, device=DEV)
    return cache, table


SCALING = {"factor": 5.0, "low": 1.0, "high": 3.0, "original": 40}
ATT_CASES = [
    # T, H, G, dk, dv, window, cap, scale, rot
    (200, 4, 2, 32, 64, 70, 9.0, 0.6, {"dims": 16, "base": 300.0, "scaling": SCALING}),   # the tensor-core kernel's sizes
    (150, 3, 3, 128, 128, 0, 0.0, 0.1, {"dims": 128, "base": 1e4}),                        # no window, no cap, every element turns
    (131, 6, 2, 24, 40, 33, 4.0, 0.7, {"dims": 6, "base": 20.0}),                          # sizes only the token kernel takes
    (260, 2, 2, 32, 32, 1, 30.0, 0.5, None),                                               # a window of one: only itself and the sink
    (190, 16, 2, 64, 64, 64, 12.0, 0.3, {"dims": 2, "base": 7.0, "scaling": SCALING}),     # a window of exactly a page
    (140, 24, 2, 64, 80, 65, 15.0, 0.4, {"dims": 32, "base": 1e5}),                        # a value longer than the key
]


@pytest.mark.parametrize("case", ATT_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotating_cache_write_and_capped_attention_with_a_sink(case, dtype):
    from turboquant_cpp_b200.kernels import bias_attention as KB
    T, H, G, dk, dv, window, cap, scale, rot = case
    rng = np.random.default_rng(T + H)
    eps = 2e-4
    m = {"scale": scale, "softcap": cap, "rot": rot}
    if window:
        m["mask"] = {"size": window}
    extra = 11                                                # the rows hold more than [q | k | v]
    qkv = rng.standard_normal((T, H * dk + G * (dk + dv) + extra)) * 1.5
    q = qkv[:, :H * dk].reshape(T, H, dk).copy()
    k = qkv[:, H * dk:H * dk + G * dk].reshape(T, G, dk).copy()
    v = qkv[:, H * dk + G * dk:H * dk + G * (dk + dv)].reshape(T, G, dv).copy()
    # a marked key per edge: the query asks for it exactly (up to the turn), and its value is ten times the others'
    asks = []
    if window > 1:
        for key_at, ask_at in ((20, 20 + window - 1), (40, 40 + window), (64, 64 + window - 1), (62, 62 + window)):
            if ask_at < T:
                q[ask_at] = np.repeat(k[key_at], H // G, axis=0) * 3.0
                v[key_at] *= 10.0
                asks.append(ask_at)
    qkv[:, :H * dk], qkv[:, H * dk:H * dk + G * dk] = q.reshape(T, -1), k.reshape(T, -1)
    qkv[:, H * dk + G * dk:H * dk + G * (dk + dv)] = v.reshape(T, -1)
    qkv = host(dev(qkv))                                     # what the kernels see: float32 roundings
    q, k = qkv[:, :H * dk].reshape(T, H, dk), qkv[:, H * dk:H * dk + G * dk].reshape(T, G, dk)
    v = qkv[:, H * dk + G * dk:H * dk + G * (dk + dv)].reshape(T, G, dv)
    sink = rng.standard_normal(H) + 1.0
    want = P.attention_core(q, k, v, m, sink, eps).reshape(T, H * dv)
    if asks:                                                  # the plain function itself sees the marked keys come and go
        moved = dict(m, mask={"size": window + 1})
        diff = np.abs(P.attention_core(q, k, v, moved, sink, eps).reshape(T, H * dv) - want).max(axis=1)
        assert diff[asks[1]] > 0.1 and diff[asks[0]] < diff[asks[1]]

    cache, table = scattered_cache(T, G, dk + dv, dtype, rng)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    seq_of_token = torch.zeros(T, dtype=torch.int32, device=DEV)
    q_dev = torch.empty((T, H, dk), dtype=dtype, device=DEV)
    KB.kv_write_rot(dev(qkv), q_dev, cache, frequencies(rot), rot["dims"] if rot else 0, False, eps, positions,
                    seq_of_token, table, 64, H, G, dk, dv)
    # the written queries and keys are the plain ones: turned, then of unit length
    q_want = np.stack([P.unit(P.rotate(q[t], t, rot, "neighbours"), eps) for t in range(T)])
    k_want = np.stack([P.unit(P.rotate(k[t], t, rot, "neighbours"), eps) for t in range(T)])
    round_tol = 1e-5 if dtype == torch.float32 else 8e-3
    assert rel(q_dev, q_want) < round_tol
    pages = table[0].tolist()
    rows = torch.cat([cache[p, 0] for p in pages], dim=1)[:, :T]            # [G, T, dk + dv]
    assert rel(rows[:, :, :dk].transpose(0, 1), k_want) < round_tol
    assert rel(rows[:, :, dk:].transpose(0, 1), v) < round_tol
    if dtype == torch.bfloat16:                               # the reference takes what the cache holds
        want = attention_of_rounded(host(q_dev), host(rows[:, :, :dk].transpose(0, 1)), host(rows[:, :, dk:].transpose(0, 1)),
                                    m, sink).reshape(T, H * dv)
    sink_dev = dev(sink)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for n_splits in (1, 2, 5, 64):
        for form in ("", "group", "heads"):
            os.environ["TQ_BIAS_TOKEN_FORM"] = form
            try:
                out = torch.full((T, H * dv), float("nan"), dtype=dtype, device=DEV)
                KB.attention(q_dev, cache, None, sink_dev, positions, seq_of_token, table, 64, window, 0, scale, out, H, G,
                             dk, dv, n_splits=n_splits, softcap=cap)
            finally:
                os.environ.pop("TQ_BIAS_TOKEN_FORM", None)
            assert rel(out, want) < tol, (n_splits, form)
    if KB.runs_usable(dtype, dk, dv, 64):
        for start in (0, 77):                                 # one run; a run that continues a sequence
            out = torch.full((T - start, H * dv), float("nan"), dtype=dtype, device=DEV)
            KB.attention_runs(q_dev[start:].contiguous(), cache, None, sink_dev, i32([0, T - start]), i32([start]), table, 64,
                              window, 0, scale, out, 1, T - start, H, G, dk, dv, softcap=cap)
            assert rel(out, want[start:]) < tol, start


def attention_of_rounded(q, k, v, m, sink):
    """Capped, masked softmax with a sink over queries and keys that are already turned and of unit length."""
    T, H, _ = q.shape
    G = k.shape[1]
    size, cap = (m["mask"]["size"] if m.get("mask") else 0), m.get("softcap", 0.0)
    out = np.zeros((T, H, v.shape[2]))
    for a in range(H):
        g = a // (H // G)
        for i in range(T):
            lo = max(0, i - size + 1) if size else 0
            s = (k[lo:i + 1, g] @ q[i, a]) * m["scale"]
            if cap:
                s = cap * np.tanh(s / cap)
            top = max(s.max(), sink[a])
            e = np.exp(s - top)
            out[i, a] = (e / (e.sum() + math.exp(sink[a] - top))) @ v[lo:i + 1, g]
    return out


@pytest.mark.parametrize("halves", [False, True])
def test_both_pairings_of_the_rotating_write(halves):
    from turboquant_cpp_b200.kernels import bias_attention as KB
    T, H, G, dk, dv = 70, 3, 1, 20, 4
    rot = {"dims": 12, "base": 50.0}
    rng = np.random.default_rng(5)
    qkv = host(dev(rng.standard_normal((T, H * dk + G * (dk + dv)))))
    start = 1000                                              # large angles: computed from the position in float32
    positions = torch.arange(start, start + T, dtype=torch.int32, device=DEV)
    q_dev = torch.empty((T, H, dk), dtype=torch.float32, device=DEV)
    KB.kv_write_rot(dev(qkv), q_dev, None, frequencies(rot), 12, halves, 0.0, positions, torch.zeros(T, dtype=torch.int32, device=DEV),
                    i32([[0]]), 64, H, G, dk, dv)
    q = qkv[:, :H * dk].reshape(T, H, dk)
    want = np.stack([P.rotate(q[t], start + t, rot, "halves" if halves else "neighbours") for t in range(T)])
    assert rel(q_dev, want) < 2e-4                            # an angle of 1,000 radians keeps 2^-14 of a turn in float32


RET_CASES = [
    # heads, dk, dv, decays, rot
    (3, 8, 12, (0.9, 0.97, 1.0), {"dims": 8, "base": 500.0}),
    (2, 64, 64, (0.5, 0.9990234375), {"dims": 32, "base": 1e4}),
    (1, 200, 3, (0.99,), None),
    (5, 5, 33, (0.1, 0.3, 0.5, 0.7, 0.9), {"dims": 4, "base": 9.0}),
    (4, 96, 128, (0.9375, 0.99, 0.999, 0.9999), {"dims": 64, "base": 2e5}),
]


@pytest.mark.parametrize("case", RET_CASES)
def test_retention_over_portions_in_used_slots(case):
    """Two sequences share every step, cut differently; their slots held other values before (the first portion starts
    from a state the test zeroes as the cache does on opening; every later one from what the step before left)."""
    from turboquant_cpp_b200.kernels import ssm as KS
    heads, dk, dv, decay, rot = case
    rng = np.random.default_rng(heads * 100 + dk)
    lens = {0: 341, 1: 28}
    m = {"decay": list(decay), "rot": rot, "heads": heads, "dim": dk, "vdim": dv}
    qk, inner = heads * dk, heads * dv
    lead = 7                                                  # the rows begin with something else
    proj = {s: host(dev(rng.standard_normal((n, lead + 2 * qk + 2 * inner)))) for s, n in lens.items()}
    want = {}
    for s, n in lens.items():
        pr = proj[s][:, lead:]
        o, _ = P.retention_core(pr[:, :qk].reshape(n, heads, dk), pr[:, qk:2 * qk].reshape(n, heads, dk),
                                pr[:, 2 * qk:2 * qk + inner].reshape(n, heads, dv), m)
        want[s] = o.reshape(n, inner)
    state = torch.full((5, heads, dv, dk), 7.0, dtype=torch.float32, device=DEV)
    slots = {0: 3, 1: 1}
    for s in slots.values():
        state[s].zero_()
    cuts = [(1, 2), (2, 1), (17, 1), (300, 5), (1, 17), (20, 2)]
    at = {0: 0, 1: 0}
    decay_dev = dev(np.array(decay))
    for n0, n1 in cuts:
        pr = dev(np.concatenate([proj[0][at[0]:at[0] + n0], proj[1][at[1]:at[1] + n1]]))
        T = n0 + n1
        positions = i32(list(range(at[0], at[0] + n0)) + list(range(at[1], at[1] + n1)))
        xbc = torch.empty((T, inner + 2 * qk), dtype=torch.float32, device=DEV)
        KS.retention_prepare(pr, lead, lead + qk, lead + 2 * qk, xbc, frequencies(rot), rot["dims"] if rot else 0, True,
                             dk ** -0.5, positions, heads, dk, dv)
        y = torch.empty((T, inner), dtype=torch.float32, device=DEV)
        KS.ssm_scan(xbc, None, 0, None, None, None, state, y, heads, dv, dk, heads, i32([0, n0, T]),
                    i32([slots[0], slots[1]]), fixed_decay=decay_dev)
        for s, lo, n in ((0, 0, n0), (1, n0, n1)):
            ref = want[s][at[s]:at[s] + n]
            assert np.abs(host(y[lo:lo + n]) - ref).max() < 3e-5 * max(1.0, np.abs(want[s]).max()), (s, at[s], n)
        at[0] += n0
        at[1] += n1
    assert at == lens
    assert float(state[0].min()) == 7.0 and float(state[4].max()) == 7.0       # other slots are not touched


@pytest.mark.parametrize("case", RET_CASES)
def test_retention_in_chunks_side_by_side(case):
    """Long runs cut into chunks that are scanned side by side from zero states, put right by the states they should
    have started from, and scanned again: the outputs of the plain recurrence, over two portions (the second goes
    on from kept states), with chunks of unequal sizes, a last chunk of one token, and other slots left alone."""
    from turboquant_cpp_b200.kernels import ssm as KS
    heads, dk, dv, decay, rot = case
    rng = np.random.default_rng(heads * 10 + dv)
    lens = {0: 341, 1: 150}
    m = {"decay": list(decay), "rot": rot, "heads": heads, "dim": dk, "vdim": dv}
    qk, inner = heads * dk, heads * dv
    proj = {s: host(dev(rng.standard_normal((n, 2 * qk + inner)))) for s, n in lens.items()}
    want, last = {}, {}
    for s, n in lens.items():
        pr = proj[s]
        o, last[s] = P.retention_core(pr[:, :qk].reshape(n, heads, dk), pr[:, qk:2 * qk].reshape(n, heads, dk),
                                      pr[:, 2 * qk:].reshape(n, heads, dv), m)
        want[s] = o.reshape(n, inner)
    state = torch.full((4, heads, dv, dk), 7.0, dtype=torch.float32, device=DEV)
    slots = {0: 2, 1: 0}
    for s in slots.values():
        state[s].zero_()
    decay_dev = dev(np.array(decay))
    at = {0: 0, 1: 0}
    for (n0, n1), size in (((193, 100), 48), ((148, 50), 64)):
        pr = dev(np.concatenate([proj[0][at[0]:at[0] + n0], proj[1][at[1]:at[1] + n1]]))
        T = n0 + n1
        positions = i32(list(range(at[0], at[0] + n0)) + list(range(at[1], at[1] + n1)))
        xbc = torch.empty((T, inner + 2 * qk), dtype=torch.float32, device=DEV)
        KS.retention_prepare(pr, 0, qk, 2 * qk, xbc, frequencies(rot), rot["dims"] if rot else 0, True, dk ** -0.5, positions,
                             heads, dk, dv)
        cu, seq_chunks, lo = [0], [0], 0
        for n in (n0, n1):
            cu += [lo + min(n, c + size) for c in range(0, n, size)]
            seq_chunks.append(len(cu) - 1)
            lo += n
        n_chunks = len(cu) - 1
        ends = torch.zeros((n_chunks, heads, dv, dk), dtype=torch.float32, device=DEV)
        starts = torch.full((n_chunks, heads, dv, dk), 3.0, dtype=torch.float32, device=DEV)
        y = torch.full((T, inner), float("nan"), dtype=torch.float32, device=DEV)
        ids = i32(list(range(n_chunks)))
        KS.ssm_scan(xbc, None, 0, None, None, None, ends, None, heads, dv, dk, heads, i32(cu), ids, fixed_decay=decay_dev)   # the states alone
        KS.retention_combine(state, i32([slots[0], slots[1]]), ends, starts, i32(seq_chunks), i32(cu), decay_dev)
        KS.ssm_scan(xbc, None, 0, None, None, None, starts, y, heads, dv, dk, heads, i32(cu), ids, fixed_decay=decay_dev)
        for s, lo, n in ((0, 0, n0), (1, n0, n1)):
            ref = want[s][at[s]:at[s] + n]
            assert np.abs(host(y[lo:lo + n]) - ref).max() < 3e-5 * max(1.0, np.abs(want[s]).max()), (s, at[s], n)
        at[0] += n0
        at[1] += n1
    assert at == lens
    for s in lens:                                            # the kept state is the plain recurrence's, [heads, dk, dv] there
        kept = host(state[slots[s]]).transpose(0, 2, 1)
        assert np.abs(kept - last[s]).max() < 3e-5 * max(1.0, np.abs(last[s]).max())
    assert float(state[1].min()) == 7.0 and float(state[3].max()) == 7.0


@pytest.mark.parametrize("case", RET_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_token_of_every_sequence_in_one_launch(case, dtype):
    """Decode steps through the one-launch form: three sequences at different positions, in slots that held other
    values, after a prompt through the kernels for runs; rotation, recurrence, unit norm and gate against the plain
    steps, and slots of other sequences left alone."""
    from turboquant_cpp_b200.kernels import ssm as KS
    heads, dk, dv, decay, rot = case
    rng = np.random.default_rng(heads + dk + dv)
    m = {"decay": list(decay), "rot": rot, "heads": heads, "dim": dk, "vdim": dv}
    qk, inner = heads * dk, heads * dv
    lead = 5
    lens, prompt = {0: 40, 1: 23, 2: 31}, {0: 17, 1: 0, 2: 30}
    proj = {s: host(dev(rng.standard_normal((n, lead + 2 * qk + 2 * inner)))) for s, n in lens.items()}
    want = {}
    for s, n in lens.items():
        pr = proj[s][:, lead:]
        o, _ = P.retention_core(pr[:, :qk].reshape(n, heads, dk), pr[:, qk:2 * qk].reshape(n, heads, dk),
                                pr[:, 2 * qk:2 * qk + inner].reshape(n, heads, dv), m)
        want[s] = (P.unit(o, 2e-4).reshape(n, inner) * P.silu(pr[:, 2 * qk + inner:]))
    state = torch.full((6, heads, dv, dk), 7.0, dtype=torch.float32, device=DEV)
    slots = {0: 4, 1: 0, 2: 2}
    decay_dev = dev(np.array(decay))
    f, rd = frequencies(rot), rot["dims"] if rot else 0
    for s, n in prompt.items():                               # prompts through the kernels for runs
        state[slots[s]].zero_()
        if n == 0:
            continue
        xbc = torch.empty((n, inner + 2 * qk), dtype=torch.float32, device=DEV)
        KS.retention_prepare(dev(proj[s][:n]), lead, lead + qk, lead + 2 * qk, xbc, f, rd, True, dk ** -0.5, i32(list(range(n))), heads, dk, dv)
        KS.ssm_scan(xbc, None, 0, None, None, None, state, torch.empty((n, inner), dtype=torch.float32, device=DEV), heads, dv, dk,
                    heads, i32([0, n]), i32([slots[s]]), fixed_decay=decay_dev)
    at = dict(prompt)
    tol = 3e-5 if dtype == torch.float32 else 1e-2
    while any(at[s] < lens[s] for s in lens):
        live = [s for s in lens if at[s] < lens[s]]
        pr = dev(np.stack([proj[s][at[s]] for s in live]))
        out = torch.empty((len(live), inner), dtype=dtype, device=DEV)
        KS.retention_step(pr, lead, lead + qk, lead + 2 * qk, lead + 2 * qk + inner, f, rd, True, dk ** -0.5,
                          i32([at[s] for s in live]), state, i32([slots[s] for s in live]), decay_dev, out, heads, dk, dv, 2e-4)
        for i, s in enumerate(live):
            ref = want[s][at[s]]
            assert np.abs(host(out[i]) - ref).max() < tol * max(1.0, np.abs(ref).max()), (s, at[s])
            at[s] += 1
    assert float(state[1].min()) == 7.0 and float(state[3].max()) == 7.0 and float(state[5].min()) == 7.0


def test_a_far_token_speaks_through_a_head_that_forgets_nothing():
    """A key along one direction at position 3, a query along it 900 tokens later, a decay of one: the output holds that
    token's value at full weight; the head beside it, with a decay of 0.9, has lost it."""
    from turboquant_cpp_b200.kernels import ssm as KS
    heads, dk, dv, T = 2, 16, 8, 904
    rng = np.random.default_rng(2)
    q, k, v = (0.01 * rng.standard_normal((T, heads, d)) for d in (dk, dk, dv))
    k[3, :, 0], q[T - 1, :, 0], v[3] = 4.0, 4.0, 5.0 * np.sign(rng.standard_normal((heads, dv)))
    m = {"decay": [1.0, 0.9], "rot": None}
    proj = host(dev(np.concatenate([a.reshape(T, -1) for a in (q, k, v)], axis=1)))
    qk, inner = heads * dk, heads * dv
    o, _ = P.retention_core(proj[:, :qk].reshape(T, heads, dk), proj[:, qk:2 * qk].reshape(T, heads, dk),
                            proj[:, 2 * qk:].reshape(T, heads, dv), m)
    assert np.abs(o[T - 1, 0]).min() > 15.0 and np.abs(o[T - 1, 1]).max() < 0.1
    state = torch.zeros((1, heads, dv, dk), dtype=torch.float32, device=DEV)
    got = []
    for lo, hi in ((0, 600), (600, 601), (601, 603), (603, 903), (903, 904)):
        n = hi - lo
        xbc = torch.empty((n, inner + 2 * qk), dtype=torch.float32, device=DEV)
        KS.retention_prepare(dev(proj[lo:hi]), 0, qk, 2 * qk, xbc, None, 0, True, dk ** -0.5, i32(list(range(lo, hi))), heads, dk, dv)
        y = torch.empty((n, inner), dtype=torch.float32, device=DEV)
        KS.ssm_scan(xbc, None, 0, None, None, None, state, y, heads, dv, dk, heads, i32([0, n]), i32([0]), fixed_decay=dev(np.array([1.0, 0.9])))
        got.append(host(y))
    got = np.concatenate(got)
    assert np.abs(got - o.reshape(T, inner)).max() < 2e-5 * np.abs(o).max()


@pytest.mark.parametrize("T,heads,dv", [(5, 3, 12), (11, 8, 128), (3, 1, 1200), (2, 5, 7)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unit_norm_per_head_then_the_gate(T, heads, dv, dtype):
    from turboquant_cpp_b200.kernels import ssm as KS
    rng = np.random.default_rng(6)
    inner = heads * dv
    y, proj = host(dev(3.0 * rng.standard_normal((T, inner)))), host(dev(rng.standard_normal((T, inner + 9))))
    out = torch.empty((T, inner), dtype=dtype, device=DEV)
    KS.gated_group_norm(dev(y), dev(proj), 9, None, heads, 3e-3, out, gate_after=True)
    want = P.unit(y.reshape(T, heads, dv), 3e-3).reshape(T, inner) * P.silu(proj[:, 9:])
    assert rel(out, want) < (1e-5 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("R,H", [(1, 36), (7, 48), (33, 1024), (3, 5000)])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_mean_of_two_normed_branches(R, H, wdtype):
    from turboquant_cpp_b200.kernels import elementwise as KE
    rng = np.random.default_rng(R + H)
    a, b = host(dev(5.0 * rng.standard_normal((R, H)))), host(dev(0.01 * rng.standard_normal((R, H))))   # unlike sizes: each has its own norm
    wa, wb = dev(1 + 0.3 * rng.standard_normal(H), wdtype), dev(1 + 0.3 * rng.standard_normal(H), wdtype)
    out = torch.empty((R, H), dtype=torch.float32, device=DEV)
    KE.mean_of_norms(dev(a), wa, dev(b), wb, 1e-5, out)
    want = 0.5 * (P.norm(a, host(wa), 1e-5) + P.norm(b, host(wb), 1e-5))
    assert rel(out, want) < 1e-5


@pytest.mark.parametrize("R,H", [(1, 36), (3, 256), (7, 1000), (2, 2048), (2, 5000), (5, 37)])
@pytest.mark.parametrize("wdtype,odtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_a_sum_under_a_norm_with_the_next_norm_along(R, H, wdtype, odtype):
    """x += norm(y), and the norm that reads the new x next in the same pass (both row forms of the kernel: rows of
    a multiple of four up to 4096 elements, and the rest)."""
    from turboquant_cpp_b200.kernels import elementwise as KE
    rng = np.random.default_rng(R * H)
    x, y = host(dev(rng.standard_normal((R, H)))), host(dev(0.02 * rng.standard_normal((R, H))))
    w, wn = dev(1 + 0.3 * rng.standard_normal(H), wdtype), dev(1 + 0.3 * rng.standard_normal(H), wdtype)
    xd = dev(x)
    copy = torch.empty((R, H), dtype=odtype, device=DEV)
    nxt = torch.empty((R, H), dtype=odtype, device=DEV)
    KE.add_rmsnorm(xd, dev(y), w, 1e-5, copy, wn, nxt, 3e-4)
    want = x + P.norm(y, host(w), 1e-5)
    tol = 1e-5 if odtype == torch.float32 else 5e-3
    assert rel(xd, want) < 1e-5 and rel(copy, want) < tol
    assert rel(nxt, P.norm(want, host(wn), 3e-4)) < tol
    xd2, nxt2 = dev(x), torch.empty((R, H), dtype=odtype, device=DEV)
    KE.add_rmsnorm(xd2, dev(y), w, 1e-5, None, wn, nxt2)              # no copy; the following norm with the same eps
    assert torch.equal(xd2, xd) and rel(nxt2, P.norm(want, host(wn), 1e-5)) < tol


@pytest.mark.parametrize("R,H", [(1, 36), (3, 256), (7, 1000), (2, 2048), (2, 5000), (5, 37)])
@pytest.mark.parametrize("wdtype,odtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_two_normed_branches_under_the_sum_and_the_next_norm(R, H, wdtype, odtype):
    """x += norm(mean of two normed branches) and the next norm of x in one pass, both row forms of the kernel; the
    branches differ in size by orders of magnitude, so a shared norm or a missing one would show."""
    from turboquant_cpp_b200.kernels import elementwise as KE
    rng = np.random.default_rng(R * H + 1)
    x = host(dev(rng.standard_normal((R, H))))
    a, b = host(dev(40.0 * rng.standard_normal((R, H)))), host(dev(0.003 * rng.standard_normal((R, H))))
    wa, wb, w, wn = (dev(1 + 0.3 * rng.standard_normal(H), wdtype) for _ in range(4))
    m = 0.5 * (P.norm(a, host(wa), 2e-5) + P.norm(b, host(wb), 2e-5))
    want = x + P.norm(m, host(w), 1e-4)
    tol = 1e-5 if odtype == torch.float32 else 5e-3
    xd, copy, nxt = dev(x), torch.empty((R, H), dtype=odtype, device=DEV), torch.empty((R, H), dtype=odtype, device=DEV)
    KE.add_rmsnorm_pair(xd, dev(a), wa, dev(b), wb, 2e-5, w, 1e-4, copy, wn, nxt, 3e-4)
    assert rel(xd, want) < 1e-5 and rel(copy, want) < tol and rel(nxt, P.norm(want, host(wn), 3e-4)) < tol
    xd2 = dev(x)
    KE.add_rmsnorm_pair(xd2, dev(a), wa, dev(b), wb, 2e-5, w, 1e-4)      # the sum alone
    assert torch.equal(xd2, xd)


@pytest.mark.parametrize("T,D,col0,width", [(1, 24, 0, 24), (9, 6, 12, 30), (40, 1, 3, 4), (5, 130, 130, 390)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_slice_of_a_token_table(T, D, col0, width, dtype):
    from turboquant_cpp_b200.kernels import elementwise as KE
    rng = np.random.default_rng(T + D)
    V = 19
    table = dev(rng.standard_normal((V, width)), dtype)
    z = host(dev(2.0 * rng.standard_normal((T, D))))
    tokens = rng.integers(0, V, size=T)
    out = torch.empty((T, D), dtype=dtype, device=DEV)
    KE.glu_table_rows(dev(z), i32(tokens.tolist()), table, col0, out, KE.GELU_TANH_GLU)
    want = P.gelu_tanh(z) * host(table)[tokens, col0:col0 + D]
    assert rel(out, want) < (1e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_tanh_form_of_gelu_as_a_gate(dtype):
    from turboquant_cpp_b200.kernels import elementwise as KE
    rng = np.random.default_rng(1)
    gu = host(dev(3.0 * rng.standard_normal((37, 2 * 50))))
    out = torch.empty((37, 50), dtype=dtype, device=DEV)
    KE.glu_mul(dev(gu), out, KE.GELU_TANH_GLU)
    assert rel(out, P.gelu_tanh(gu[:, :50]) * gu[:, 50:]) < (1e-6 if dtype == torch.float32 else 5e-3)


def test_scaled_columns():
    from turboquant_cpp_b200.kernels import elementwise as KE
    rng = np.random.default_rng(2)
    x = host(dev(rng.standard_normal((6, 301))))
    assert rel(KE.scale_bias_cols(dev(x), 0.37), 0.37 * x) < 1e-6
    bias = host(dev(rng.standard_normal(100)))
    want = x.copy()
    want[:, :100] = 2.0 * want[:, :100] + bias
    assert rel(KE.scale_bias_cols(dev(x), 2.0, dev(bias), cols=100), want) < 1e-6


@pytest.mark.parametrize("T,E,k,H", [(1, 12, 2, 64), (8, 60, 4, 128), (5, 8, 8, 40), (300, 16, 3, 72), (24, 1, 1, 36), (70, 72, 6, 48)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_bias_on_the_routers_logits_in_every_router_form(T, E, k, H, dtype):
    """The bias decides the choice (it is larger than the logits' spread) and enters the weights: the separate kernels,
    the one for logits alone, and the one-launch form of small steps."""
    from turboquant_cpp_b200.kernels import moe as KM
    rng = np.random.default_rng(T * 100 + E)
    x, wr = dev(rng.standard_normal((T, H)), dtype), dev(0.05 * rng.standard_normal((E, H)), dtype)
    bias = host(dev(2.0 * rng.standard_normal(E)))
    w = {"router": host(wr), "router.b": bias}
    ids, wts, margins = P.route(host(x), {"router": {"top": k}}, w, "")
    i32k, f32k = dict(dtype=torch.int32, device=DEV), dict(dtype=torch.float32, device=DEV)
    forms = []
    ids_a, w_a = torch.empty((T, k), **i32k), torch.empty((T, k), **f32k)
    KM.router_topk(x, wr, None, k, True, ids_a, w_a, None, logit_bias=dev(bias))
    forms.append(("topk", ids_a, w_a))
    logits = KM.router_logits(x, wr, None, torch.empty((T, E + 1), **f32k), logit_bias=dev(bias))
    assert rel(logits[:, :E], host(x) @ host(wr).T + bias) < 1e-5
    ids_b, w_b = torch.empty((T, k), **i32k), torch.empty((T, k), **f32k)
    KM.router_select(logits, k, True, ids_b, w_b, None)
    forms.append(("select", ids_b, w_b))
    if KM.router_small_usable(T, k, E, H):
        ids_c, w_c = torch.empty((T, k), **i32k), torch.empty((T, k), **f32k)
        lay = KM.ExpertLayout(T * k, E, 16, DEV)
        KM.router_small(x, wr, None, k, True, ids_c, w_c, None, lay, torch.empty((T * k, H), dtype=dtype, device=DEV), logit_bias=dev(bias))
        forms.append(("small", ids_c, w_c))
    unbiased = np.argsort(-(host(x) @ host(wr).T), axis=-1, kind="stable")[:, :k]
    assert E == k or (np.sort(unbiased, axis=1) != np.sort(ids, axis=1)).any()          # without the bias the choice is another
    for name, gi, gw in forms:
        gi, gw = gi.cpu().numpy(), host(gw)
        for t in range(T):
            if margins[t] > 1e-5:
                order = np.argsort(gi[t])
                assert gi[t][order].tolist() == sorted(ids[t].tolist()), (name, t)
                assert np.abs(gw[t][order] - wts[t][np.argsort(ids[t])]).max() < 1e-5, (name, t)
