"""The kernels behind the Tasadra parts, each alone against the plain functions (tests/plain/tasadra_plain.py): the
dynamic-tanh norm with the token shift over portions in slots that held other values, the weighted sum over depth, the
cache write with head norms, stretched rotation, turned values and shared values, the attention kernels with cells of
positions (a marked key just inside and just outside a cell, at page borders, in a prompt and for single tokens, over
scattered pages), the turn back with the gate, the two maps' combination, and the delta rule with its state carried
over portions."""
import os

import numpy as np
import pytest
import torch

from plain import tasadra_plain as P

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


def scattered_cache(T, G, dr, dtype, rng, extra_pages=3):
    """More pages than the sequence needs, a large value where nothing is written, pages visited in a shuffled order."""
    n = -(-T // 64)
    cache = torch.full((n + extra_pages, 1, G, 64, dr), 1e30, dtype=dtype, device=DEV)
    table = torch.tensor(rng.permutation(n + extra_pages)[:n].reshape(1, n), dtype=torch.int32, device=DEV)
    return cache, table


# ---- norm, shift, depth ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("H,pad", [(70, 13), (72, 12)])          # rows the 16-byte form cannot take, and rows it takes
@pytest.mark.parametrize("wdtype,odtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_dynamic_tanh_with_sums_rows_and_the_shift_over_portions(wdtype, odtype, H, pad):
    from turboquant_cpp_b200.kernels import elementwise as K
    rng = np.random.default_rng(3)
    alpha = 0.7
    w, b, s = (host(dev(a, wdtype)) for a in (1 + 0.2 * rng.standard_normal(H), 0.3 * rng.standard_normal(H), rng.random(H)))
    wt = {"n": w, "n.b": b, "n.alpha": alpha}
    tol = 1e-5 if odtype == torch.float32 else 8e-3
    # plain rows, a sum with a factor on the way (the stream takes it), chosen rows
    x, y = rng.standard_normal((9, H)) * 2, rng.standard_normal((9, H))
    xd = dev(x)
    out = K.dyt(xd, alpha, dev(w, wdtype), dev(b, wdtype), torch.empty((9, H), dtype=odtype, device=DEV))
    assert rel(out, P.dyt(host(xd), wt, "n")) < tol
    out = K.dyt(xd, alpha, dev(w, wdtype), dev(b, wdtype), torch.empty((9, H), dtype=odtype, device=DEV), add=dev(y), add_scale=0.6)
    summed = host(dev(x)) + 0.6 * host(dev(y))
    assert rel(xd, summed) < 1e-6 and rel(out, P.dyt(summed, wt, "n")) < tol
    rows = [7, 0, 3]
    out = K.dyt(xd, alpha, dev(w, wdtype), dev(b, wdtype), torch.empty((3, H), dtype=odtype, device=DEV), rows=i32(rows))
    assert rel(out, P.dyt(summed[rows], wt, "n")) < tol
    # three sequences in portions of unequal sizes, down to one and two tokens; slots in another order than the batch;
    # the rows of the state area hold other values where no sequence lives, and views with a stride
    lens = [23, 40, 5]
    seqs = [rng.standard_normal((n, H)) * 2 for n in lens]
    want = [P.token_shift(P.dyt(host(dev(q)), wt, "n"), s) for q in seqs]
    area = torch.full((6, 4 + H + pad), 7.0, device=DEV)
    kept = area[:, 4:4 + H]
    slots = [4, 0, 2]
    for sl in slots:
        kept[sl].zero_()
    done = [0, 0, 0]
    for portion in ([1, 17, 2], [2, 1, 1], [1, 1, 1], [19, 21, 1]):
        live = [i for i in range(3) if done[i] < lens[i]]
        take = [min(portion[i], lens[i] - done[i]) for i in live]
        xs = np.concatenate([seqs[i][done[i]:done[i] + n] for i, n in zip(live, take)])
        cu = np.concatenate([[0], np.cumsum(take)])
        out = K.dyt(dev(xs), alpha, dev(w, wdtype), dev(b, wdtype), torch.empty((len(xs), H), dtype=odtype, device=DEV),
                    shift=dev(s, wdtype), state=kept, seq_of_token=i32(np.repeat(np.arange(len(live)), take)),
                    cu_seqlens=i32(cu), slots=i32([slots[i] for i in live]), single_tokens=max(take) == 1)
        ref = np.concatenate([want[i][done[i]:done[i] + n] for i, n in zip(live, take)])
        assert rel(out, ref) < tol, portion
        for i, n in zip(live, take):
            done[i] += n
    assert done == lens
    assert float(area[1].min()) == 7.0 and float(area[:, :4].min()) == 7.0 and float(area[:, 4 + H:].min()) == 7.0


def test_weighted_sum_over_depth_and_bias_before_the_square_of_relu():
    from turboquant_cpp_b200.kernels import elementwise as K
    rng = np.random.default_rng(5)
    T, H, n = 13, 50, 4
    hist = rng.standard_normal((n, T, H))
    x, f, bias, wts = rng.standard_normal((T, H)), rng.standard_normal((T, H)), rng.standard_normal(H), rng.standard_normal(n)
    for fdtype in (torch.float32, torch.bfloat16):
        hd, xd = dev(hist), dev(x)
        fr, br = host(dev(f, fdtype)), host(dev(bias, fdtype))
        K.depth_mix(hd, 2, xd, dev(wts), xd, add=dev(f, fdtype), add_scale=0.7, bias=dev(bias, fdtype))
        new = host(dev(x)) + 0.7 * (fr + br)
        assert rel(hd[2], new) < 1e-6 and rel(hd[3], host(dev(hist[3]))) == 0.0
        assert rel(xd, wts[0] * hist[0] + wts[1] * hist[1] + wts[2] * new) < 1e-6
    hd, xd = dev(hist), dev(x)
    K.depth_mix(hd, 0, xd, dev(wts), torch.empty_like(xd))                     # nothing to add: the entry is the stream itself
    assert rel(hd[0], host(dev(x))) == 0.0
    u = rng.standard_normal((T, H))
    out = K.bias_map(dev(u), dev(bias), torch.empty((T, H), device=DEV), K.MAP_RELU_SQUARED)
    assert rel(out, np.maximum(host(dev(u)) + host(dev(bias)), 0.0) ** 2) < 1e-6


# ---- the cache write --------------------------------------------------------------------------------------------
WRITE_CASES = [
    # H, G, dk, dv, rot dims, scaling, turned values, shared values
    (4, 2, 16, 8, 8, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}, True, 1),
    (3, 3, 40, 12, 40, None, True, 1),
    (6, 2, 24, 10, 0, None, False, 2),
    (2, 1, 64, 128, 32, {"factor": 16.0, "original": 16, "fast": 4.0, "slow": 0.5}, True, 1),
]


@pytest.mark.parametrize("case", WRITE_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cache_write_with_head_norms_stretched_rotation_and_turned_values(case, dtype):
    from turboquant_cpp_b200.kernels import bias_attention as KB
    H, G, dk, dv, dims, scaling, turn_values, share = case
    rng = np.random.default_rng(H * 100 + dk)
    T, eps, base = 150, 3e-4, 5000.0
    Gv = G // share
    rows = host(dev(rng.standard_normal((T, H * dk + G * dk + Gv * dv + 9)) * 1.5))
    q = rows[:, :H * dk].reshape(T, H, dk)
    k = rows[:, H * dk:(H + G) * dk].reshape(T, G, dk)
    v = rows[:, (H + G) * dk:(H + G) * dk + Gv * dv].reshape(T, Gv, dv)
    wq, wk = host(dev(1 + 0.3 * rng.standard_normal(dk))), host(dev(1 + 0.3 * rng.standard_normal(dk)))
    normed = dims > 0
    pos = np.arange(T)
    freq, mag = P.scaled_frequencies(dims, base, scaling) if dims else (np.zeros(0), 1.0)
    q_want = P.unit_rms(q, eps) * wq if normed else q
    k_want = P.unit_rms(k, eps) * wk if normed else k
    if dims:
        q_want, k_want = P.rotate_halves(q_want, pos, freq, mag), P.rotate_halves(k_want, pos, freq, mag)
    vf = P.plain_frequencies(dv, base)
    v_want = P.rotate_halves(v, pos, vf) if turn_values else v
    v_want = np.repeat(v_want, share, axis=1)
    cache, table = scattered_cache(T, G, dk + dv, dtype, rng)
    q_dev = torch.empty((T, H, dk), dtype=dtype, device=DEV)
    KB.kv_write_rot(dev(rows), q_dev, cache, dev(freq) if dims else None, dims, True, 0.0, torch.arange(T, dtype=torch.int32, device=DEV),
                    torch.zeros(T, dtype=torch.int32, device=DEV), table, 64, H, G, dk, dv, mag=mag,
                    q_norm=dev(wq) if normed else None, k_norm=dev(wk) if normed else None, norm_eps=eps,
                    v_freq=dev(vf) if turn_values else None, v_share=share)
    tol = 2e-5 if dtype == torch.float32 else 8e-3
    assert rel(q_dev, q_want) < tol
    got = torch.cat([cache[p, 0] for p in table[0].tolist()], dim=1)[:, :T]            # [G, T, dk + dv]
    assert rel(got[:, :, :dk].transpose(0, 1), k_want) < tol
    assert rel(got[:, :, dk:].transpose(0, 1), v_want) < tol
    # rows that hold queries only, for a layer that reads another's cache
    q_only = torch.empty((T, H, dk), dtype=dtype, device=DEV)
    KB.kv_write_rot(dev(rows[:, :H * dk]), q_only, None, dev(freq) if dims else None, dims, True, 0.0,
                    torch.arange(T, dtype=torch.int32, device=DEV), torch.zeros(T, dtype=torch.int32, device=DEV), table, 64, H, G, dk, dv,
                    mag=mag, q_norm=dev(wq) if normed else None, k_norm=dev(wk) if normed else None, norm_eps=eps, v_share=share)
    assert torch.equal(q_only, q_dev)


# ---- attention inside cells ---------------------------------------------------------------------------------------
def softmax_attention(q, k, v, scale, seen, cap=0.0):
    """q [Tq, H, dk], k [Tk, G, dk], v [Tk, G, dv], seen [Tq, Tk]."""
    H, G = q.shape[1], k.shape[1]
    out = np.zeros((q.shape[0], H, v.shape[2]))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale
        if cap:
            s = cap * np.tanh(s / cap)
        out[:, a] = P.softmax_rows(s, seen) @ v[:, g]
    return out


CELL_CASES = [
    # T, H, G, dk, dv, cell, scale
    (300, 4, 2, 64, 64, 70, 0.3),         # tensor-core sizes, two query heads a key head, cells wider than a page
    (280, 2, 2, 32, 128, 64, 0.4),        # cells of exactly a page, one query head a key head
    (260, 16, 1, 128, 32, 37, 0.15),      # sixteen query heads a key head, cells that divide nothing
    (200, 6, 2, 24, 40, 50, 0.6),         # sizes only the token kernel takes
    (150, 3, 3, 20, 6, 1, 0.5),           # cells of one position: every token sees itself alone
    (330, 4, 4, 64, 64, 130, 0.3),        # cells of more than two pages
]


@pytest.mark.parametrize("case", CELL_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_inside_cells_sees_the_cell_and_nothing_else(case, dtype):
    from turboquant_cpp_b200.kernels import bias_attention as KB
    T, H, G, dk, dv, cell, scale = case
    rng = np.random.default_rng(T + cell)
    q = rng.standard_normal((T, H, dk))
    k = rng.standard_normal((T, G, dk))
    v = rng.standard_normal((T, G, dv))
    # marked keys: the first of a cell (just inside for every query of the cell) and the last of the cell before (just
    # outside); queries at a cell's first, second and last position and at page borders ask for both, and the marked
    # values are ten times the others
    asks = []
    if cell > 1:
        for c in range(1, T // cell):
            inside, outside = c * cell, c * cell - 1
            k[outside] = np.roll(k[inside], 1, axis=-1)       # of one length: a query that asks for both weighs them alike
            v[inside] *= 10.0
            v[outside] *= 10.0
            for i in {c * cell, c * cell + 1, min(T - 1, c * cell + cell - 1), min(T - 1, (c * cell // 64 + 1) * 64)}:
                if i // cell == c:
                    q[i] = np.repeat(k[inside] + k[outside], H // G, axis=0) * 2.0
                    asks.append(i)
    q, k, v = (host(dev(a, dtype)) for a in (q, k, v))
    pos = np.arange(T)
    want = softmax_attention(q, k, v, scale, P.cell_mask(pos, pos, cell)).reshape(T, H * dv)
    if asks:                                                  # the plain function itself sees the marked keys come and go
        moved = softmax_attention(q, k, v, scale, P.cell_mask(pos + 1, pos + 1, cell)).reshape(T, H * dv)
        assert np.abs(moved - want).max(axis=1)[asks].min() > 0.05
    cache, table = scattered_cache(T, G, dk + dv, dtype, rng)
    for t in range(T):
        page = int(table[0, t // 64])
        cache[page, 0, :, t % 64, :dk] = dev(k[t], dtype)
        cache[page, 0, :, t % 64, dk:] = dev(v[t], dtype)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    seq_of_token = torch.zeros(T, dtype=torch.int32, device=DEV)
    q_dev = dev(q, dtype)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for n_splits in (1, 2, 5):
        for form in ("", "group", "heads"):
            os.environ["TQ_BIAS_TOKEN_FORM"] = form
            try:
                out = torch.full((T, H * dv), float("nan"), dtype=dtype, device=DEV)
                KB.attention(q_dev, cache, None, None, positions, seq_of_token, table, 64, 0, 0, scale, out, H, G, dk, dv,
                             n_splits=n_splits, cell=cell)
            finally:
                os.environ.pop("TQ_BIAS_TOKEN_FORM", None)
            assert rel(out, want) < tol, (n_splits, form)
    if KB.runs_usable(dtype, dk, dv, 64):
        for start in (0, 77, T - 3):                          # one run; runs that continue a sequence inside a cell
            out = torch.full((T - start, H * dv), float("nan"), dtype=dtype, device=DEV)
            KB.attention_runs(q_dev[start:].contiguous(), cache, None, None, i32([0, T - start]), i32([start]), table, 64, 0, 0,
                              scale, out, 1, T - start, H, G, dk, dv, cell=cell)
            assert rel(out, want[start:]) < tol, start


# ---- what follows the weighted sums -------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dv,turn", [(4, 8, True), (3, 128, True), (5, 7, False), (1, 2, True)])
def test_heads_turned_back_and_gated(H, dv, turn, dtype):
    from turboquant_cpp_b200.kernels import bias_attention as KB
    rng = np.random.default_rng(H + dv)
    T = 70
    o = host(dev(rng.standard_normal((T, H, dv)), dtype))
    gates = host(dev(rng.standard_normal((T, 5 + H + 3)) * 2))
    pos = rng.integers(0, 500, size=T)                        # angles are float32 products: their rounding grows with the position
    vf = P.plain_frequencies(dv, 777.0)
    want = (P.rotate_halves(o, pos, vf, sign=-1.0) if turn else o) * P.sigmoid(gates[:, 5:5 + H])[:, :, None]
    od = dev(o.reshape(T, H * dv), dtype)
    KB.heads_unrotate_gate(od, dev(gates), 5, dev(vf) if turn else None, True, i32(pos), od, H, dv)
    assert rel(od, want.reshape(T, H * dv)) < (5e-5 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dv", [(4, 2, 16), (3, 3, 96), (8, 1, 128), (1, 1, 1)])
def test_two_maps_combined_normed_and_gated(H, G, dv, dtype):
    from turboquant_cpp_b200.kernels import bias_attention as KB
    rng = np.random.default_rng(H + dv)
    T, lam, eps, diff, per = 33, 0.83, 2e-4, 0.3, H // G
    maps = host(dev(rng.standard_normal((T, G, 2, per, dv)), dtype))                   # as the attention kernels leave them
    gates = host(dev(rng.standard_normal((T, 7 + H * dv)) * 2))
    want = np.zeros((T, H, dv))
    for a in range(H):
        want[:, a] = P.differential_combine(maps[:, a // per, 0, a % per], maps[:, a // per, 1, a % per], lam, eps, diff)
    want = want.reshape(T, H * dv) * P.sigmoid(gates[:, 7:])
    out = torch.empty((T, H * dv), dtype=dtype, device=DEV)
    KB.diff_combine(dev(maps.reshape(T, -1), dtype), dev(gates), 7, lam, eps, 1.0 - diff, out, H, G, dv)
    assert rel(out, want) < (2e-5 if dtype == torch.float32 else 8e-3)


# ---- the delta rule -------------------------------------------------------------------------------------------------
DELTA_CASES = [
    # H, G, dk, dv
    (4, 2, 8, 12),
    (2, 2, 64, 40),
    (3, 1, 100, 16),
    (1, 1, 200, 21),
    (2, 1, 1, 1),
    (2, 2, 128, 128),
]


@pytest.mark.parametrize("form", ["delta_scan", "delta_scan_runs"])
@pytest.mark.parametrize("case", DELTA_CASES)
def test_delta_rule_over_portions_in_used_slots(case, form):
    from turboquant_cpp_b200.kernels import ssm as KS
    H, G, dk, dv = case
    rng = np.random.default_rng(dk * 10 + dv)
    lens = [61, 9, 130]
    unit_eps, q_scale = 1e-6, dk ** -0.5
    a_log, dt_bias = host(dev(rng.standard_normal(H) * 0.7)), host(dev(rng.standard_normal(H * dk)))
    C = 2 * G * dk + H * dv
    b_off, a_off = 3, 2
    data, want = [], []
    for n in lens:
        xqkv = host(dev(rng.standard_normal((n, C))))
        proj = host(dev(rng.standard_normal((n, b_off + H + 4)) * 2))
        raw = host(dev(rng.standard_normal((n, a_off + H * dk + 1)) * 2 - 2))
        data.append((xqkv, proj, raw))
        q = xqkv[:, :G * dk].reshape(n, G, dk)
        k = xqkv[:, G * dk:2 * G * dk].reshape(n, G, dk)
        v = xqkv[:, 2 * G * dk:].reshape(n, H, dv)
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + unit_eps) * q_scale
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + unit_eps)
        beta = P.sigmoid(proj[:, b_off:b_off + H])
        decay = np.exp(-np.exp(a_log)[None, :, None] * P.softplus(raw[:, a_off:a_off + H * dk] + dt_bias).reshape(n, H, dk))
        outs = [P.delta_rule(q[:, a // (H // G)], k[:, a // (H // G)], v[:, a], beta[:, a], decay[:, a]) for a in range(H)]
        want.append((np.stack([o for o, _ in outs], axis=1).reshape(n, H * dv), np.stack([S for _, S in outs])))
    area = torch.full((5, 11 + H * dv * dk), 3.0, device=DEV)              # rows of other values; the state is a view with a stride
    state = area[:, 11:].unflatten(1, (H, dv, dk))
    slots = [3, 0, 4]
    for sl in slots:
        state[sl].zero_()
    done = [0, 0, 0]
    for portion in ([1, 2, 17], [2, 1, 1], [40, 6, 100], [18, 0, 12]):
        live = [i for i in range(3) if done[i] < lens[i]]
        take = [min(portion[i], lens[i] - done[i]) for i in live]
        parts = [np.concatenate([data[i][j][done[i]:done[i] + n] for i, n in zip(live, take)]) for j in range(3)]
        cu = np.concatenate([[0], np.cumsum(take)])
        y = torch.full((int(cu[-1]), H * dv), float("nan"), device=DEV)
        getattr(KS, form)(dev(parts[0]), 0, G * dk, 2 * G * dk, dev(parts[1]), b_off, dev(parts[2]), a_off, dev(dt_bias), dev(a_log),
                      state, y, H, G, dk, dv, unit_eps, q_scale, i32(cu), i32([slots[i] for i in live]))
        ref = np.concatenate([want[i][0][done[i]:done[i] + n] for i, n in zip(live, take)])
        assert rel(y, ref) < 3e-5, portion
        for i, n in zip(live, take):
            done[i] += n
    assert done == lens
    for i, sl in enumerate(slots):                                           # [H, dk, dv] of the plain function, kept as [H, dv, dk]
        assert rel(state[sl].transpose(1, 2), want[i][1]) < 3e-5
    assert float(area[1].min()) == 3.0 and float(area[:, :11].min()) == 3.0


def test_sigmoid_gate_behind_the_norm_of_the_heads():
    from turboquant_cpp_b200.kernels import ssm as KS
    rng = np.random.default_rng(8)
    T, H, dv, eps = 21, 3, 20, 1e-4
    y, z, w = (host(dev(a)) for a in (rng.standard_normal((T, H * dv)), rng.standard_normal((T, H * dv)) * 2, 1 + 0.2 * rng.standard_normal(dv)))
    want = (P.unit_rms(y.reshape(T, H, dv), eps) * w).reshape(T, H * dv) * P.sigmoid(z)
    out = torch.empty((T, H * dv), device=DEV)
    KS.gated_group_norm(dev(y), dev(z), 0, dev(np.tile(w, H)), H, eps, out, gate_after=True, sigmoid_gate=True)
    assert rel(out, want) < 1e-5
