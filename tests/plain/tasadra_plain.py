"""A plain, slow implementation of the Tasadra decoder, one function per mechanism, in float64 on the CPU.

It reads a model folder (config.json, model.safetensors) with its own few lines of file parsing and shares no code
with the library.  Every function takes a whole sequence and loops over positions where the definition does; nothing
is cached, so the logits of a position are those of the definition itself.

Notation: X_0 is the embedding, r the residual multiplier, dyt(v) = tanh(alpha v) * w + b.  Layer i computes

    h = shift(dyt1(x));  y = x + r * mixer(h);  X_(i+1) = y + r * ffn(dyt2(y))  (the second sum only with a feed-forward)
    x <- sum_j dwa_i[j] * X_j  over j = 0 .. i+1

with shift(h)_t = h_t + (h_(t-1) - h_t) * s (h_(-1) = 0).  Three mixers: softmax attention with normed and rotated
queries and keys, rotated values and a gate per head; a delta rule with a decay per key channel; differential
attention inside chunks of positions, which may read an earlier layer's keys and values.
"""
import json
import math
import os
import struct

import numpy as np

F = np.float64
DELTA_UNIT_EPS = 1e-6


# ---- file reading ---------------------------------------------------------------------------------------------
def read_safetensors(path):
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        raw = data[a:b]
        if meta["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(F)
        elif meta["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(F)
        elif meta["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"dtype {meta['dtype']} of '{name}'")
        out[name] = arr.reshape(meta["shape"])
    return out


def load(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# ---- small functions --------------------------------------------------------------------------------------------
def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def silu(v):
    return v * sigmoid(v)


def softplus(v):
    return np.logaddexp(0.0, v)


def unit_rms(v, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def dyt(v, w, name):
    """The norm of this design: no statistics, tanh(alpha v) * weight + bias."""
    return np.tanh(float(w[name + ".alpha"]) * v) * w[name] + w[name + ".b"]


def token_shift(h, s):
    """h_t + (h_(t-1) - h_t) * s with zeros before the first token; the earlier rows enter unshifted."""
    before = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (before - h) * s


def softmax_rows(s, seen):
    s = np.where(seen, s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(axis=-1, keepdims=True)


# ---- rotation ---------------------------------------------------------------------------------------------------
def plain_frequencies(dims, base):
    return np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)


def scaled_frequencies(dims, base, scaling):
    """(frequencies, factor on cos and sin).  Slow pairs are divided by `factor`, fast ones kept, a ramp between."""
    f = plain_frequencies(dims, base)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    where = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    out = f.copy()
    for i in range(dims // 2):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def rotate_halves(v, positions, freq, mag=1.0, sign=1.0):
    """v [T, heads, n]: element i of the first 2 * len(freq) is paired with i + len(freq); position p turns the pair by
    sign * p * freq[i]; cos and sin are multiplied by mag.  The rest of a head passes."""
    half = len(freq)
    out = v.copy()
    ang = sign * positions[:, None, None].astype(F) * freq[None, None, :]
    c, s = np.cos(ang) * mag, np.sin(ang) * mag
    a, b = v[..., :half], v[..., half:2 * half]
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = b * c + a * s
    return out


# ---- mixer: attention ---------------------------------------------------------------------------------------------
def attention_keys_values(h, w, p, m, eps):
    """What the layer caches: normed, rotated keys [T, G, dim] and rotated values [T, G, vdim]."""
    T = h.shape[0]
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    k = (h @ w[p + "k"].T).reshape(T, G, dim)
    k = unit_rms(k, eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).reshape(T, G, vdim)
    rot = m.get("rot")
    if rot and rot["dims"]:
        f, mag = scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        k = rotate_halves(k, pos, f, mag)
    if rot:
        v = rotate_halves(v, pos, plain_frequencies(vdim, rot["base"]))
    return k, v


def attention_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, dim)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    rot = m.get("rot")
    if rot and rot["dims"]:
        f, mag = scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q = rotate_halves(q, pos, f, mag)
    k, v = attention_keys_values(h, w, p, m, eps)
    cap = float(m.get("softcap") or 0.0)
    seen = pos[None, :] <= pos[:, None]
    out = np.zeros((T, H, vdim), dtype=F)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * np.tanh(s / cap)
        out[:, a] = softmax_rows(s, seen) @ v[:, g]
    if rot:
        out = rotate_halves(out, pos, plain_frequencies(vdim, rot["base"]), sign=-1.0)
    gate = sigmoid(h @ w[p + "g"].T)                        # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * vdim) @ w[p + "o"].T


# ---- mixer: delta rule with a decay per key channel -----------------------------------------------------------------
def short_convolution(u, taps_w):
    """u [T, C], taps_w [C, taps]: the last column meets the current token, zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    out = np.zeros_like(u)
    for k in range(taps):
        back = taps - 1 - k
        out[back:] += u[:T - back] * taps_w[:, k] if back else u * taps_w[:, k]
    return out


def delta_rule(q, k, v, beta, decay, S=None):
    """One head: q, k [T, dim] (already unit vectors), v [T, vdim], beta [T], decay [T, dim]; S [dim, vdim] the state
    before the first token (zeros if None).  Returns (outputs [T, vdim], the state after the last token)."""
    T, dim = k.shape
    S = np.zeros((dim, v.shape[1]), dtype=F) if S is None else S.astype(F).copy()
    out = np.zeros((T, v.shape[1]), dtype=F)
    for t in range(T):
        S = decay[t][:, None] * S                     # every key channel's row decays by its own factor
        u = beta[t] * (v[t] - S.T @ k[t])             # what the state lacks of the value, as far as beta allows
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]                           # the read-out sees the token's own write
    return out, S


def delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, dim)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, dim)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, vdim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + DELTA_UNIT_EPS) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + DELTA_UNIT_EPS)
    beta = sigmoid(h @ w[p + "b"].T)                                              # [T, H]
    step = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(T, H, dim)
    decay = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * step)                  # [T, H, dim]
    gate = sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, vdim)
    out = np.zeros((T, H, vdim), dtype=F)
    for a in range(H):
        g = a // (H // G)
        out[:, a], _ = delta_rule(q[:, g], k[:, g], v[:, a], beta[:, a], decay[:, a])
    out = unit_rms(out, eps) * w[p + "norm"] * gate
    return out.reshape(T, H * vdim) @ w[p + "o"].T


# ---- mixer: differential attention inside chunks -------------------------------------------------------------------
def differential_keys_values(h, w, p, m):
    T = h.shape[0]
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    return (h @ w[p + "k"].T).reshape(T, G, 2, dim), (h @ w[p + "v"].T).reshape(T, G, vdim)


def differential_combine(a1, a2, lam, eps, diff):
    """Two maps' outputs of one head [T, vdim]: their difference, divided by its root mean square, times 1 - diff."""
    return unit_rms(a1 - lam * a2, eps) * (1.0 - diff)


def cell_mask(positions_q, positions_k, size):
    """seen[i, j]: key j is not ahead of query i and, with cells of `size` positions counted from position 0, lies in
    the query's own cell."""
    seen = positions_k[None, :] <= positions_q[:, None]
    if size:
        seen = seen & (positions_k[None, :] // size == positions_q[:, None] // size)
    return seen


def differential_mixer(h, w, p, m, eps, kv=None):
    """kv: (keys, values) of the layer this one reads, or None if it has projections of its own."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, 2, dim)
    k, v = kv if kv is not None else differential_keys_values(h, w, p, m)
    seen = cell_mask(pos, pos, m["mask"]["size"] if m.get("mask") else 0)
    diff = float(m["diff"])
    lam = math.exp(float(np.sum(w[p + "lq1"] * w[p + "lk1"]))) - math.exp(float(np.sum(w[p + "lq2"] * w[p + "lk2"]))) + diff
    out = np.zeros((T, H, vdim), dtype=F)
    for a in range(H):
        g = a // (H // G)
        maps = [softmax_rows((q[:, a, i] @ k[:, g, i].T) * m["scale"], seen) @ v[:, g] for i in range(2)]
        out[:, a] = differential_combine(maps[0], maps[1], lam, eps, diff)
    out = out.reshape(T, H * vdim) * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---- feed-forward ---------------------------------------------------------------------------------------------------
def dense_ffn(h, w, p):
    u = np.maximum(h @ w[p + "up"].T + w[p + "up.b"], 0.0)
    return (u * u) @ w[p + "down"].T + w[p + "down.b"]


# ---- the model ------------------------------------------------------------------------------------------------------
def forward(cfg, w, tokens, streams=None):
    """Logits [T, vocab] of one sequence.  streams: a list that receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    r = float(cfg.get("residual_mult", 1.0))
    x = w["embed"][np.asarray(tokens)].astype(F)
    kept = [x]                                     # X_0 .. X_(i+1)
    shared = {}                                    # keys and values of differential layers, for layers that read them
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = token_shift(dyt(x, w, p + "norm1"), w[p + "shift"])
        kind = layer["type"]
        if kind == "attention":
            y = attention_mixer(h, w, p + "mix.", m, eps)
        elif kind == "channel_delta":
            y = delta_mixer(h, w, p + "mix.", m, eps)
        elif kind == "attention_2":
            src = m.get("kv_from")
            if src is None:
                shared[i] = differential_keys_values(h, w, p + "mix.", m)
            y = differential_mixer(h, w, p + "mix.", m, eps, kv=shared[i if src is None else src])
        else:
            raise ValueError(f"layer type '{kind}'")
        x = x + r * y
        if layer.get("mlp") is not None:
            x = x + r * dense_ffn(dyt(x, w, p + "norm2"), w, p + "mlp.")
        kept.append(x)
        x = sum(float(w[p + "dwa"][j]) * kept[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x)
    return dyt(x, w, "final.norm") @ w["head"].T


class PlainTasadra:
    """A model folder and its logits."""

    def __init__(self, folder):
        self.cfg, self.w = load(folder)

    def forward(self, tokens, streams=None):
        return forward(self.cfg, self.w, tokens, streams)
