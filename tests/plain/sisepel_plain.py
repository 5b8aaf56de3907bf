"""A plain, slow implementation of the Sisepel decoder, one function per mechanism, in float64 on the CPU.

It reads a model folder (config.json, model.safetensors) with its own few lines of file parsing and shares no code
with the library.  Every function takes a whole sequence and loops over positions where the definition does; nothing
is cached, so the logits of a position are those of the definition itself.

Notation: h is a sub-layer's input [T, width]; unit(v) = v / sqrt(mean(v^2) + eps); positions start at 0; a layer is

    x += norm1b(mixer(norm1(x)));  x += norm2b(ffn(norm2(x)))  (if it has a feed-forward);  x += side(x, tokens)

and the mixer is the mean of two branches that read the same input: windowed softmax attention and retention.
"""
import json
import math
import os
import struct

import numpy as np

F = np.float64
GELU_CUBIC = 0.044715


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


# ---- small functions --------------------------------------------------------------------------------------------
def unit(v, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def norm(v, w, eps):
    return unit(v, eps) * w


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def silu(v):
    return v * sigmoid(v)


def gelu_tanh(v):
    return 0.5 * v * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (v + GELU_CUBIC * v ** 3)))


# ---- rotation ---------------------------------------------------------------------------------------------------
def frequencies(rot):
    """f_i = base^(-2i/dims); with `scaling`, long waves are slowed by `factor`, short ones kept, and the band
    between the two wavelengths original/low and original/high is a straight blend of both."""
    dims = rot["dims"]
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        if sc is not None:
            wave = 2.0 * math.pi / f
            if wave > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wave >= sc["original"] / sc["high"]:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return np.array(out, dtype=F)


def rotate(v, pos, rot, pairing):
    """v [heads, dim] at position pos: the first rot['dims'] elements of each head are turned pair by pair;
    pairing 'neighbours': (2i, 2i+1); 'halves': (i, i + dims/2)."""
    if rot is None or rot["dims"] == 0:
        return v
    dims = rot["dims"]
    f = frequencies(rot)
    out = v.copy()
    for i in range(dims // 2):
        a, b = (2 * i, 2 * i + 1) if pairing == "neighbours" else (i, i + dims // 2)
        c, s = math.cos(pos * f[i]), math.sin(pos * f[i])
        out[:, a] = v[:, a] * c - v[:, b] * s
        out[:, b] = v[:, b] * c + v[:, a] * s
    return out


# ---- the softmax branch ------------------------------------------------------------------------------------------
def attention_core(q, k, v, m, sink, eps):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] as projected, positions 0 .. T-1.  Queries and keys are rotated
    (neighbouring pairs), then made unit length per head; scores are scaled, capped by cap * tanh(score / cap), masked
    to the last `size` positions, and the softmax's denominator also holds exp(sink) (sink [H], or None)."""
    T, H, dk = q.shape
    G, dv = k.shape[1], v.shape[2]
    rot = m.get("rot")
    q, k = q.copy(), k.copy()
    for t in range(T):
        q[t] = unit(rotate(q[t], t, rot, "neighbours"), eps)
        k[t] = unit(rotate(k[t], t, rot, "neighbours"), eps)
    size = m["mask"]["size"] if m.get("mask") else 0
    cap = m.get("softcap", 0.0)
    out = np.zeros((T, H, dv), dtype=F)
    for a in range(H):
        g = a // (H // G)
        for i in range(T):
            lo = max(0, i - size + 1) if size else 0
            s = (k[lo:i + 1, g] @ q[i, a]) * m["scale"]
            if cap:
                s = cap * np.tanh(s / cap)
            top = s.max() if sink is None else max(s.max(), sink[a])
            e = np.exp(s - top)
            den = e.sum() + (0.0 if sink is None else math.exp(sink[a] - top))
            out[i, a] = (e / den) @ v[lo:i + 1, g]
    return out


def window_attention(h, m, w, p, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = (h @ w[p + "q"].T).reshape(T, H, dk)
    k = (h @ w[p + "k"].T).reshape(T, G, dk)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    return attention_core(q, k, v, m, w.get(p + "sink"), eps).reshape(T, H * dv) @ w[p + "o"].T


# ---- the retention branch ----------------------------------------------------------------------------------------
def retention_core(q, k, v, m, S=None, start=0):
    """q, k [T, H, dk], v [T, H, dv] as projected, at positions start .. start+T-1.  Per head: S <- decay * S + k v^T,
    o = S^T q, with q and k rotated (halves) and k scaled by dk^(-1/2).  Returns (o [T, H, dv], S [H, dk, dv])."""
    T, H, dk = q.shape
    dv = v.shape[2]
    rot = m.get("rot")
    S = np.zeros((H, dk, dv), dtype=F) if S is None else S.copy()
    o = np.zeros((T, H, dv), dtype=F)
    for t in range(T):
        qt = rotate(q[t], start + t, rot, "halves")
        kt = rotate(k[t], start + t, rot, "halves") * dk ** -0.5
        for a in range(H):
            S[a] = m["decay"][a] * S[a] + np.outer(kt[a], v[t, a])
            o[t, a] = S[a].T @ qt[a]
    return o, S


def retention(h, m, w, p, eps):
    """The recurrence's output is made unit length per head, gated by silu(W_g h) and projected."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m.get("vdim", m["dim"])
    q = (h @ w[p + "q"].T).reshape(T, H, dk)
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    o, _ = retention_core(q, k, v, m)
    o = unit(o, eps).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h, m, w, p, eps):
    left = window_attention(h, m["left"], w, p + "left.", eps)
    right = retention(h, m["right"], w, p + "right.", eps)
    return 0.5 * (norm(left, w[p + "left.out"], eps) + norm(right, w[p + "right.out"], eps))


# ---- feed-forwards -----------------------------------------------------------------------------------------------
def gated(h, w, p, act):
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, ml, w, p):
    """Logits with a bias; the `top` largest (the lower index wins a tie); weights = softmax over the chosen.
    Also each row's margin: how far the last chosen expert lies above the best one left out, as probabilities of a
    softmax over all experts (0 if every expert is chosen)."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    top = ml["router"]["top"]
    order = np.argsort(-z, axis=-1, kind="stable")
    ids = order[:, :top]
    prob = np.exp(z - z.max(axis=-1, keepdims=True))
    prob /= prob.sum(axis=-1, keepdims=True)
    ranked = np.take_along_axis(prob, order, axis=-1)
    margins = ranked[:, top - 1] - ranked[:, top] if top < z.shape[1] else np.ones(z.shape[0])
    return ids, chosen_weights(z, ids), margins


def chosen_weights(z, ids):
    zs = np.take_along_axis(z, ids, axis=-1)
    e = np.exp(zs - zs.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def experts(h, ml, w, p, ids=None, record=None):
    """ids: another choice of experts than the router's own (a test hands it in where two logits nearly tie); the
    weights are then the softmax over those experts' logits.  record: a list that receives (ids, weights, margins)."""
    own_ids, wts, margins = route(h, ml, w, p)
    if record is not None:
        record.append((own_ids, wts, margins))
    if ids is not None:
        wts = chosen_weights(h @ w[p + "router"].T + w[p + "router.b"], ids)
    else:
        ids = own_ids
    y = np.zeros_like(h)
    for t in range(h.shape[0]):
        for j, e in enumerate(ids[t]):
            y[t] += wts[t, j] * gated(h[t:t + 1], w, f"{p}e{int(e)}.", silu)[0]
    if ml.get("shared"):
        y += gated(h, w, p + "shared.", silu)
    return y


def feed_forward(h, ml, w, p, ids=None, record=None):
    if ml.get("kind", "dense") == "dense":
        return gated(h, w, p + "mlp.", gelu_tanh)
    return experts(h, ml, w, p + "mlp.", ids, record)


# ---- per-layer token input ----------------------------------------------------------------------------------------
def token_side(x, tokens, i, dim, w, p, eps):
    e = w["side.embed"][tokens, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ w[p + "gate"].T) * e
    return norm(g @ w[p + "proj"].T, w[p + "norm"], eps)


# ---- the model -----------------------------------------------------------------------------------------------------
class PlainSisepel:
    def __init__(self, folder):
        with open(os.path.join(folder, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = read_safetensors(os.path.join(folder, "model.safetensors"))

    def forward(self, tokens, routing=None, forced=None, streams=None):
        """Logits [T, vocab] of one sequence.  routing: a list that receives (ids, weights, margins) of every routed
        layer in order; forced: expert choices [T, top] for the first routed layers, taken instead of the router's
        own; streams: a list that receives the residual stream after every layer."""
        cfg, w = self.cfg, self.w
        eps = cfg["norm"]["eps"]
        tokens = np.asarray(tokens, dtype=np.int64)
        x = w["embed"][tokens].astype(F)
        side = cfg.get("token_side")
        routed = 0
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{i}."
            if layer["type"] != "parallel":
                raise ValueError(f"layer type {layer['type']}")
            y = parallel_mixer(norm(x, w[p + "norm1"], eps), layer["mixer"], w, p + "mix.", eps)
            x = x + norm(y, w[p + "norm1b"], eps)
            ml = layer.get("mlp")
            if ml is not None:
                ids = None
                if ml.get("kind", "dense") == "moe":
                    if forced is not None and routed < len(forced):
                        ids = np.asarray(forced[routed])
                    routed += 1
                y = feed_forward(norm(x, w[p + "norm2"], eps), ml, w, p, ids, routing)
                x = x + norm(y, w[p + "norm2b"], eps)
            if side:
                x = x + token_side(x, tokens, i, side["dim"], w, p + "side.", eps)
            if streams is not None:
                streams.append(x.copy())
        return norm(x, w["final.norm"], eps) @ w["head"].T * cfg.get("logit_scale", 1.0)
