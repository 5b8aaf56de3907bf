"""Helpers of the Tasadra tests: small configurations and model folders with weights made for the test."""
import numpy as np

from nuforax_util import assert_close, run_steps, spread_error, write_folder      # noqa: F401  (file writing, schedules)


def rotation(dims, base=10000.0, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def attention(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.5, softcap=6.0, rot=rotation(8, 10000.0, (4.0, 64, 8.0, 1.0))):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        m["softcap"] = softcap
    if rot:
        m["rot"] = rot
    return m


def delta(heads=4, kv_heads=2, dim=8, vdim=12, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def differential(heads=4, kv_heads=2, dim=8, vdim=16, scale=0.4, diff=0.25, size=10, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if size:
        m["mask"] = {"size": size}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, vocab=97, width=48, eps=3e-5, mult=0.8):
    return {"architecture": "Tasadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "layers": layers}


# Configurations that differ in every size, in the order and kinds of layers, and in the options.
CONFIGS = {
    # grouped heads, a partial rotation with stretched frequencies, a reader of another layer's rows with WIDER cells
    # than its source, a layer without feed-forward, cells narrower than a page
    "a": config([layer("attention", attention(), ff=40),
                 layer("channel_delta", delta()),
                 layer("attention_2", differential(), ff=56),
                 layer("attention_2", differential(size=25, diff=0.1, scale=0.7, kv_from=2), ff=24),
                 layer("channel_delta", delta(heads=2, kv_heads=2, dim=16, vdim=8, conv=2), ff=32)]),
    # sizes the tensor-core kernels take (32 / 64 / 128), differential attention first, cells around one and two
    # pages, a residual factor of one, several query heads a key/value head and one
    "b": config([layer("attention_2", differential(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.2, diff=0.4, size=70), ff=72),
                 layer("attention", attention(heads=4, kv_heads=1, dim=64, vdim=128, scale=0.15, softcap=0, rot=rotation(32, 1000.0)), ff=48),
                 layer("channel_delta", delta(heads=2, kv_heads=1, dim=64, vdim=40, conv=4), ff=40),
                 layer("attention_2", differential(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.3, diff=0.2, size=130, kv_from=0)),
                 layer("attention", attention(heads=2, kv_heads=2, dim=32, vdim=32, scale=0.25, softcap=9.0,
                                              rot=rotation(32, 5e5, (8.0, 32, 16.0, 2.0))), ff=56)],
                vocab=61, width=64, eps=1e-6, mult=1.0),
    # the recurrence first with one tap, odd sizes, one head, no cells, keys of more than 128 elements, eight taps
    "c": config([layer("channel_delta", delta(heads=3, kv_heads=3, dim=20, vdim=7, conv=1), ff=24),
                 layer("attention", attention(heads=1, kv_heads=1, dim=40, vdim=12, scale=0.3, softcap=3.0, rot=rotation(6, 300.0))),
                 layer("attention_2", differential(heads=3, kv_heads=3, dim=12, vdim=6, scale=0.5, diff=0.5, size=0), ff=16),
                 layer("channel_delta", delta(heads=1, kv_heads=1, dim=130, vdim=20, conv=8), ff=28)],
                vocab=128, width=40, mult=0.35),
}

DECAY_RANK, GATE_RANK = 5, 6


def tensor_shapes(cfg, decay_rank=DECAY_RANK, gate_rank=GATE_RANK):
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "head": (V, W)}

    def norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = (W,), (W,), ()

    norm("final.norm")
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        norm(p + "norm1")
        out[p + "shift"], out[p + "dwa"] = (W,), (i + 2,)
        q = p + "mix."
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if l["type"] == "attention":
            out[q + "q"], out[q + "k"], out[q + "v"] = (H * dk, W), (G * dk, W), (G * dv, W)
            out[q + "q.norm"], out[q + "k.norm"] = (dk,), (dk,)
            out[q + "g"], out[q + "o"] = (H, W), (W, H * dv)
        elif l["type"] == "channel_delta":
            out[q + "q"], out[q + "k"], out[q + "v"] = (G * dk, W), (G * dk, W), (H * dv, W)
            out[q + "q.conv"], out[q + "k.conv"], out[q + "v.conv"] = (G * dk, m["conv"]), (G * dk, m["conv"]), (H * dv, m["conv"])
            out[q + "b"], out[q + "A_log"], out[q + "norm"] = (H, W), (H,), (dv,)
            out[q + "a1"], out[q + "a2"], out[q + "dt_bias"] = (decay_rank, W), (H * dk, decay_rank), (H * dk,)
            out[q + "g1"], out[q + "g2"], out[q + "o"] = (gate_rank, W), (H * dv, gate_rank), (W, H * dv)
        else:
            out[q + "q"] = (H * 2 * dk, W)
            if m.get("kv_from") is None:
                out[q + "k"], out[q + "v"] = (G * 2 * dk, W), (G * dv, W)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[q + n] = (dk,)
            out[q + "g"], out[q + "o"] = (H * dv, W), (W, H * dv)
        if l["mlp"] is not None:
            norm(p + "norm2")
            ff = l["mlp"]["ff"]
            out[p + "mlp.up"], out[p + "mlp.up.b"], out[p + "mlp.down"], out[p + "mlp.down.b"] = (ff, W), (ff,), (W, ff), (W,)
    return out


def make_weights(cfg, seed, sharp=1.0, **ranks):
    """Random weights with magnitudes that keep every mechanism visible: projections of unit gain, norm weights
    around 1 with biases and slopes of order 1, shifts between 0 and 1, depth weights of both signs, decays from
    fast to slow.  `sharp` scales the query projections (peaked attention)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, **ranks).items():
        leaf = name.split(".")[-1]
        parent = name.rsplit(".", 1)[0].split(".")[-1] if "." in name else ""
        if leaf == "alpha":
            w = np.asarray(0.4 + 0.6 * rng.random())
        elif leaf == "b" and parent in ("norm1", "norm2", "norm", "up", "down"):
            w = 0.3 * rng.standard_normal(shape)
        elif leaf in ("norm1", "norm2", "norm") or name == "final.norm":
            w = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf == "shift":
            w = rng.random(shape)
        elif leaf == "dwa":
            w = rng.standard_normal(shape) * 0.3 + 1.0 / shape[0]
            w[-1] += 0.7
        elif leaf in ("A_log", "dt_bias"):
            w = rng.standard_normal(shape)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            w = rng.standard_normal(shape) * 0.3
        elif leaf == "conv":
            w = rng.standard_normal(shape) * 0.6
        elif name == "embed":
            w = rng.standard_normal(shape)
        else:
            w = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if leaf == "q":
                w = w * sharp
            if leaf in ("a2", "g2", "b", "g"):
                w = w * 2.0
        out[name] = np.asarray(w, dtype=np.float32)
    return out
