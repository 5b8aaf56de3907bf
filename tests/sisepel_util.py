"""Helpers of the Sisepel tests: small configurations, model folders with weights made for the test, and the
comparison with the plain model, which takes the engine's expert choices where its own were a near-tie."""
import numpy as np

from lumevik_util import check_against_plain, run_steps_with_routing      # noqa: F401  (the comparison that follows expert choices)
from nuforax_util import assert_close, run_steps, spread_error, write_folder      # noqa: F401  (file writing, schedules)


def rotation(dims, base=10000.0, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def left(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.5, size=24, softcap=6.0, rot=rotation(8, 10000.0, (4.0, 1.0, 3.0, 64))):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:                  # size 0: no mask, every earlier position is seen
        m["mask"] = {"size": size}
    if softcap:
        m["softcap"] = softcap
    if rot:
        m["rot"] = rot
    return m


def right(heads=3, dim=8, vdim=12, decay=(0.9, 0.97, 0.999), rot=rotation(8, 500.0)):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = rot
    return m


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=8, top=3, ff=16, shared=24):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(l, r, mlp=None):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}


def config(layers, vocab=97, width=48, eps=3e-5, side=6, logit_scale=0.7):
    cfg = {"architecture": "Sisepel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


# Configurations that differ in every size, in the feed-forwards' order and kinds, and in the options.
CONFIGS = {
    # grouped heads, partial rotations with and without stretched frequencies, routed experts, a dense layer, a
    # layer without feed-forward, a window wider than a page
    "a": config([layer(left(), right(), moe()),
                 layer(left(heads=6, kv_heads=2, dim=8, vdim=8, scale=1.2, size=9, softcap=4.0, rot=rotation(4, 100.0)),
                       right(heads=2, dim=16, vdim=4, decay=(0.5, 1.0), rot=rotation(6, 10000.0)), dense()),
                 layer(left(heads=2, kv_heads=2, dim=24, vdim=40, scale=0.4, size=70, softcap=0, rot=rotation(24, 30000.0, (6.0, 1.0, 5.0, 96))),
                       right(heads=1, dim=4, vdim=20, decay=(0.98,), rot=rotation(4, 10.0)), None)]),
    # sizes the tensor-core kernels take (32 / 64 / 128), one key/value head, windows around two pages, no token
    # input, unscaled logits, one expert chosen, no shared expert
    "b": config([layer(left(heads=4, kv_heads=1, dim=32, vdim=64, scale=0.3, size=130, softcap=8.0, rot=rotation(32, 1000.0)),
                       right(heads=2, dim=64, vdim=40, decay=(0.99, 0.9), rot=rotation(64, 2e5)), moe(experts=6, top=1, ff=24, shared=0)),
                 layer(left(heads=2, kv_heads=2, dim=64, vdim=32, scale=0.15, size=64, softcap=0, rot=rotation(16, 5000.0, (2.0, 0.5, 2.0, 40))),
                       right(heads=4, dim=32, vdim=32, decay=(0.999, 0.95, 0.8, 0.99), rot=rotation(32, 1e4)), dense(ff=56)),
                 layer(left(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.08, size=65, softcap=25.0, rot=rotation(64, 1e5)),
                       right(heads=1, dim=40, vdim=72, decay=(0.97,), rot=None), moe(experts=4, top=2, ff=8, shared=8))],
                vocab=61, width=40, eps=1e-6, side=0, logit_scale=None),
    # no window at all, every query head its own key/value head, no rotation on the left, all experts chosen
    "c": config([layer(left(heads=3, kv_heads=3, dim=16, vdim=16, scale=0.6, size=0, softcap=3.0, rot=None),
                       right(heads=2, dim=12, vdim=6, decay=(1.0, 0.93), rot=rotation(2, 7.0)), moe(experts=3, top=3, ff=12, shared=16)),
                 layer(left(heads=1, kv_heads=1, dim=40, vdim=12, scale=0.3, size=1, softcap=0, rot=rotation(40, 300.0)),
                       right(heads=5, dim=6, vdim=6, decay=(0.9, 0.91, 0.92, 0.93, 0.94), rot=rotation(6, 50.0)), dense(ff=9))],
                vocab=128, width=64, side=10, logit_scale=2.5),
}


def tensor_shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    side = cfg.get("token_side")
    if side:
        out["side.embed"] = (V, side["dim"] * len(cfg["layers"]))
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        a, r = l["mixer"]["left"], l["mixer"]["right"]
        out[p + "norm1"], out[p + "norm1b"] = (W,), (W,)
        q = p + "mix.left."
        out[q + "q"], out[q + "k"] = (a["heads"] * a["dim"], W), (a["kv_heads"] * a["dim"], W)
        out[q + "v"], out[q + "o"] = (a["kv_heads"] * a["vdim"], W), (W, a["heads"] * a["vdim"])
        out[q + "sink"] = (a["heads"],)
        q = p + "mix.right."
        for n in ("q", "k"):
            out[q + n] = (r["heads"] * r["dim"], W)
        for n in ("v", "g"):
            out[q + n] = (r["heads"] * r["vdim"], W)
        out[q + "o"] = (W, r["heads"] * r["vdim"])
        out[p + "mix.left.out"], out[p + "mix.right.out"] = (W,), (W,)
        mlp = l["mlp"]
        if mlp is not None:
            out[p + "norm2"], out[p + "norm2b"] = (W,), (W,)
            q = p + "mlp."
            if mlp["kind"] == "dense":
                out[q + "gate"], out[q + "up"], out[q + "down"] = (mlp["ff"], W), (mlp["ff"], W), (W, mlp["ff"])
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                for e in range(E):
                    out[f"{q}e{e}.gate"], out[f"{q}e{e}.up"], out[f"{q}e{e}.down"] = (ff, W), (ff, W), (W, ff)
                out[q + "router"], out[q + "router.b"] = (E, W), (E,)
                if mlp.get("shared"):
                    s = mlp["shared"]["ff"]
                    out[q + "shared.gate"], out[q + "shared.up"], out[q + "shared.down"] = (s, W), (s, W), (W, s)
        if side:
            out[p + "side.gate"], out[p + "side.proj"], out[p + "side.norm"] = (side["dim"], W), (W, side["dim"]), (W,)
    return out


def make_weights(cfg, seed):
    """Random weights with magnitudes that keep every mechanism visible: projections of unit gain, norms around 1,
    sinks and router biases of order 1, routers spread enough for clear margins.  (Queries and keys are made unit
    length by the model, so how peaked the softmax is lies with the configurations' scale and cap.)"""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm1b", "norm2", "norm2b", "norm", "out") or name == "final.norm":
            w = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf in ("sink", "b"):
            w = rng.standard_normal(shape)
        elif name in ("embed", "side.embed"):
            w = rng.standard_normal(shape)
        else:
            w = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if leaf in ("gate", "up", "router"):
                w = w * 2.0
        out[name] = np.asarray(w, dtype=np.float32)
    return out
