"""Parts of the Tasadra decoder that need no GPU: the configuration reader, the model's plan of tensors, cache and
state needs, the frequencies of the stretched rotation, and the plain implementation's own consistency."""
import copy

import numpy as np
import pytest

from plain import tasadra_plain as P
from tasadra_util import CONFIGS, DECAY_RANK, GATE_RANK, make_weights, tensor_shapes, write_folder


def test_the_models_plan_names_every_tensor_with_its_shape():
    import turboquant_cpp_b200 as tq
    for name, cfg in CONFIGS.items():
        model = tq.build_model(cfg, "bfloat16")
        plan = {s.name: tuple(s.shape) for s in model.weight_specs()}
        want = tensor_shapes(cfg, decay_rank=-1, gate_rank=-1)           # the low-rank pairs' inner sizes come from the file
        assert plan == want, name
        given = copy.deepcopy(cfg)
        for l in given["layers"]:
            if l["type"] == "channel_delta":
                l["mixer"].update(decay_rank=DECAY_RANK, gate_rank=GATE_RANK)
        plan = {s.name: tuple(s.shape) for s in tq.build_model(given, "bfloat16").weight_specs()}
        assert plan == tensor_shapes(cfg), name


def test_cache_and_state_needs_follow_the_layers():
    import turboquant_cpp_b200 as tq
    model = tq.build_model(CONFIGS["a"], "float32")
    needs, states = model.cache_needs(), model.state_needs()
    # attention: a row of key and value per key/value head; differential attention: two key heads a key/value head,
    # each with the value; the layer that others read keeps rows for the widest cells among its readers; readers and
    # the recurrence keep no pages
    assert [(n.window, n.planes, n.n_kv_heads, n.head_dim) if n else None for n in needs] == \
        [(0, 1, 2, 24), None, (25, 1, 4, 24), None, None]
    assert [e.cache_of for e in model.schedule] == [None, None, None, 2, None]
    W = 48        # every layer keeps the norm's last row for the shift; the recurrence its taps and its state behind it
    assert [s.shape for s in states] == [(W,), (W + 2 * (2 * 2 * 8 + 4 * 12) + 4 * 12 * 8,), (W,), (W,), (W + 1 * (2 * 2 * 16 + 2 * 8) + 2 * 8 * 16,)]
    assert model.capturable()
    assert tq.build_model(CONFIGS["c"], "float32").cache_needs()[2].window == 0


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].__setitem__("type", "parallel"), "type"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 9), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 18), "dims"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("vdim", 7), "vdim"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("conv", 9), "conv"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("dim", 300), "dim"),
    (lambda c: c["layers"][2]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("vdim", 8), "kv_from"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "kind"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_configuration_that_cannot_run_is_refused_with_the_key(change, word):
    import turboquant_cpp_b200 as tq
    cfg = copy.deepcopy(CONFIGS["a"])
    change(cfg)
    with pytest.raises(tq.ConfigError) as e:
        tq.build_model(cfg, "float32")
    assert word in str(e.value)


def test_stretched_frequencies_of_the_part_are_the_plain_ones():
    from turboquant_cpp_b200.parts import make_position_encoding
    for dims, base, sc in ((8, 10000.0, (4.0, 64, 8.0, 1.0)), (32, 5e5, (8.0, 32, 16.0, 2.0)), (12, 50.0, None), (64, 250.0, (2.0, 4096, 32.0, 1.0))):
        scaling = dict(zip(("factor", "original", "fast", "slow"), sc)) if sc else None
        f, mag = P.scaled_frequencies(dims, base, scaling)
        pe = make_position_encoding("rotary_scaled", dims=dims, base=base, pairing="halves", **(scaling or {}))
        assert pe.halves and abs(pe.mag - mag) < 1e-12
        assert np.abs(pe._freq64.numpy() - f).max() < 1e-15


def test_plain_decoding_by_recomputation_is_causal(tmp_path):
    """The plain model has no cache: the logits of a prefix are the first rows of the logits of the whole."""
    cfg = CONFIGS["a"]
    folder = write_folder(str(tmp_path / "m"), cfg, make_weights(cfg, 1))
    m = P.PlainTasadra(folder)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 40).tolist()
    assert np.abs(m.forward(toks)[:25] - m.forward(toks[:25])).max() < 1e-9


def test_the_delta_rule_of_the_plain_model_continues_from_a_state():
    rng = np.random.default_rng(2)
    T, dk, dv = 30, 6, 5
    q, k, v = rng.standard_normal((T, dk)), rng.standard_normal((T, dk)), rng.standard_normal((T, dv))
    beta, decay = rng.random(T), rng.random((T, dk))
    whole, S = P.delta_rule(q, k, v, beta, decay)
    first, S1 = P.delta_rule(q[:11], k[:11], v[:11], beta[:11], decay[:11])
    rest, S2 = P.delta_rule(q[11:], k[11:], v[11:], beta[11:], decay[11:], S=S1)
    assert np.abs(np.concatenate([first, rest]) - whole).max() < 1e-12 and np.abs(S2 - S).max() < 1e-12
