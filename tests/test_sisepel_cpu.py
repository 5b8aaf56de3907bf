"""Parts of the Sisepel decoder that need no GPU: the configuration reader, the model's plan of tensors, cache and
state needs, the frequencies of the stretched rotation, and the plain implementation's own consistency."""
import copy
import math

import numpy as np
import pytest

from plain import sisepel_plain as P
from sisepel_util import CONFIGS, make_weights, tensor_shapes, write_folder


def test_the_models_plan_names_every_tensor_with_its_shape():
    import turboquant_cpp_b200 as tq
    for name, cfg in CONFIGS.items():
        model = tq.build_model(cfg, "bfloat16")
        assert {s.name: tuple(s.shape) for s in model.weight_specs()} == tensor_shapes(cfg), name


def test_every_layer_keeps_a_window_of_keys_and_a_state():
    import turboquant_cpp_b200 as tq
    model = tq.build_model(CONFIGS["a"], "float32")
    needs, states = model.cache_needs(), model.state_needs()
    # a position's row is a key and a value per key/value head, one plane; the state is heads x dim x vdim floats
    assert [(n.window, n.planes, n.n_kv_heads, n.head_dim) for n in needs] == [(24, 1, 2, 24), (9, 1, 2, 16), (70, 1, 2, 64)]
    assert [s.shape for s in states] == [(3 * 8 * 12,), (2 * 16 * 4,), (1 * 4 * 20,)]
    assert tq.build_model(CONFIGS["c"], "float32").cache_needs()[0].window == 0
    assert model.capturable()


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].__setitem__("type", "attention"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 9), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 18), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5, 0.6]), "decay"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].__setitem__("high", 0.5), "high"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda c: c["layers"][2]["mixer"]["left"].__setitem__("vdim", 300), "vdim"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_configuration_that_cannot_run_is_refused_with_the_key(change, word):
    import turboquant_cpp_b200 as tq
    cfg = copy.deepcopy(CONFIGS["a"])
    change(cfg)
    with pytest.raises(tq.ConfigError) as e:
        tq.build_model(cfg, "float32")
    assert word in str(e.value)


def test_plain_decoding_by_recomputation_is_causal(tmp_path):
    """The plain model has no cache: the logits of a prefix are the first rows of the logits of the whole."""
    cfg = CONFIGS["a"]
    folder = write_folder(str(tmp_path / "m"), cfg, make_weights(cfg, 1))
    m = P.PlainSisepel(folder)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 40).tolist()
    assert np.abs(m.forward(toks)[:25] - m.forward(toks[:25])).max() < 1e-9


def test_stretched_frequencies_keep_short_waves_and_slow_down_long_ones():
    from turboquant_cpp_b200.parts import make_position_encoding
    rot = {"dims": 32, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128}}
    f0, f1 = P.frequencies({"dims": 32, "base": 10000.0}), P.frequencies(rot)
    wave = 2.0 * math.pi / f0
    assert np.all(f1[wave < 32] == f0[wave < 32]) and np.allclose(f1[wave > 128], f0[wave > 128] / 8.0, rtol=1e-15)
    between = (wave >= 32) & (wave <= 128)
    assert between.any() and np.all(f1[between] <= f0[between]) and np.all(f1[between] >= f0[between] / 8.0)
    pe = make_position_encoding("rotary_bands", dims=32, base=10000.0, pairing="halves", factor=8.0, low=1.0, high=4.0, original=128)
    assert np.allclose(pe._freq64.numpy(), f1, rtol=1e-14) and pe.halves
    plain = make_position_encoding("rotary_bands", dims=6, base=50.0)
    assert np.allclose(plain._freq64.numpy(), [1.0, 50.0 ** (-1 / 3), 50.0 ** (-2 / 3)], rtol=1e-14) and not plain.halves


def test_the_two_pairings_turn_the_pairs_the_plain_model_says():
    v = np.arange(1.0, 9.0).reshape(1, 8)
    rot = {"dims": 4, "base": 1.0}                 # every pair turns by the position itself
    c, s = math.cos(2.0), math.sin(2.0)
    n = P.rotate(v, 2, rot, "neighbours")[0]
    assert np.allclose(n, [1 * c - 2 * s, 2 * c + 1 * s, 3 * c - 4 * s, 4 * c + 3 * s, 5, 6, 7, 8])
    h = P.rotate(v, 2, rot, "halves")[0]
    assert np.allclose(h, [1 * c - 3 * s, 2 * c - 4 * s, 3 * c + 1 * s, 4 * c + 2 * s, 5, 6, 7, 8])
