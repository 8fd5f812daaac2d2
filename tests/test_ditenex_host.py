"""Ditenex without a GPU: its configuration, what its layers ask of the cache, the tensors it declares, and the plain
implementation's own mechanisms against cases worked by hand."""
import copy

import numpy as np
import pytest

from friday_inference_engine_b200 import ConfigError, describe_model, read_config

import ditenex_models as dm
import plain_ditenex as plain

CFG = dm.CONFIGS["P"]


def test_the_name_selects_the_design():
    assert read_config(CFG)["architecture"] == "Ditenex"
    d = describe_model(CFG)
    assert d["architecture"] == "Ditenex" and d["n_layers"] == 4 and d["max_positions"] == 1024
    assert [c["layer"] for c in d["program"]] == [0, 1, 2, 3] and not any(c["add_input"] for c in d["program"])


def test_cache_requests():
    reqs = describe_model(CFG)["cache_requests"]
    # keys and values behind the layer's own window, values of a size of their own; and the shift's row, 32-bit
    assert reqs["0"] == {"kind": "several", "parts": [
        {"kind": "kv", "n_kv_heads": 2, "head_dim": 16, "window": 20, "v_head_dim": 24, "keep_first": 0},
        {"kind": "state", "shape": [96], "dtype": "float32"}]}
    assert reqs["3"]["parts"][0] == {"kind": "kv", "n_kv_heads": 1, "head_dim": 32, "window": 130, "v_head_dim": 24, "keep_first": 0}
    assert all(reqs[str(i)]["parts"][1] == {"kind": "state", "shape": [96], "dtype": "float32"} for i in range(4))


def test_declared_tensors():
    d = describe_model(CFG)
    shapes = {p["name"]: p["shape"] for p in d["params"]}
    assert shapes["embed"] == [300, 96] and shapes["pos"] == [1024, 96] and "head" not in shapes
    assert shapes["final.norm"] == [96] and shapes["l0.shift"] == [96] and shapes["l0.norm1b"] == [96] and shapes["l0.norm2b"] == [96]
    assert shapes["l0.mix.q"] == [64, 96] and shapes["l0.mix.q.b"] == [64] and shapes["l0.mix.v"] == [48, 96]
    assert shapes["l0.mix.g"] == [96, 96] and shapes["l0.mix.o"] == [96, 96] and shapes["l0.mix.talk"] == [4, 4]
    assert shapes["l0.mlp.up"] == [40, 96] and shapes["l0.mlp.act"] == [2]
    assert shapes["l1.mlp.router"] == [6, 96] and shapes["l1.mlp.correction"] == [6] and shapes["l1.mlp.e5.down"] == [96, 24]
    assert shapes["l1.mlp.shared.gate"] == [40, 96] and "l1.mlp.router.b" not in shapes
    # the first blending layer's weight is not used, a layer that does not blend has none; no feed-forward, no second norms
    assert "l0.mix.vmix" not in shapes and "l1.mix.vmix" not in shapes and shapes["l2.mix.vmix"] == []
    assert {"l0.mix.vmix", "l1.mix.vmix", "l2.norm2", "l2.norm2b"} <= set(d["ignorable"]) and "l2.mlp.up" not in shapes


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="retention"), "retention"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "share"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "gated"),
    (lambda c: c["layers"][1]["mlp"]["router"].pop("top"), "top"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "v_mix"),
])
def test_bad_config_names_the_key(change, word):
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        read_config(cfg)
    assert word in str(e.value)


# ---- the plain implementation's mechanisms against cases worked by hand
def test_plain_token_shift_and_norm():
    h = np.array([[1.0, 2.0], [3.0, 6.0], [5.0, 0.0]])
    s = np.array([0.5, 1.0])
    # the row before the first is zero; a weight of one replaces a channel by the row before's
    assert np.allclose(plain.token_shift(h, s), [[0.5, 0.0], [2.0, 2.0], [4.0, 6.0]])
    x = np.array([[3.0, 4.0]])
    assert np.allclose(plain.rms(x, np.array([1.0, 2.0]), 0.0), [[3 / np.sqrt(12.5), 8 / np.sqrt(12.5)]])


def test_plain_activation_meets_at_zero_and_slopes():
    z = np.array([-1e-6, 0.0, 1e-6, 2.0, -2.0])
    y = plain.two_sided_activation(z, 0.3, -0.4)
    assert abs(y[1]) == 0.0 and abs(y[0] + 0.5e-6) < 1e-10 and abs(y[2] - 0.5e-6) < 1e-10       # slope 1/2 on both sides
    assert np.isclose(y[3], np.log1p(np.exp(0.3)) * 4.0 + 1.0)
    assert np.isclose(y[4], (0.5 + np.log1p(np.exp(-0.4))) * (np.exp(-2.0) - 1.0 + 2.0) - 1.0)


def test_plain_distance_slopes():
    assert np.allclose(plain.distance_slopes(4), [2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8])
    assert np.allclose(plain.distance_slopes(1), [2.0 ** -8])
