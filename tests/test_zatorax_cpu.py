"""CPU-side checks of the Zatorax family: config parsing, tensor inventory, the safetensors reader / writer, bfloat16 rounding,
the registry, and hand-made cases that pin how the plain reference (tests/zatorax_ref.py) reads the design's branches."""
import json
import os

import numpy as np
import pytest

from crabml_b200 import models, zatorax
from crabml_b200.capi import TensorError
from tests import zatorax_ref as R
from tests.zatorax_common import attn_layer, config, delta_layer, mixed_config, moe_cfg


def test_parse_config_fills_defaults_and_rejects_unknowns():
    c = zatorax.parse_config(config([delta_layer(), attn_layer(mlp=None)]))
    assert c["layers"][1]["mixer"]["kv_from"] is None and c["layers"][1]["mlp"] is None
    raw = config([delta_layer(mlp={"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 4, "top": 2}})])
    c = zatorax.parse_config(raw)
    assert c["layers"][0]["mlp"]["router"]["groups"] == {"count": 1, "keep": 1} and c["layers"][0]["mlp"]["shared"] is None
    with pytest.raises(TensorError):
        zatorax.parse_config(config([{"type": "conv", "mixer": {}, "mlp": None}]))
    with pytest.raises(TensorError):
        zatorax.parse_config(dict(config([delta_layer()]), architecture="other"))


def test_expected_tensors_follow_the_config():
    c = zatorax.parse_config(mixed_config())
    t = zatorax.expected_tensors(c)
    assert t["l0.mix.q"] == [2 * 16, 48] and t["l0.mix.v.conv"] == [4 * 24, 3] and t["l0.mix.norm"] == [24]
    assert "l2.mix.k" not in t and "l2.mix.k.norm" not in t and t["l2.mix.q"] == [4 * 16, 48]           # the borrower has no key / value tensors
    assert "l3.norm2" not in t and "l3.mlp.router" not in t                                               # no feed-forward
    assert t["l2.mlp.e3.down"] == [48, 24] and "l2.mlp.shared.gate" not in t
    assert t["l0.mlp.shared.up"] == [16, 48] and t["final.norm"] == []


def test_safetensors_roundtrip_and_bf16_rounding(tmp_path):
    c = zatorax.parse_config(config([delta_layer()]))
    w = zatorax.random_weights(c, seed=3)
    p = os.path.join(tmp_path, "model.safetensors")
    zatorax.write_safetensors(p, w)
    got, bf16 = zatorax.read_safetensors(p)
    assert set(got) == set(w) and bf16 == set(w)
    for k in w:
        assert np.array_equal(zatorax.bf16_to_f32(got[k]).reshape(w[k].shape), w[k]), k
    # round to nearest even on the 16 dropped bits
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e-39, 65504.0], np.float32)
    bits = zatorax.f32_to_bf16(x)
    assert zatorax.bf16_to_f32(bits).tolist() == [1.0, 1.0, 1.015625, zatorax.bf16_to_f32(bits)[3], 65536.0]


def test_registry_knows_the_family(tmp_path):
    assert "Zatorax" in models.architectures()
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump(config([delta_layer()]), f)
    assert models.architecture_of(str(tmp_path)) == "Zatorax"
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump({"architecture": "nothing"}, f)
    with pytest.raises(TensorError):
        models.load_model(str(tmp_path), None)


# ---- hand-made cases for the reference itself ---------------------------------------------------------------------------------------------
def test_ref_conv_last_column_is_the_current_token():
    x = np.arange(1, 6, dtype=np.float64).reshape(5, 1)
    w = np.array([[100.0, 10.0, 1.0]])
    assert R.causal_conv(x, w)[:, 0].tolist() == [1, 12, 123, 234, 345]


def test_ref_delta_rule_reads_its_own_write_and_decays_first():
    # one head, dk = dv = 1: S <- g S ; u = b (v - S k) ; S <- S + k u ; o = S q
    q = np.ones((2, 1, 1)); k = np.ones((2, 1, 1)); v = np.array([[[2.0]], [[0.0]]])
    beta = np.array([[1.0], [0.5]]); decay = np.array([[0.25], [0.5]])
    o, S = R.delta_rule(q, k, v, beta, decay)
    assert o[:, 0, 0].tolist() == [2.0, 0.5] and S[0, 0, 0] == 0.5          # t=1: S = 1.0 after decay, u = 0.5 * (0 - 1) -> 0.5


def test_ref_window_counts_itself():
    T, win = 6, 3
    q = np.zeros((T, 1, 2)); k = np.zeros((T, 1, 2)); v = np.eye(T)[:, None, :]
    out = R.windowed_softmax_attention(q, k, v, win, 1.0, np.zeros(1), np.zeros(1))
    assert np.allclose(out[5, 0], [0, 0, 0, 1 / 3, 1 / 3, 1 / 3]) and np.allclose(out[1, 0], [0.5, 0.5, 0, 0, 0, 0])


def test_ref_distance_penalty_is_subtracted():
    T = 3
    q = np.zeros((T, 1, 1)); k = np.zeros((T, 1, 1)); v = np.eye(T)[:, None, :]
    out = R.windowed_softmax_attention(q, k, v, 8, 1.0, np.array([1.0]), np.array([1.0]))       # weights ~ 1 / (1 + distance)
    assert np.allclose(out[2, 0], np.array([1 / 3, 1 / 2, 1.0]) / (1 / 3 + 1 / 2 + 1.0))


def test_ref_router_groups_mask_with_minus_infinity_and_weights_ignore_the_correction():
    # 4 experts in 2 groups, keep 1, top 2; all choice scores of the better group are NEGATIVE, the masked ones would be 0 if masked with 0
    D = 4
    w = {"m.router": np.eye(4), "m.correction": np.array([-0.9, -2.0, -5.0, -5.0])}
    h = np.array([[2.0, 0.0, 1.0, 1.0]])
    chosen, weights = R.route(h, w, "m", {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}})
    s = np.exp(h[0]) / np.exp(h[0]).sum()
    assert chosen[0].tolist() == [0, 1] and np.allclose(weights[0], s[[0, 1]])
