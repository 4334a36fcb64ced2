"""What needs no GPU of the Meresun family: configuration, tensor inventory, registry, the frequency tables, and hand-made cases
that pin the plain reference itself (tests/meresun_ref.py), so that the GPU tests compare against something known."""
import json
import os

import numpy as np
import pytest

from crabml_b200 import meresun, models, rotary
from crabml_b200.capi import TensorError
from tests import meresun_ref as R
from tests.meresun_common import config, layer, mixed_config, moe, rot


def test_parse_config_fills_defaults_and_rejects_unknowns():
    c = meresun.parse_config(config([layer(mlp=None), layer(mlp=moe(groups=0))], side=0))
    assert c["loop"] == {"start": 0, "stop": 0, "times": 1} and c["token_side"] is None
    assert c["layers"][1]["mlp"]["router"]["groups"] == {"count": 1, "keep": 1}
    raw = config([layer()])
    del raw["embedding"]; del raw["norm"]["groups"]
    c = meresun.parse_config(raw)
    assert c["embedding"]["scale"] == 1.0 and c["norm"]["groups"] == 1
    bad = config([layer()]); bad["layers"][0]["type"] = "convolution"
    with pytest.raises(TensorError):
        meresun.parse_config(bad)
    bad = config([layer()]); bad["layers"][0]["mlp"]["kind"] = "sparse"
    with pytest.raises(TensorError):
        meresun.parse_config(bad)
    with pytest.raises(TensorError):
        meresun.parse_config(config([layer()], loop=(0, 2, 2)))
    with pytest.raises(TensorError):
        meresun.parse_config(config([layer()], width=35, groups=3))
    with pytest.raises(TensorError):
        meresun.parse_config({**config([layer()]), "architecture": "Zatorax"})


def test_expected_tensors_follow_the_config():
    c = meresun.parse_config(mixed_config())
    t = meresun.expected_tensors(c)
    assert t["side.embed"] == [53, 5 * 4] and t["l1.mix.uq"] == [2 * (12 + 6), 9] and t["l1.mix.dkv"] == [14 + 6, 36]
    assert t["l1.mlp.e5.down"] == [36, 12] and "l1.mlp.e6.gate" not in t and t["l0.mlp.act"] == [4]
    assert "l2.rg2" not in t and "l2.rg1" in t and "l2.mlp.up" not in t
    assert t["l3.mix.uk"] == [4 * 4, 11] and t["l3.mix.uv"] == [4 * 16, 11] and t["l3.mix.sink"] == [4]
    w = meresun.random_weights(c, 0)
    assert sorted(w) == sorted(t) and all(list(w[n].shape) == s for n, s in t.items())


def test_registry_knows_the_family(tmp_path):
    assert "Meresun" in models.architectures()
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump(mixed_config(), f)
    assert models.architecture_of(str(tmp_path)) == "Meresun"


@pytest.mark.parametrize("r", [rot(16), rot(8, base=5e5, scaling={"factor": 2.5, "original": 1000, "fast": 20.0, "slow": 0.5}), rot(6, scaling=None),
                               rot(2, base=50.0), rot(64, base=1e6, scaling={"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0})])
def test_frequency_tables_against_the_reference(r):
    f, mag = rotary.table_of(r)
    fr, magr = R.rotary_frequencies(r)
    assert f.dtype == np.float32 and f.shape == (r["dims"] // 2,)
    assert np.abs(f / fr - 1).max() < 1e-7 and abs(mag - magr) < 1e-7
    if not r.get("scaling"):
        assert mag == 1.0 and abs(f[-1] - r["base"] ** (-(r["dims"] - 2) / r["dims"])) < 1e-9


def test_yarn_keeps_fast_pairs_and_slows_the_slow_ones():
    r = rot(32, base=10000.0, scaling={"factor": 5.0, "original": 1024, "fast": 32.0, "slow": 1.0})
    f, mag = R.rotary_frequencies(r)
    plain, _ = R.rotary_frequencies({"dims": 32, "base": 10000.0})
    turns = 1024 * plain / (2 * np.pi)
    assert np.allclose(f[turns > 40], plain[turns > 40]) and np.allclose(f[turns < 0.7], plain[turns < 0.7] / 5.0)
    assert np.all(np.diff(f / plain) <= 1e-12) and mag == pytest.approx(0.1 * np.log(5.0) + 1.0)


# ---- the reference pinned by hand ------------------------------------------------------------------------------------------------------
def test_ref_rotation_pairs_neighbours_and_position_zero_is_identity():
    v = np.arange(1.0, 9.0).reshape(2, 1, 4)
    out = R.rotate_pairs(v, [0, 3], np.array([0.5, 0.25]), 2.0)
    assert np.allclose(out[0], 2.0 * v[0])
    a, b = 3 * 0.5, 3 * 0.25
    want = 2.0 * np.array([5 * np.cos(a) - 6 * np.sin(a), 6 * np.cos(a) + 5 * np.sin(a), 7 * np.cos(b) - 8 * np.sin(b), 8 * np.cos(b) + 7 * np.sin(b)])
    assert np.allclose(out[1, 0], want)


def test_ref_group_norm_and_poly_norm():
    x = np.array([[3.0, 4.0, 0.0, 2.0]])
    out = R.group_rms_norm(x, np.array([1.0, 1.0, 2.0, 2.0]), 2, 0.0)
    assert np.allclose(out, [[3 / np.sqrt(12.5), 4 / np.sqrt(12.5), 0.0, 2 * 2 / np.sqrt(2.0)]])
    z = np.full((1, 6), -2.0)
    assert np.allclose(R.poly_norm(z, [0.5, 0.25, 0.125, 7.0], 0.0), -0.5 + 0.25 - 0.125 + 7.0)


def _attention_weights(H=1, dn=2, dr=2, dv=2, rank=2, D=4):
    """identity-like projections: the latent is the first `rank` inputs, the rotated key part the next dr"""
    w = {"dq": np.eye(D), "dq.norm": np.ones(D), "uq": np.zeros((H * (dn + dr), D)), "dkv": np.eye(rank + dr, D), "dkv.norm": np.ones(rank),
         "uk": np.tile(np.eye(dn, rank), (H, 1)), "uv": np.tile(np.eye(dv, rank), (H, 1)), "o": np.eye(D, H * dv), "sink": np.full(H, -1e30)}
    return {"m." + k: v for k, v in w.items()}


def test_ref_window_counts_itself_and_the_sink_counts_once_unscaled():
    m = {"heads": 1, "dim": 2, "rot_dim": 2, "vdim": 2, "q_rank": 4, "kv_rank": 2, "mask": {"size": 2}, "scale": 123.0, "rot": {"dims": 2, "base": 10.0}}
    w = _attention_weights()
    h = np.array([[1.0, 0, 0, 0], [0, 1.0, 0, 0], [1.0, 1.0, 0, 0]])
    # queries are zero: every visible key scores 0, so the result is the mean of the visible values (window 2: itself and one before)
    out = R.latent_attention(h, w, "m.", m, 0.0)
    c = h[:, :2] / np.sqrt((h[:, :2] ** 2).mean(-1, keepdims=True))
    assert np.allclose(out[0, :2], c[0]) and np.allclose(out[2, :2], (c[1] + c[2]) / 2)
    w["m.sink"] = np.array([0.0])                        # exp(0) = 1 joins the denominator whatever the scale is
    out = R.latent_attention(h, w, "m.", m, 0.0)
    assert np.allclose(out[0, :2], c[0] / 2) and np.allclose(out[2, :2], (c[1] + c[2]) / 3)


def test_ref_router_sums_two_per_group_masks_with_minus_infinity_and_renormalises():
    s_logit = np.log(np.array([[0.9, 0.1, 0.6, 0.55, 0.2, 0.3]]) / (1 - np.array([[0.9, 0.1, 0.6, 0.55, 0.2, 0.3]])))
    router = np.eye(6)
    # groups (0,1) (2,3) (4,5): sums 1.0, 1.15, 0.5 -> keep the first two; the largest single score alone would have kept the same,
    # so shift group 0 down with the correction: choice sums -1.0+..., group 0 falls out although expert 0 has the best score
    ids, wt = R.route(s_logit, router, np.zeros(6), 2, 3, 2)
    assert ids.tolist() == [[0, 2]] and np.allclose(wt, [[0.9 / 1.5, 0.6 / 1.5]])
    corr = np.array([-5.0, -5.0, -3.0, -3.0, -3.0, -3.0])
    ids, wt = R.route(s_logit, router, corr, 3, 3, 2)
    # all choice scores are negative; the kept groups are (2,3) and (4,5); three experts come from them, never from group 0 (a masked
    # score of 0 would have won), and the weights are the scores WITHOUT the correction, renormalised
    assert ids.tolist() == [[2, 3, 5]] and np.allclose(wt, np.array([[0.6, 0.55, 0.3]]) / 1.45)


def test_ref_expert_clamps_gate_above_only_and_up_both_sides():
    gate = np.array([[1.0], [1.0], [1.0]]); up = gate.copy(); down = np.eye(3)
    h = np.array([10.0])
    out = R.expert(h, gate, up, down, 2.0)
    assert np.allclose(out, 2.0 * R.sigmoid(1.702 * 2.0) * 3.0)
    out = R.expert(-h, gate, up, down, 2.0)
    assert np.allclose(out, -10.0 * R.sigmoid(-17.02) * (-2.0 + 1.0))


def test_ref_layer_runs_follow_the_loop():
    c = config([layer()] * 5, loop=(2, 4, 3))
    assert R.layer_runs(c) == [(0, False), (1, False), (2, False), (3, False), (2, True), (3, False), (2, True), (3, False), (4, False)]
    assert R.layer_runs(config([layer()] * 2)) == [(0, False), (1, False)]
    assert R.layer_runs(config([layer()] * 2, loop=(0, 2, 2))) == [(0, False), (1, False), (0, True), (1, False)]
