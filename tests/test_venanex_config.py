"""The Venanex configuration: what it reads, what it refuses, its run order, and the plain
model's own mechanisms on hand-made inputs. No GPU."""

import copy
import math

import numpy as np
import pytest

import plain_venanex as plain
import semantic_aware_adaptive_kv_cache_precision_b200 as sakv
from semantic_aware_adaptive_kv_cache_precision_b200.config import (ConfigError, config_from_dict,
                                                                   known_architectures)
from semantic_aware_adaptive_kv_cache_precision_b200.engine.model import DecoderModel
from venanex_configs import CONFIGS, MIXED, ODD, PLAIN


def test_registered_and_round_trips():
    assert "Venanex" in known_architectures()
    for config, _ in CONFIGS.values():
        typed = config_from_dict(copy.deepcopy(config))
        assert config_from_dict(typed.to_dict()) == typed


def test_run_order_repeats_the_run_with_a_cache_each_and_marks_each_pass():
    spec = config_from_dict(copy.deepcopy(MIXED)).model_spec()
    assert [c.block for c in spec.run_order] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [c.cache for c in spec.run_order] == list(range(8))
    assert [c.mix_input for c in spec.run_order] == [False, True, False, True, False, True,
                                                     False, False]
    assert [(i, f) for i, f in plain.run_order(MIXED)] == \
        [(c.block, c.mix_input) for c in spec.run_order]
    assert spec.input_mix_name == "loop.in" and spec.tie_head
    plain_spec = config_from_dict(copy.deepcopy(PLAIN)).model_spec()       # no repeated run
    assert plain_spec.input_mix_name is None
    assert not any(c.mix_input for c in plain_spec.run_order)
    once = config_from_dict(copy.deepcopy(ODD)).model_spec()               # a run of one pass
    assert [c.mix_input for c in once.run_order] == [True, False, False]


def test_declared_tensors_carry_the_configuration_s_sizes():
    spec = config_from_dict(copy.deepcopy(MIXED)).model_spec()
    shapes = {d.name: tuple(d.shape) for d in DecoderModel.tensor_decls_of(spec)}
    assert shapes["embed"] == (211, 96) and shapes["loop.in"] == (96, 192)
    assert shapes["l0.mix.dq"] == (24, 96) and shapes["l0.mix.uq"] == (4 * 24, 24)
    assert shapes["l0.mix.dkv"] == (48, 96) and shapes["l0.mix.dkv.norm"] == (40,)
    assert shapes["l0.mix.uk"] == (64, 40) and shapes["l0.mix.uv"] == (96, 40)
    assert shapes["l0.mlp.e5.down"] == (96, 48) and shapes["l0.mlp.shared.sg"] == (1, 96)
    assert shapes["l1.mix.q"] == (4 * 2 * 16, 96) and shapes["l1.mix.k"] == (2 * 2 * 16, 96)
    assert shapes["l1.mix.v"] == (48, 96) and shapes["l1.mix.g"] == (96, 96)
    assert shapes["l1.mix.lq2"] == (16,)
    assert "l1.norm2" not in shapes and "l1.mlp.router" not in shapes     # no feed-forward
    assert shapes["l2.mix.q"] == (3 * 40, 96) and "l2.mix.dq" not in shapes   # no query latent
    assert "l2.mlp.shared.gate" not in shapes and "final.norm" in shapes


def test_problems_are_listed_together():
    bad = copy.deepcopy(MIXED)
    bad["layers"][0]["mixer"]["rot"]["dims"] = 6
    bad["layers"][1]["mixer"]["kv_heads"] = 3
    bad["layers"][0]["mlp"]["router"]["top"] = 9
    bad["layers"][3]["type"] = "convolution"
    bad["loop"]["stop"] = 7
    with pytest.raises(ConfigError) as err:
        config_from_dict(bad)
    text = str(err.value)
    for piece in ("rot.dims", "kv_heads", "router.top", "convolution", "loop"):
        assert piece in text


def test_stretched_frequencies_by_hand():
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 50, "fast": 4.0,
                                                  "slow": 0.5}}
    f, mag = plain.yarn_frequencies(rot)
    plain_f = [100.0 ** (-2 * i / 8) for i in range(4)]
    where = lambda turns: 8 * math.log(50 / (2 * math.pi * turns)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(where(4.0)), 0), min(math.ceil(where(0.5)), 7)
    assert (lo, hi) == (0, 3)
    for i in range(4):
        ramp = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert f[i] == pytest.approx(plain_f[i] / 4.0 * ramp + plain_f[i] * (1 - ramp))
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert plain.yarn_frequencies({"base": 100.0, "dims": 8})[1] == 1.0
    # the library's table is the same
    from semantic_aware_adaptive_kv_cache_precision_b200.config import RampScaling, RotarySpec
    from semantic_aware_adaptive_kv_cache_precision_b200.parts import RotaryHalf
    part = RotaryHalf(RotarySpec(8, 8, 100.0, 64, scaling=RampScaling(4.0, 50, 4.0, 0.5)), "", "float32")
    got, got_mag = part.frequencies()
    assert np.allclose(got, f, rtol=1e-15) and got_mag == pytest.approx(mag)


def test_chunks_count_from_the_sequence_s_start_in_the_plain_model():
    """A query sees its own run of positions only: the first token of a run sees itself."""
    rng = np.random.default_rng(0)
    n, width = 9, 8
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 1.0, "diff": 0.0,
         "mask": {"size": 4}}
    t = {"q": rng.normal(size=(8, width)), "k": rng.normal(size=(8, width)),
         "v": rng.normal(size=(4, width)), "g": np.zeros((4, width)), "o": np.eye(width, 4),
         "lq1": np.zeros(4), "lk1": np.zeros(4), "lq2": np.zeros(4), "lk2": np.zeros(4)}
    h = rng.normal(size=(n, width))
    out = plain.differential_attention(h, t, "", m, 0.0)
    # lambda = 1 - 1 + 0 = 0: the first map alone; at positions 0, 4, 8 it is the value itself
    v = h @ t["v"].T
    for i in (0, 4, 8):
        unit = v[i] / np.sqrt(np.mean(v[i] ** 2))
        assert np.allclose(out[i, :4], unit * 0.5)


def test_the_weight_multiplies_the_expert_s_input():
    rng = np.random.default_rng(1)
    t = {"router": np.array([[10.0, 0.0], [-10.0, 0.0]]), "e0.gate": rng.normal(size=(3, 2)),
         "e0.up": rng.normal(size=(3, 2)), "e0.down": rng.normal(size=(2, 3)),
         "e1.gate": rng.normal(size=(3, 2)), "e1.up": rng.normal(size=(3, 2)),
         "e1.down": rng.normal(size=(2, 3))}
    m = {"router": {"experts": 2, "top": 1}, "expert": {"ff": 3, "limit": 0.5}}
    h = np.array([[0.3, 1.0], [-0.2, 2.0]])
    out = plain.moe(h, t, "", m)
    w0, w1 = plain.sigmoid(3.0), plain.sigmoid(2.0)       # token 0 -> expert 0, token 1 -> expert 1
    assert np.allclose(out[0], plain.expert(w0 * h[:1], t, "e0.", 0.5)[0])
    assert np.allclose(out[1], plain.expert(w1 * h[1:], t, "e1.", 0.5)[0])
    assert not np.allclose(out[0], w0 * plain.expert(h[:1], t, "e0.", 0.5)[0])
