"""The Tebonex configuration, its tensors, and the cache needs of its layers. No GPU."""

import json

import numpy as np
import pytest
import torch

import plain_tebonex as plain
import semantic_aware_adaptive_kv_cache_precision_b200 as sakv
from semantic_aware_adaptive_kv_cache_precision_b200.cache import (BLOCK, KVNeed, MultiNeed,
                                                                    SequenceCache, StateNeed)
from semantic_aware_adaptive_kv_cache_precision_b200.config import ConfigError, TebonexConfig
from semantic_aware_adaptive_kv_cache_precision_b200.engine.model import DecoderModel
from semantic_aware_adaptive_kv_cache_precision_b200.weights import Checkpoint, check_tensors
from tebonex_configs import CONFIGS, MIXED, PLAIN, SINGLE


def test_every_size_and_the_order_of_layers_come_from_config_json():
    spec = sakv.config_from_dict(MIXED).model_spec()
    assert spec.streams == 3 and spec.vocab_size == 211 and spec.embed_scale == 12.0
    kinds = [b.mixer.kind for b in spec.blocks]
    assert kinds == ["log_distance_attention", "general_delta"] * 2
    a, d, a2, d2 = (b.mixer for b in spec.blocks)
    assert (a.heads, a.kv_heads, a.head_dim, a.value_dim, a.window, a.scale) == (4, 2, 16, 24, 37, 0.3)
    assert a2.window is None and (d.heads, d.head_dim, d.decay_rank) == (3, 16, 8)
    assert d2.head_dim == 48 and d2.eps == 1e-5
    assert spec.blocks[2].ffn is None and spec.blocks[3].ffn.intermediate == 72
    plain_spec = sakv.config_from_dict(PLAIN).model_spec()
    assert plain_spec.streams == 1 and not plain_spec.blocks[0].connections
    assert sakv.config_from_dict(SINGLE).model_spec().blocks[0].connections
    assert sakv.config_from_dict(TebonexConfig.from_dict(MIXED).to_dict()) == \
        TebonexConfig.from_dict(MIXED)


def test_the_decay_rank_is_read_from_the_checkpoint(tmp_path):
    folder = sakv.write_random_model(tmp_path / "m", dict(MIXED), seed=1)
    raw = json.loads((folder / "config.json").read_text())
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None)          # as a folder from elsewhere has it
    (folder / "config.json").write_text(json.dumps(raw))
    config = sakv.config_from_folder(folder)
    assert [l.decay_rank for l in config.layers if l.type == "general_delta"] == [8, 5]
    spec = config.model_spec()
    check_tensors(Checkpoint(folder), DecoderModel.tensor_decls_of(spec), "config.json",
                  spec.ignore_tensors)
    _, tensors = plain.read_model_folder(folder)
    assert tensors["l1.mix.w1"].shape == (8, 96) and tensors["l0.mix.g"].shape == (4, 96)
    assert tensors["l0.hc1.mix"].shape == (3, 3) and "l2.norm2" not in tensors
    assert (tensors["l0.mix.r2"] > 0).all()


def test_problems_are_named_together():
    bad = json.loads(json.dumps(MIXED))
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    bad["layers"][1]["type"] = "conv"
    del bad["norm"]
    with pytest.raises(ConfigError) as err:
        sakv.config_from_dict(bad)
    text = str(err.value)
    assert "kv_heads" in text and "'conv'" in text and "norm.eps" in text
    with pytest.raises(ConfigError, match="not registered"):
        sakv.config_from_dict({"architecture": "Nobody"})


def test_a_layer_call_may_need_several_things_of_the_cache():
    needs = [MultiNeed((KVNeed(2, 16, 37, value_dim=24), StateNeed((96,)))),
             MultiNeed((StateNeed((3, 16, 16)), StateNeed((96,)))),
             MultiNeed((KVNeed(2, 16, 37, value_dim=24), StateNeed((96,))))]
    cache = SequenceCache(needs, 4 * BLOCK, 1 << 20, torch.float32, "cpu")
    assert len(cache.groups) == 1 and cache.groups[0].keys.shape[0] == 2
    assert cache.groups[0].values.shape[-1] == 24
    view = cache.entry_view(2, ["table"])
    assert view.parts[0].keys.shape == (4, 2, BLOCK, 16) and view.parts[0].block_table == "table"
    assert view.parts[1].state.shape == (cache.max_slots, 96)
    (slot,) = cache.open(1)
    cache.entry_view(1, ["table"]).parts[0].state[slot] += 1.0
    cache.close([slot])
    (again,) = cache.open(1)
    assert again == slot and float(cache.entry_view(1, ["table"]).parts[0].state[slot].abs().sum()) == 0


def test_the_plain_model_carries_its_state_as_the_equations_say():
    rng = np.random.default_rng(0)
    n, heads, dim = 9, 2, 5
    r, k, v = (rng.standard_normal((n, heads, dim)) for _ in range(3))
    w, a = rng.uniform(0.5, 1, (n, heads, dim)), rng.uniform(0, 1, (n, heads, dim))
    whole, last = plain.delta_rule_scan(r, k, v, w, a)
    first, state = plain.delta_rule_scan(r[:4], k[:4], v[:4], w[:4], a[:4])
    second, end = plain.delta_rule_scan(r[4:], k[4:], v[4:], w[4:], a[4:], state)
    assert np.allclose(np.concatenate([first, second]), whole) and np.allclose(end, last)
    # with no decay and no removal the state is the sum of the outer products
    o, s = plain.delta_rule_scan(r, k, v, np.ones_like(w), np.zeros_like(a))
    assert np.allclose(s, np.einsum("nhk,nhv->hkv", k, v))
    # one stream with identity connections is the plain residual sum
    xs, y = rng.standard_normal((1, n, 7)), rng.standard_normal((n, 7))
    assert np.allclose(plain.streams_write(xs, y, np.eye(1), np.ones(1))[0], xs[0] + y)
    # a window of one token sees the token itself only
    s = plain.distance_scores(r[:, 0], k[:, 0], 1.0, 0.3, 0.2, 1)
    assert np.isfinite(s).sum() == n and np.isfinite(np.diag(s)).all()
    h = rng.standard_normal((n, 7))
    shifted = plain.token_shift(h, np.full(7, 0.25))
    assert np.allclose(shifted[0], 0.75 * h[0]) and np.allclose(shifted[3], 0.75 * h[3] + 0.25 * h[2])
