"""Venanex configurations drawn at random over what config.json allows (sizes, head counts,
the order of the layers, chunk sizes, experts and how many are chosen, with and without a
shared expert, a query latent, stretched wavelengths, a repeated run), each through the engine
against the plain model: a whole prompt, its last tokens one by one, and an unequal batch."""

import numpy as np
import pytest

import plain_venanex as plain
import semantic_aware_adaptive_kv_cache_precision_b200 as sakv
from helpers import assert_close_to_plain, assert_same_logits
from venanex_configs import attention, latent, moe

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = np.random.default_rng(1000 + seed)
    pick = lambda options: options[int(rng.integers(len(options)))]
    width = pick([48, 64, 80, 100, 128, 160, 320])

    def feed_forward():
        if rng.random() < 0.25:
            return None
        experts = int(rng.integers(1, 13))
        shared = None if rng.random() < 0.3 else (pick([16, 40, 128]), float(rng.uniform(0.5, 3)))
        return moe(experts, int(rng.integers(1, min(experts, 4) + 1)), pick([16, 24, 50, 64]),
                   float(rng.uniform(0.5, 3)), shared)

    layers = []
    for _ in range(int(rng.integers(1, 6))):
        if rng.random() < 0.5:
            rot_dim = pick([2, 4, 8, 16, 32])
            scaling = None if rng.random() < 0.3 else (
                float(rng.uniform(1.5, 8)), int(pick([32, 64, 2048])), float(pick([8, 16, 32])),
                float(pick([0.5, 1, 2])))
            dim = pick([8, 16, 24, 32, 40])
            layers.append(latent(pick([1, 2, 3, 4, 8]), dim, rot_dim, pick([8, 16, 20, 32, 48]),
                                 pick([8, 24, 40, 64, 128]), pick([None, 16, 48, 80]),
                                 float((dim + rot_dim) ** -0.5), float(pick([100, 1e4, 5e5])),
                                 scaling, feed_forward()))
        else:
            kv_heads = pick([1, 2, 4])
            dim = pick([8, 16, 24, 48])
            layers.append(attention(kv_heads * pick([1, 2, 3]), kv_heads, dim,
                                    pick([8, 12, 32, 96]), float(dim ** -0.5),
                                    float(rng.uniform(0.1, 0.6)), pick([None, 1, 5, 32, 64, 70, 128]),
                                    feed_forward()))
    config = {"architecture": "Venanex", "vocab": int(rng.integers(50, 600)), "width": width,
              "norm": {"eps": float(pick([1e-6, 1e-5]))}, "initializer_range": 0.1,
              "layers": layers}
    if rng.random() < 0.7:
        start = int(rng.integers(0, len(layers)))
        stop = int(rng.integers(start + 1, len(layers) + 1))
        config["loop"] = {"start": start, "stop": stop, "times": int(rng.integers(1, 4))}
    return config


def rows_without_close_calls(config, tensors, p):
    margins = []
    want = plain.forward(config, tensors, p, None, margins)
    clear = np.ones(len(p), dtype=bool)
    for m in margins:
        clear &= m >= 2e-4
    return want, clear


@pytest.mark.parametrize("seed", range(24))
def test_a_drawn_configuration_in_32_bits(seed, tmp_path):
    config = draw(seed)
    folder = sakv.write_random_model(tmp_path / "m", config, seed, dtype="float32")
    cfg, tensors = plain.read_model_folder(folder)
    engine = sakv.Engine(folder, dtype="float32", max_tokens=1024, poison_freed=True).load_weights()
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, config["vocab"], n).astype(np.int64) for n in (150, 37, 2)]
    wants = [rows_without_close_calls(cfg, tensors, p) for p in prompts]
    whole = [engine.forward(p) for p in prompts]
    for got, (want, clear) in zip(whole, wants):
        assert_close_to_plain(got[clear], want[clear], "float32", f"seed {seed}")
    # the longest prompt again: most of it in one step, its last 40 tokens one by one
    p, (_, clear) = prompts[0], wants[0]
    (slot,) = engine.open(1)
    rows = [engine.step([slot], [p[:110]], [list(range(110))]).cpu().numpy()]
    for t in range(110, len(p)):
        rows.append(engine.step([slot], [p[t:t + 1]]).cpu().numpy())
    engine.close([slot])
    assert_same_logits(np.concatenate(rows)[clear], whole[0][clear], "float32", f"seed {seed}: decoded")
    # the three together, then decoded together until each ends
    slots = engine.open(3)
    heads = [len(q) - k for q, k in zip(prompts, (5, 3, 1))]
    out = engine.step(slots, [q[:h] for q, h in zip(prompts, heads)],
                      [list(range(h)) for h in heads]).cpu().numpy()
    got = [[out[sum(heads[:i]):sum(heads[:i + 1])]] for i in range(3)]
    fed = list(heads)
    live = [0, 1, 2]
    while live:
        out = engine.step([slots[i] for i in live], [prompts[i][fed[i]:fed[i] + 1] for i in live])
        for k, i in enumerate(live):
            got[i].append(out[k:k + 1].cpu().numpy())
            fed[i] += 1
        done = [i for i in live if fed[i] == len(prompts[i])]
        if done:
            engine.close([slots[i] for i in done])
        live = [i for i in live if fed[i] < len(prompts[i])]
    for i in range(3):
        clear = wants[i][1]
        assert_same_logits(np.concatenate(got[i])[clear], whole[i][clear], "float32",
                           f"seed {seed}: request {i} of the batch")
    engine.cache.check()
    assert engine.graph_failure is None


@pytest.mark.parametrize("seed", range(24))
def test_a_drawn_configuration_in_16_bits(seed, tmp_path):
    """Every expert for every token (no choice for rounding to turn); judged by the median
    row within a tenth of its spread, since a drawn configuration may be deep (up to 13 layer
    runs, each carrying its sublayers' rounding to the stream at full size through the norm
    after them: 0.8 % of the stream a run was measured on the worst draw, 7 % of the logits'
    spread at its end) or badly conditioned (two maps that nearly cancel)."""
    config = draw(seed)
    for layer in config["layers"]:
        if layer["mlp"] is not None:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    folder = sakv.write_random_model(tmp_path / "m", config, seed, dtype="bfloat16")
    cfg, tensors = plain.read_model_folder(folder)
    engine = sakv.Engine(folder, dtype="bfloat16", max_tokens=1024, poison_freed=True).load_weights()
    p = np.random.default_rng(seed).integers(0, config["vocab"], 150).astype(np.int64)
    want = plain.forward(cfg, tensors, p)
    (slot,) = engine.open(1)
    rows = [engine.step([slot], [p[:110]], [list(range(110))]).cpu().numpy()]
    for t in range(110, len(p)):
        rows.append(engine.step([slot], [p[t:t + 1]]).cpu().numpy())
    engine.close([slot])
    got = np.concatenate(rows)
    assert np.isfinite(got).all()
    worst = np.abs(got - want).max(axis=-1) / want.std(axis=-1)
    assert np.median(worst[:110]) <= 0.1, f"seed {seed}: the prompt's median row {np.median(worst[:110]):.3f}"
    assert np.median(worst[110:]) <= 0.1, f"seed {seed}: the decoded median row {np.median(worst[110:]):.3f}"
    assert engine.graph_failure is None
