"""Tebonex models with random weights through the engine, against the plain model: whole
prompts, pieces of prompts down to two tokens, the last tokens one by one, unequal batches
whose slots and cache blocks are used again, long decoding past windows and block borders,
greedy generation through `Engine.generate`, and the trace-replay program."""

import numpy as np
import pytest

import plain_tebonex as plain
import semantic_aware_adaptive_kv_cache_precision_b200 as sakv
from helpers import assert_close_to_plain, assert_same_logits
from tebonex_configs import CONFIGS

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("tebonex")
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            config, seed = CONFIGS[name]
            made[name, dtype] = sakv.write_random_model(root / f"{name}_{dtype}", dict(config),
                                                        seed, dtype=dtype)
        return made[name, dtype]

    return get


def prompts_of(name, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, CONFIGS[name][0]["vocab"], n).astype(np.int64) for n in lengths]


def setup(folders, name, dtype, max_tokens=1024):
    folder = folders(name, dtype)
    config, tensors = plain.read_model_folder(folder)
    engine = sakv.Engine(folder, dtype=dtype, max_tokens=max_tokens, poison_freed=True)
    return engine.load_weights(), config, tensors


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_and_every_layer(name, dtype, folders):
    engine, config, tensors = setup(folders, name, dtype)
    for p in prompts_of(name, (1, 2, 63, 201)):
        sums = []
        want = plain.forward(config, tensors, p, sums)
        got, states = engine.forward(p, capture_hidden_states=True)
        assert_close_to_plain(got, want, dtype, f"{name}: a prompt of {len(p)}")
        for i, s in enumerate(sums[:-1]):        # the stream after each layer but the last
            bound = (2e-5 if dtype == "float32" else 3e-2) * np.abs(s).max()
            assert np.abs(states[i + 1] - s).max() <= bound, f"{name}: after layer {i}"
    assert engine.graph_failure is None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_pieces_of_a_prompt_and_tokens_one_by_one(name, dtype, folders):
    engine, config, tensors = setup(folders, name, dtype)
    (p,) = prompts_of(name, (230,), seed=1)
    whole = engine.forward(p)
    assert_close_to_plain(whole, plain.forward(config, tensors, p), dtype, name)
    for pieces in ([2, 3, 59, 1, 64, 65, 7, 29], [128, 2, 100], [1] * 3 + [190] + [1] * 37):
        (slot,) = engine.open(1)
        rows, at = [], 0
        for n in pieces:
            rows.append(engine.step([slot], [p[at:at + n]], [list(range(n))]).cpu().numpy())
            at += n
        engine.close([slot])
        assert at == len(p)
        assert_same_logits(np.concatenate(rows), whole, dtype, f"{name}: pieces {pieces[:4]}...")
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batches_with_slots_and_blocks_used_again(name, dtype, folders):
    """The cache holds exactly one batch, so every batch gets blocks and slots that
    the batch before gave back (filled with NaN when they were freed)."""
    lengths = (150, 9, 77, 1)
    engine, config, tensors = setup(folders, name, dtype, max_tokens=7 * 64)
    prompts = prompts_of(name, lengths, seed=2)
    alone = [engine.forward(p) for p in prompts]
    for g, w in zip(alone, prompts):
        assert_close_to_plain(g, plain.forward(config, tensors, w), dtype, name)
    tails = (6, 3, 9, 0)
    for round_ in range(3):
        order = [(i + round_) % 4 for i in range(4)]
        if round_ == 1:
            spare, *slots = engine.open(5)
            engine.close([spare])
        else:
            slots = engine.open(4)
        heads = [lengths[i] - tails[i] for i in order]
        out = engine.step(slots, [prompts[i][:h] for i, h in zip(order, heads)],
                          [list(range(h)) for h in heads]).cpu().numpy()
        rows = {i: [out[sum(heads[:k]):sum(heads[:k + 1])]] for k, i in enumerate(order)}
        fed = dict(zip(order, heads))
        live = [(i, s) for i, s in zip(order, slots)]
        while True:
            done = [(i, s) for i, s in live if fed[i] == lengths[i]]
            if done:
                engine.close([s for _, s in done])
            live = [(i, s) for i, s in live if fed[i] < lengths[i]]
            if not live:
                break
            out = engine.step([s for _, s in live], [prompts[i][fed[i]:fed[i] + 1] for i, _ in live])
            for k, (i, _) in enumerate(live):
                rows[i].append(out[k:k + 1].cpu().numpy())
                fed[i] += 1
        for i in range(4):
            assert_same_logits(np.concatenate(rows[i]), alone[i], dtype,
                               f"{name}: round {round_}, request {i}")
        engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "plain"])
def test_long_decoding_past_windows_and_block_borders(name, dtype, folders):
    engine, config, tensors = setup(folders, name, dtype, max_tokens=512)
    (p,) = prompts_of(name, (300,), seed=3)
    want = plain.forward(config, tensors, p)
    (slot,) = engine.open(1)
    rows = [engine.step([slot], [p[:5]], [list(range(5))]).cpu().numpy()]
    for t in range(5, len(p)):
        rows.append(engine.step([slot], [p[t:t + 1]]).cpu().numpy())
    engine.close([slot])
    assert_close_to_plain(np.concatenate(rows), want, dtype, f"{name}: 295 tokens one by one")
    assert engine.graph_failure is None


@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_engine(name, folders):
    engine, config, tensors = setup(folders, name, "float32")
    prompts = [p.tolist() for p in prompts_of(name, (7, 40, 1), seed=4)]
    got = engine.generate(prompts, 12, stop_at_eos=False)
    for p, g in zip(prompts, got):
        assert g.tolist() == plain.generate(config, tensors, p, 12)
    assert all(e.state == sakv.COMPLETE for e in engine.endings)
    engine.cache.check()
    assert engine.cache.slots.held == 0


def test_generation_in_bfloat16_follows_the_plain_model(folders):
    engine, config, tensors = setup(folders, "mixed", "bfloat16")
    prompts = [p.tolist() for p in prompts_of("mixed", (33, 5), seed=5)]
    got = engine.generate(prompts, 10, stop_at_eos=False)
    for p, g in zip(prompts, got):         # each token is the plain model's choice or a near tie
        ref = plain.forward(config, tensors, p + g.tolist()[:-1])[len(p) - 1:]
        for k, token in enumerate(g.tolist()):
            assert ref[k].max() - ref[k, token] <= 0.06 * ref[k].std()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_runs_a_tebonex_folder(dtype, folders, tmp_path):
    from test_trace_run_gpu import Trace, entry
    folder = folders("mixed", dtype)
    config, tensors = plain.read_model_folder(folder)
    a, b, c = prompts_of("mixed", (90, 41, 3), seed=6)
    want = {k: plain.forward(config, tensors, p) for k, p in (("a", a), ("b", b), ("c", c))}
    trace = Trace(folder, dtype, tmp_path / "out", 512)
    got = trace.send([entry("a", a[:80], range(80)), entry("b", b[:40], [0, 39]),
                      entry("c", c, [2])], end=["c"])
    assert_close_to_plain(got[:80], want["a"][:80], dtype, "a's prompt")
    assert_close_to_plain(got[80:82], want["b"][[0, 39]], dtype, "b's prompt")
    assert_close_to_plain(got[82:], want["c"][2:], dtype, "c")
    got = trace.send([entry("a", a[80:81], [0]), entry("b", b[40:], [0])], end=["b"])
    assert_close_to_plain(got, np.stack([want["a"][80], want["b"][40]]), dtype, "one token each")
    for t in range(81, 90):
        got = trace.send([entry("a", a[t:t + 1], [0])], end=["a"] if t == 89 else [])
        assert_close_to_plain(got, want["a"][t:t + 1], dtype, f"a alone at {t}")
    trace.finish()


def test_the_command_line_writes_and_runs_a_tebonex_folder(tmp_path):
    """`random-model` from a config.json, then `generate` and `throughput` on the folder."""
    import json
    from test_cli import run
    config = tmp_path / "config.json"
    config.write_text(json.dumps(CONFIGS["single"][0]))
    run("random-model", "--config", str(config), "--seed", "3", "--out", str(tmp_path / "m"),
        "--stored-dtype", "float32")
    cfg, tensors = plain.read_model_folder(tmp_path / "m")
    assert cfg["architecture"] == "Tebonex" and tensors["l1.mix.r1"].shape == (8,)
    (p,) = prompts_of("single", (11,), seed=7)
    records, _ = run("generate", "--model", str(tmp_path / "m"), "--dtype", "float32",
                     "--ignore-eos", "--prompt-ids", ",".join(map(str, p)), "--new-tokens", "6")
    assert records[0]["tokens"] == plain.generate(cfg, tensors, p.tolist(), 6)
    records, _ = run("throughput", "--model", str(tmp_path / "m"), "--lengths", "70",
                     "--repeat", "1", "--warmup", "1", "--batch", "2")
    assert records[0]["decode_tokens_per_second"] > 0
