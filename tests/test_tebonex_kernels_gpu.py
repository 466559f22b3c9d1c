"""The kernels of the Tebonex mechanisms, each alone against the plain functions, on inputs
made so that a fault shows: a key far back that only an undecayed state still holds, a key
that stands out just inside and just outside a window (in a prompt and decoded, at block
borders), the first token of a sequence, streams with odd counts."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_tebonex as plain
from semantic_aware_adaptive_kv_cache_precision_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype, device=DEV).contiguous()


def step_of(counts, slots, starts=None):
    """What the kernels read of a step: `counts[i]` tokens of the sequence in `slots[i]`."""
    starts = starts or [0] * len(counts)
    cu = np.concatenate([[0], np.cumsum(counts)])
    seq = np.repeat(np.arange(len(counts)), counts)
    pos = np.concatenate([np.arange(s, s + c) for s, c in zip(starts, counts)])
    i32 = lambda a: torch.as_tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    return SimpleNamespace(sequences=len(counts), cu_seqlens=i32(cu), token_seq=i32(seq),
                           slots=i32(slots), positions=i32(pos))


@pytest.mark.parametrize("streams", [1, 2, 3, 5, 9])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_streams_step(streams, wdtype):
    rng = np.random.default_rng(streams)
    n, width, eps = 7, 50, 1e-5
    bf = lambda a: dev(a, wdtype).float().cpu().numpy().astype(np.float64)
    xs, y = rng.standard_normal((streams, n, width)), rng.standard_normal((n, width))
    mix, out_w, in_w = (bf(rng.standard_normal(s)) for s in ((streams, streams), streams, streams))
    norm_w = bf(1 + 0.1 * rng.standard_normal(width))
    want_xs = plain.streams_write(xs, y, mix, out_w)
    want_h = plain.rms(plain.streams_read(want_xs, in_w), eps) * norm_w
    got_xs = dev(xs)
    got_h = ops.streams_step(got_xs, y=dev(y), mix=dev(mix, wdtype), out_w=dev(out_w, wdtype),
                             in_w=dev(in_w, wdtype), norm_w=dev(norm_w, wdtype), eps=eps)
    assert np.abs(got_xs.cpu().numpy() - want_xs).max() <= 1e-5 * np.abs(want_xs).max()
    assert np.abs(got_h.cpu().numpy() - want_h).max() <= 1e-5 * np.abs(want_h).max()
    # the read alone, the write-back alone, and the plain sum of the streams
    again = dev(xs)
    h = ops.streams_step(again, in_w=dev(in_w, wdtype), norm_w=dev(norm_w, wdtype), eps=eps,
                         out_dtype=torch.bfloat16)
    ref = plain.rms(plain.streams_read(xs, in_w), eps) * norm_w
    assert torch.equal(again, dev(xs)) and h.dtype == torch.bfloat16
    assert np.abs(h.float().cpu().numpy() - ref).max() <= 1e-2 * np.abs(ref).max()
    assert ops.streams_step(again, y=dev(y), reduce=False) is None       # identity, ones
    assert np.abs(again.cpu().numpy() - (xs + y[None])).max() <= 1e-6 * np.abs(xs).max() + 1e-6
    total = ops.streams_step(again)
    assert np.abs(total.cpu().numpy() - (xs + y[None]).sum(0)).max() <= 1e-5 * streams


def test_token_shift_takes_the_row_before_from_the_state_and_leaves_the_last():
    rng = np.random.default_rng(1)
    width = 33
    shift = rng.uniform(0, 1, width)
    rows = {7: rng.standard_normal((9, width)), 2: rng.standard_normal((4, width))}
    state = torch.zeros((12, width), device=DEV)
    state[5] = 99.0                                       # another sequence's: stays
    got = {s: [] for s in rows}
    for counts in ([3, 1], [1, 1], [5, 2]):               # slot 7 then slot 2 in each step
        h = np.concatenate([rows[7][len(np.concatenate(got[7] or [np.zeros((0, width))])):][:counts[0]],
                            rows[2][len(np.concatenate(got[2] or [np.zeros((0, width))])):][:counts[1]]])
        out = ops.token_shift(dev(h), state, dev(shift), step_of(counts, [7, 2]), torch.float32)
        got[7].append(out[:counts[0]].cpu().numpy())
        got[2].append(out[counts[0]:].cpu().numpy())
    for s in rows:
        want = plain.token_shift(rows[s], shift)
        assert np.abs(np.concatenate(got[s]) - want).max() <= 1e-6 * np.abs(want).max()
        assert np.allclose(state[s].cpu().numpy(), rows[s][-1])
    assert float(state[5].min()) == 99.0


def test_the_shift_inside_the_streams_step_is_the_shift_after_it():
    """One token a sequence: norm and blend in one kernel give the bits of the two kernels."""
    rng = np.random.default_rng(2)
    streams, width, eps = 3, 70, 1e-6
    xs = dev(rng.standard_normal((streams, 4, width)))
    in_w, norm_w, shift = dev(rng.uniform(0.2, 0.8, streams)), dev(1 + 0.1 * rng.standard_normal(width)), \
        dev(rng.uniform(0, 1, width))
    kept = dev(rng.standard_normal((9, width)))
    step = step_of([1, 1, 1, 1], [8, 0, 3, 5], [4, 0, 9, 2])
    state_a, state_b = kept.clone(), kept.clone()
    h = ops.streams_step(xs, in_w=in_w, norm_w=norm_w, eps=eps)
    two = ops.token_shift(h, state_a, shift, step, torch.float32)
    one = ops.streams_step(xs, in_w=in_w, norm_w=norm_w, eps=eps, shift=(state_b, shift, step))
    assert torch.equal(one, two) and torch.equal(state_a, state_b)
    assert torch.equal(state_a[[8, 0, 3, 5]], h) and torch.equal(state_a[1], kept[1])
    want = h + (kept[[8, 0, 3, 5]] - h) * shift
    assert float((one - want).abs().max()) <= 1e-6 * float(want.abs().max())


def delta_inputs(rng, n, heads, dim, rank, w0, a_bias):
    hd = heads * dim
    proj = rng.standard_normal((n, 5 * hd + rank)).astype(np.float32)
    consts = dict(w2=0.3 * rng.standard_normal((hd, rank)), w0=np.full(hd, w0) + 0.1 * rng.standard_normal(hd),
                  a_bias=np.full(hd, a_bias) + 0.1 * rng.standard_normal(hd),
                  norm_w=1 + 0.1 * rng.standard_normal(hd))
    return proj, {k: v.astype(np.float32) for k, v in consts.items()}


def delta_plain(proj, c, heads, dim, eps, state=None):
    n, hd = proj.shape[0], heads * dim
    p = proj.astype(np.float64)
    cols = lambda i: p[:, i * hd:(i + 1) * hd]
    w = np.exp(-plain.DECAY_SCALE * plain.sigmoid(np.tanh(p[:, 5 * hd:]) @ c["w2"].T.astype(np.float64) + c["w0"]))
    a = plain.sigmoid(cols(4) + c["a_bias"])
    shape = (n, heads, dim)
    o, state = plain.delta_rule_scan(cols(0).reshape(shape), cols(1).reshape(shape),
                                     cols(2).reshape(shape), w.reshape(shape), a.reshape(shape), state)
    return plain.rms(o, eps).reshape(n, hd) * c["norm_w"] * plain.sigmoid(cols(3)), state


@pytest.mark.parametrize("heads,dim,rank", [(3, 16, 8), (1, 64, 16), (2, 48, 5), (5, 8, 1),
                                            (2, 128, 3), (1, 136, 2), (2, 32, 70), (1, 256, 100),
                                            (3, 80, 4), (7, 20, 9)])
def test_delta_rule_whole_in_pieces_and_beside_another_sequence(heads, dim, rank):
    rng = np.random.default_rng(dim)
    n, eps = 75, 1e-5
    proj, c = delta_inputs(rng, n, heads, dim, rank, -1.0, 0.0)
    other, _ = delta_inputs(rng, 20, heads, dim, rank, -1.0, 0.0)
    want, want_state = delta_plain(proj, c, heads, dim, eps)
    offsets = tuple(i * heads * dim for i in range(6))
    consts = [dev(c[k]) for k in ("w2", "w0", "a_bias", "norm_w")]
    state = torch.zeros((6, heads, dim, dim), device=DEV)
    run = lambda rows, step: ops.delta_rule(dev(rows), offsets, *consts, state, step, heads, dim,
                                            plain.DECAY_SCALE, plain.KEY_EPS, eps, torch.float32)
    whole = run(proj, step_of([n], [4])).cpu().numpy()
    assert np.abs(whole - want).max() <= 2e-5 * np.abs(want).max()
    assert np.abs(state[4].cpu().numpy() - want_state).max() <= 2e-5 * np.abs(want_state).max()
    assert float(state[3].abs().max()) == 0 and float(state[5].abs().max()) == 0
    # pieces of 2, 1, 40, ... tokens in slot 1, the other sequence beside it in slot 0
    got, at, fed = [], 0, 0
    for piece in (2, 1, 40, 1, 1, 30):
        more = min(5, 20 - fed)
        rows = np.concatenate([other[fed:fed + more], proj[at:at + piece]])
        out = run(rows, step_of([more, piece] if more else [piece], [0, 1] if more else [1]))
        got.append(out[more:].cpu().numpy())
        at, fed = at + piece, fed + more
    assert np.array_equal(np.concatenate(got), whole)       # the same sums in the same order
    assert torch.equal(state[1], state[4])


def test_delta_rule_keeps_a_far_key_when_nothing_decays_or_removes():
    """Decay ~1 and removal ~0: the state is the sum of the outer products, and a query along
    the first key still reads the first value 400 tokens later; with the decay on it is gone."""
    rng = np.random.default_rng(5)
    heads, dim, rank, n, eps = 2, 32, 4, 400, 1e-6
    hd = heads * dim
    proj, c = delta_inputs(rng, n, heads, dim, rank, -30.0, -30.0)
    proj[:, hd:2 * hd] *= 0.02                              # small keys everywhere ...
    key = rng.standard_normal(hd).astype(np.float32)
    proj[0, hd:2 * hd] = key                                # ... but the first,
    proj[-1, 0:hd] = 20 * key                               # which the last token asks for
    offsets = tuple(i * hd for i in range(6))
    run = lambda c, state: ops.delta_rule(
        dev(proj), offsets, *[dev(c[k]) for k in ("w2", "w0", "a_bias", "norm_w")], state,
        step_of([n], [0]), heads, dim, plain.DECAY_SCALE, plain.KEY_EPS, eps, torch.float32)
    state = torch.zeros((1, heads, dim, dim), device=DEV)
    kept = run(c, state).cpu().numpy()
    want, _ = delta_plain(proj, c, heads, dim, eps)
    assert np.abs(kept - want).max() <= 2e-5 * np.abs(want).max()
    first_value = proj[0, 2 * hd:3 * hd].reshape(heads, dim).astype(np.float64)
    raw = (kept[-1] / c["norm_w"] / plain.sigmoid(proj[-1, 3 * hd:4 * hd])).reshape(heads, dim)
    cosine = (raw * first_value).sum(-1) / np.linalg.norm(raw, axis=-1) / np.linalg.norm(first_value, axis=-1)
    assert (cosine > 0.95).all(), cosine
    decayed, _ = delta_plain(proj, dict(c, w0=c["w0"] + 32), heads, dim, eps)
    raw = (decayed[-1] / c["norm_w"] / plain.sigmoid(proj[-1, 3 * hd:4 * hd])).reshape(heads, dim)
    cosine = (raw * first_value).sum(-1) / np.linalg.norm(raw, axis=-1) / np.linalg.norm(first_value, axis=-1)
    assert (np.abs(cosine) < 0.7).all()


def attention_case(rng, n, heads, kv_heads, dim, vdim, dtype):
    cols = heads * dim + kv_heads * (dim + vdim) + heads
    qkv = rng.standard_normal((n, cols)).astype(np.float32)
    qkv = dev(qkv, dtype)
    return qkv, qkv.float().cpu().numpy().astype(np.float64)


def attention_plain(q64, heads, kv_heads, dim, vdim, scale, slope, rate, window):
    n = q64.shape[0]
    q = q64[:, :heads * dim].reshape(n, heads, dim)
    k = q64[:, heads * dim:heads * dim + kv_heads * dim].reshape(n, kv_heads, dim)
    v = q64[:, (heads + kv_heads) * dim:(heads + kv_heads) * dim + kv_heads * vdim].reshape(n, kv_heads, vdim)
    gate = plain.sigmoid(q64[:, -heads:])
    out = np.empty((n, heads, vdim))
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = plain.distance_scores(q[:, h], k[:, g], scale, slope[h], rate[h], window)
        e = np.exp(s - s.max(-1, keepdims=True))
        out[:, h] = (e / e.sum(-1, keepdims=True)) @ v[:, g] * gate[:, h:h + 1]
    return out.reshape(n, heads * vdim)


def run_attention(qkv, pieces, heads, kv_heads, dim, vdim, scale, slope, rate, window, blocks,
                  splits=1):
    """The tokens of one sequence in `pieces`, through a cache whose blocks are `blocks`."""
    k_cache = torch.full((8, kv_heads, 64, dim), float("nan"), dtype=qkv.dtype, device=DEV)
    v_cache = torch.full((8, kv_heads, 64, vdim), float("nan"), dtype=qkv.dtype, device=DEV)
    table = torch.as_tensor([blocks], dtype=torch.int32, device=DEV)
    out, at = [], 0
    for n in pieces:
        step = step_of([n], [0], [at])
        rows = qkv[at:at + n]
        ops.kv_store(rows, heads * dim, (heads + kv_heads) * dim, step.positions, step.token_seq,
                     table, k_cache, v_cache)
        out.append(ops.distance_attention(rows, k_cache, v_cache, step.positions, step.token_seq,
                                          table, heads, scale, window, dev(slope), dev(rate),
                                          gate_off=(heads + kv_heads) * dim + kv_heads * vdim,
                                          splits=splits))
        at += n
    return torch.cat(out).float().cpu().numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window",
                         [(4, 2, 16, 24, 37), (1, 1, 64, 64, 64), (3, 1, 8, 8, 1), (2, 2, 32, 16, None),
                          (8, 4, 16, 32, 130), (2, 1, 72, 40, 65), (1, 1, 160, 264, 5),
                          (6, 1, 20, 12, 40), (5, 5, 128, 256, 70), (12, 2, 8, 200, None)])
def test_distance_attention_in_a_prompt_in_pieces_and_decoded(heads, kv_heads, dim, vdim, window, dtype):
    rng = np.random.default_rng(dim + vdim)
    n = 200
    qkv, q64 = attention_case(rng, n, heads, kv_heads, dim, vdim, dtype)
    slope, rate = rng.uniform(0, 2, heads), rng.uniform(0.1, 0.5, heads)
    slope32, rate32 = slope.astype(np.float32), rate.astype(np.float32)
    want = attention_plain(q64, heads, kv_heads, dim, vdim, 0.2, slope32.astype(np.float64),
                           rate32.astype(np.float64), window)
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    blocks = [5, 2, 7, 0]
    whole = run_attention(qkv, [n], heads, kv_heads, dim, vdim, 0.2, slope32, rate32, window, blocks)
    assert np.abs(whole - want).max() <= tol * np.abs(want).max()
    cut = run_attention(qkv, [2, 61, 1, 1, 64, 3] + [1] * 68, heads, kv_heads, dim, vdim, 0.2,
                        slope32, rate32, window, blocks)
    assert np.array_equal(cut, whole)
    # the plain form (a key at a time) and warps that share a token's keys: the same numbers
    # within rounding, and each of them the same to the bit however the tokens are cut
    for splits in (0, 2, 16):
        other = run_attention(qkv, [n], heads, kv_heads, dim, vdim, 0.2, slope32, rate32, window,
                              blocks, splits)
        assert np.abs(other - want).max() <= tol * np.abs(want).max(), splits
        again = run_attention(qkv, [150] + [1] * 50, heads, kv_heads, dim, vdim, 0.2, slope32,
                              rate32, window, blocks, splits)
        assert np.array_equal(again, other), splits


@pytest.mark.parametrize("window", [1, 2, 63, 64, 65, 72, 128])
def test_a_key_that_stands_out_just_inside_and_just_outside_the_window(window):
    """Token `at` gets a key that every later query scores far above all others. The query
    `window - 1` tokens later still sees it and returns its value; the next one does not. The
    same whether the queries come in the prompt or one by one, wherever the block borders are."""
    rng = np.random.default_rng(window)
    heads = kv_heads = 1
    dim, vdim, n = 16, 8, 300
    for at in (0, 1, 63, 64, 100):
        base = 0.05 * rng.standard_normal((n, 2 * dim + vdim + 1)).astype(np.float32)
        direction = np.ones(dim, dtype=np.float32)
        base[:, :dim] += 4 * direction                      # every query looks along it
        base[at, dim:2 * dim] += 6 * direction              # one key lies along it
        base[:, -1] = 8.0                                   # gates open
        base[at, 2 * dim:2 * dim + vdim] = np.arange(1, vdim + 1)
        qkv = dev(base)
        slope = rate = np.zeros(1, dtype=np.float32)
        inside, outside = at + window - 1, at + window
        for pieces, splits in (([n], 1), ([at + 1] + [1] * (n - at - 1), 1), ([n], 0),
                               ([at + 1] + [1] * (n - at - 1), 4)):
            out = run_attention(qkv, pieces, heads, kv_heads, dim, vdim, 1.0, slope, rate, window,
                                [3, 1, 6, 4, 0], splits)
            marked = np.arange(1, vdim + 1)
            assert np.abs(out[inside] - marked).max() < 1e-2, (window, at, "inside")
            assert np.abs(out[outside]).max() < 0.5, (window, at, "outside")
            if window > 1:
                assert np.abs(out[at + 1] - marked).max() < 1e-2


def test_the_distance_penalty_takes_weight_from_far_keys():
    """Equal scores everywhere: the weights are (1 + rate * d)^(-slope), exactly."""
    n, dim = 90, 8
    base = np.zeros((n, 2 * dim + 1 + 1), dtype=np.float32)
    base[:, -1] = 30.0
    base[:, 2 * dim] = np.arange(n)                         # the value is the position
    slope, rate = np.array([1.5], dtype=np.float32), np.array([0.25], dtype=np.float32)
    out = run_attention(dev(base), [n], 1, 1, dim, 1, 1.0, slope, rate, None, [0, 1])
    d = np.arange(n)
    for i in (0, 1, 50, 89):
        w = (1 + 0.25 * (i - d[:i + 1])) ** -1.5
        assert abs(out[i, 0] - (w * d[:i + 1]).sum() / w.sum()) < 1e-4 * max(i, 1)


def test_gelu_tanh():
    z = torch.linspace(-6, 6, 1001, device=DEV)
    want = plain.gelu_tanh(z.cpu().numpy().astype(np.float64))
    assert np.abs(ops.gelu_tanh(z).cpu().numpy() - want).max() < 1e-6
    zb = z.to(torch.bfloat16)
    want = plain.gelu_tanh(zb.float().cpu().numpy().astype(np.float64))
    assert np.abs(ops.gelu_tanh(zb).float().cpu().numpy() - want).max() < 2e-2
