"""The kernels of the Venanex mechanisms, each alone against the plain functions, on inputs
made so that a fault shows: a key far back that stands out among hundreds, a key that stands
out just inside and just outside a chunk (in a prompt and decoded, at block borders), the
first tokens of a sequence, the two maps of a head with a large lambda, experts that nobody
chose, every expert chosen, rows whose norm's mean is far from zero."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_venanex as plain
from semantic_aware_adaptive_kv_cache_precision_b200 import ops
from semantic_aware_adaptive_kv_cache_precision_b200.ops import mixture

pytestmark = pytest.mark.gpu
DEV = "cuda"
TYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype, device=DEV).contiguous()


def rounded(a, dtype):
    """What the device holds of `a` in `dtype`, as float64."""
    return dev(a, dtype).float().cpu().numpy().astype(np.float64)


def i32(a):
    return torch.as_tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def close(got, want, dtype, what=""):
    got = got.float().cpu().numpy().astype(np.float64)
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    worst = np.abs(got - want).max()
    assert worst <= tol * np.abs(want).max() + 1e-7, f"{what}: differs by {worst:.3e}"


# -- layer norm -----------------------------------------------------------------------------

@pytest.mark.parametrize("width", [1, 7, 100, 256, 1000, 4100])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_layer_norm_and_the_step_between_two_sublayers(width, wdtype):
    rng = np.random.default_rng(width)
    n, eps = 5, 1e-5
    x = rng.standard_normal((n, width)) + 30.0          # a mean far from zero
    y = 4.0 * rng.standard_normal((n, width)) - 7.0
    w1, w2 = (rounded(1 + 0.2 * rng.standard_normal(width), wdtype) for _ in range(2))
    want = plain.layer_norm(x, w1, eps)
    got = ops.layer_norm(dev(x), dev(w1, wdtype), eps, torch.float32)
    x32 = dev(x).cpu().numpy().astype(np.float64)
    want = plain.layer_norm(x32, w1, eps)
    assert np.abs(got.cpu().numpy() - want).max() <= 2e-5 * max(np.abs(want).max(), 1.0)
    rows = i32([3, 0, 3])
    some = ops.layer_norm(dev(x), dev(w1, wdtype), eps, torch.float32, rows=rows)
    assert torch.equal(some, got[[3, 0, 3]])
    # x += norm(y) w2; out = norm(x) w1, in one pass, and the first half alone
    stream = dev(x)
    y32 = dev(y).cpu().numpy().astype(np.float64)
    out = ops.layer_norm(stream, dev(w1, wdtype), eps, torch.float32, add=dev(y),
                         add_weight=dev(w2, wdtype))
    want_x = x32 + plain.layer_norm(y32, w2, eps)
    assert np.abs(stream.cpu().numpy() - want_x).max() <= 2e-6 * np.abs(want_x).max()
    want_h = plain.layer_norm(want_x, w1, eps)
    assert np.abs(out.cpu().numpy() - want_h).max() <= 3e-5 * max(np.abs(want_h).max(), 1.0)
    alone = dev(x)
    assert ops.layer_norm(alone, None, eps, torch.float32, add=dev(y),
                          add_weight=dev(w2, wdtype)) is None
    assert torch.equal(alone, stream)
    low = ops.layer_norm(dev(x), dev(w1, wdtype), eps, torch.bfloat16)
    assert low.dtype == torch.bfloat16
    assert np.abs(low.float().cpu().numpy() - want).max() <= 1e-2 * max(np.abs(want).max(), 1.0)


# -- a cache of one sequence a slot, for the attention kernels --------------------------------

class Cache:
    """Blocks of 64 positions handed out in a scrambled order, so that a wrong block shows."""

    def __init__(self, kv_heads, k_row, v_row, dtype, blocks=40, seed=0):
        self.keys = torch.full((blocks, kv_heads, 64, k_row), float("nan"), dtype=dtype, device=DEV)
        self.values = None if v_row is None else torch.full((blocks, kv_heads, 64, v_row),
                                                            float("nan"), dtype=dtype, device=DEV)
        self.order = np.random.default_rng(seed).permutation(blocks).tolist()
        self.tables = {}

    def table(self, seqs, length):
        need = -(-length // 64)
        rows = []
        for s in seqs:
            mine = self.tables.setdefault(s, [])
            while len(mine) < need:
                mine.append(self.order.pop())
            rows.append(mine + [-1] * (8 - len(mine)))
        return i32(rows)

    def put(self, seq, k, v=None):
        """k: [n, kv_heads, k_row] for positions 0..n-1 of sequence `seq`."""
        table = self.table([seq], len(k))[0].tolist()
        for p in range(len(k)):
            self.keys[table[p // 64], :, p % 64] = dev(k[p], self.keys.dtype)
            if v is not None:
                self.values[table[p // 64], :, p % 64] = dev(v[p], self.values.dtype)


def step_for(seq_index, positions):
    return SimpleNamespace(positions=i32(positions), token_seq=i32(seq_index))


def plain_attention(q, k, v, scale, visible):
    """q: [n, D], k: [m, D], v: [m, Dv] -> [n, Dv]."""
    return plain.softmax_rows(q @ k.T * scale, visible) @ v


# -- attention over a latent: split queries, values inside the key rows -------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,rank,rot", [(4, 40, 8), (1, 36, 6), (5, 128, 32), (2, 512, 64)])
def test_latent_attention_finds_a_key_far_back(dtype, heads, rank, rot):
    """Among 700 keys one, far back, stands out for one head; a prompt's pieces and single
    tokens with 1 to 16 warps a token give what the plain attention gives."""
    T = TYPES[dtype]
    rng = np.random.default_rng(rank)
    n, width, scale = 700, rank + rot, 0.3
    rows = 0.3 * rng.standard_normal((n, width))
    qa = 0.3 * rng.standard_normal((n, heads, rank))
    qb = 0.3 * rng.standard_normal((n, heads, rot))
    far, asker = 13, 650
    rows[far] *= 4.0
    qa[asker, heads - 1] = rows[far, :rank] * 3.0          # one score far above the rest
    qb[asker, heads - 1] = rows[far, rank:] * 3.0
    rows, qa, qb = rounded(rows, T), rounded(qa, T), rounded(qb, T)
    cache = Cache(1, width, None, T, seed=1)
    cache.put(0, rows[:, None, :])
    q = np.concatenate([qa, qb], axis=-1)
    visible = np.arange(n)[:, None] >= np.arange(n)[None, :]
    want = np.stack([plain_attention(q[:, h], rows, rows[:, :rank], scale, visible)
                     for h in range(heads)], axis=1).reshape(n, heads * rank)
    weights = plain.softmax_rows(q[:, heads - 1] @ rows.T * scale, visible)
    assert weights[asker, far] > 0.5                       # the far key is what the asker sees
    # the second source is a slice of a wider projection output, as in the mixer
    wide = torch.zeros((n, heads, 5 + rot), dtype=T, device=DEV)
    wide[:, :, 5:] = dev(qb, T)
    table = cache.table([0], n)
    for lo, hi, splits, across in ((0, n, 1, 1), (600, n, 1, 1), (asker, asker + 1, 1, 1),
                                   (asker, asker + 1, 4, 1), (asker, asker + 1, 16, 1), (0, 3, 1, 1),
                                   (0, 1, 2, 1), (asker, asker + 2, 4, 4), (asker - 1, asker + 1, 8, 16),
                                   (2, 4, 2, 8), (asker, asker + 1, 1, -1), (asker - 1, asker + 2, 1, -4),
                                   (asker, asker + 1, 1, -16), (0, 2, 1, -2), (40, 41, 1, -8)):
        if dtype == "float32" and splits > 1:
            continue
        first = across < 0                      # (negative: the heads-first form)
        across = abs(across)
        step = step_for([0] * (hi - lo), range(lo, hi))
        got = ops.cached_attention(dev(qa[lo:hi], T), cache.keys, None, step.positions,
                                   step.token_seq, table, heads, width, rank, scale,
                                   q2=wide[lo:hi, :, 5:], q_split=rank, splits=splits,
                                   key_splits=across, warp_stage=splits in (4, 8),
                                   heads_first=first)
        close(got, want[lo:hi], T, f"positions {lo}..{hi}, {splits} warps, {across} blocks")
        if across > 1:      # the tickets were left clean: the same again
            again = ops.cached_attention(dev(qa[lo:hi], T), cache.keys, None, step.positions,
                                         step.token_seq, table, heads, width, rank, scale,
                                         q2=wide[lo:hi, :, 5:], q_split=rank, splits=splits,
                                         key_splits=across, heads_first=first)
            assert torch.equal(again, got)


# -- two maps a head inside chunks ------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,chunk", [
    (4, 2, 16, 24, 37), (1, 1, 64, 64, 64), (6, 2, 20, 12, 3), (3, 3, 24, 36, 100),
    (4, 1, 128, 320, 128), (2, 2, 8, 8, None)])
def test_two_maps_inside_chunks_at_their_edges(dtype, heads, kv_heads, dim, vdim, chunk):
    """A key stands out for map 1 at the first position of a chunk and for map 2 at the last
    position of the chunk before: queries just inside see the one and never the other."""
    T = TYPES[dtype]
    rng = np.random.default_rng(dim + vdim)
    n, scale, lam, diff, eps = 300, 0.4, 0.8, 0.3, 1e-6
    size = chunk or n
    edge = (150 // size) * size if chunk else 0            # a chunk's first position
    k = 0.4 * rng.standard_normal((n, kv_heads, 2, dim))
    v = rng.standard_normal((n, kv_heads, vdim))
    q = 0.4 * rng.standard_normal((n, heads, 2, dim))
    gate = rng.standard_normal((n, heads * vdim))
    k[edge] *= 3.0
    if edge:
        k[edge - 1] *= 3.0
    group = heads // kv_heads
    for ask in {edge, min(edge + 1, n - 1), min(edge + size - 1, n - 1)}:
        for h in range(heads):
            q[ask, h, 0] = k[edge, h // group, 0] * 4.0
            if edge:
                q[ask, h, 1] = k[edge - 1, h // group, 1] * 4.0      # outside: must not be seen
    k, v, q, gate = rounded(k, T), rounded(v, T), rounded(q, T), rounded(gate, T)
    pos = np.arange(n)
    visible = pos[:, None] >= pos[None, :]
    if chunk:
        visible &= (pos[:, None] // chunk) == (pos[None, :] // chunk)
    want = np.empty((n, heads, vdim))
    for h in range(heads):
        g = h // group
        a1 = plain_attention(q[:, h, 0], k[:, g, 0], v[:, g], scale, visible)
        a2 = plain_attention(q[:, h, 1], k[:, g, 1], v[:, g], scale, visible)
        want[:, h] = plain.rms_norm(a1 - lam * a2, None, eps) * (1 - diff)
    want = want.reshape(n, heads * vdim) * plain.sigmoid(gate)
    cache = Cache(kv_heads, 2 * dim, vdim, T, seed=2)
    cache.put(0, k.reshape(n, kv_heads, 2 * dim), v)
    table = cache.table([0], n)
    q_cols = heads * 2 * dim
    fused = dev(np.concatenate([q.reshape(n, q_cols), np.zeros((n, 3)), gate], axis=1), T)
    last = min(edge + size, n)
    for lo, hi, splits, across in ((0, n, 1, 1), (edge - 2 if edge else 0, edge + 3, 1, 1),
                                   (edge, edge + 1, 1, 1), (edge + 1, edge + 2, 2, 1),
                                   (last - 1, last, 8, 1), (0, 2, 1, 1), (130, 200, 1, 1),
                                   (last - 2, last, 2, 4), (edge, edge + 2, 4, 2),
                                   (last - 1, last, 1, -1), (last - 2, last, 1, -4),
                                   (edge, edge + 2, 1, -2), (edge + 1, edge + 2, 1, -8)):
        if dtype == "float32" and splits > 1:
            continue
        first = across < 0                      # (negative: the heads-first form)
        across = abs(across)
        step = step_for([0] * (hi - lo), range(lo, hi))
        part = fused[lo:hi]
        got = ops.cached_attention(part[:, :q_cols].view(hi - lo, heads * 2, dim), cache.keys,
                                   cache.values, step.positions, step.token_seq, table, heads, dim,
                                   vdim, scale, maps=2, chunk=chunk, lam=lam, out_scale=1 - diff,
                                   eps=eps, gate_elem_off=q_cols + 3, splits=splits,
                                   key_splits=across, warp_stage=splits in (2, 8),
                                   heads_first=first)
        close(got, want[lo:hi], T, f"positions {lo}..{hi}, {splits} warps, {across} blocks")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_over_two_sequences_of_one_step(dtype):
    """Tokens of two sequences in one step read their own blocks."""
    T = TYPES[dtype]
    rng = np.random.default_rng(5)
    heads, dim, vdim, scale = 2, 16, 16, 0.5
    lens = {0: 130, 1: 70}
    cache = Cache(1, 2 * dim, vdim, T, seed=3)
    data = {}
    for s, n in lens.items():
        k = rounded(0.5 * rng.standard_normal((n, 1, 2 * dim)), T)
        v = rounded(rng.standard_normal((n, 1, vdim)), T)
        q = rounded(0.5 * rng.standard_normal((n, heads, 2, dim)), T)
        cache.put(s, k, v)
        data[s] = (k, v, q)
    table = torch.cat([cache.table([0], 130), cache.table([1], 70)])
    take = [(1, 69), (0, 129), (0, 64), (1, 0)]
    seq, pos = [s for s, _ in take], [p for _, p in take]
    q = np.stack([data[s][2][p] for s, p in take])
    got = ops.cached_attention(dev(q.reshape(4, heads * 2, dim), T), cache.keys, cache.values,
                               i32(pos), i32(seq), table, heads, dim, vdim, scale, maps=2,
                               chunk=64, lam=0.5, out_scale=1.0, eps=1e-6)
    if dtype == "bfloat16":                      # one block and three blocks a token
        for across in (1, 3):
            other = ops.cached_attention(dev(q.reshape(4, heads * 2, dim), T), cache.keys,
                                         cache.values, i32(pos), i32(seq), table, heads, dim, vdim,
                                         scale, maps=2, chunk=64, lam=0.5, out_scale=1.0, eps=1e-6,
                                         heads_first=True, key_splits=across)
            assert float((other.float() - got.float()).abs().max()) <= 2e-2
    for i, (s, p) in enumerate(take):
        k, v, qq = data[s]
        visible = (np.arange(lens[s]) <= p) & (np.arange(lens[s]) // 64 == p // 64)
        row = []
        for h in range(heads):
            a = [plain_attention(qq[p:p + 1, h, m], k[:, 0, m * dim:(m + 1) * dim], v[:, 0], scale,
                                 visible[None, :]) for m in (0, 1)]
            row.append(plain.rms_norm(a[0] - 0.5 * a[1], None, 1e-6))
        close(got[i:i + 1], np.concatenate(row, axis=1), T, f"sequence {s} position {p}")


# -- the latent's preparation and the rotation -------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("q_rank,rank,rot", [(24, 40, 8), (0, 56, 16), (28, 36, 6), (96, 512, 64)])
def test_latent_prepare_norms_rotates_and_stores(dtype, q_rank, rank, rot):
    from semantic_aware_adaptive_kv_cache_precision_b200.config import RampScaling, RotarySpec
    from semantic_aware_adaptive_kv_cache_precision_b200.parts import RotaryHalf
    T = TYPES[dtype]
    rng = np.random.default_rng(rank)
    scaling = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}
    rot_config = {"base": 10000.0, "dims": rot, "scaling": scaling}
    part = RotaryHalf(RotarySpec(rot, rot, 10000.0, 512, scaling=RampScaling(4.0, 64, 8.0, 2.0)),
                      "", dtype)
    part.prepare(DEV, 512)
    positions = [0, 1, 63, 64, 200, 511]
    n, eps = len(positions), 1e-5
    down = rng.standard_normal((n, q_rank + rank + rot)) * 3.0
    wq = rounded(1 + 0.2 * rng.standard_normal(max(q_rank, 1)), T)
    wkv = rounded(1 + 0.2 * rng.standard_normal(rank), T)
    cache = Cache(1, rank + rot, None, T, blocks=9, seed=4)
    view = SimpleNamespace(keys=cache.keys, block_table=cache.table([0], 512))
    step = step_for([0] * n, positions)
    got_q = ops.latent_prepare(dev(down), q_rank, rank, rot, dev(wq, T) if q_rank else None,
                               dev(wkv, T), eps, step, view, part.cos, part.sin, T)
    d32 = dev(down).cpu().numpy().astype(np.float64)
    if q_rank:
        close(got_q, plain.rms_norm(d32[:, :q_rank], wq, eps), T, "the query latent")
    else:
        assert got_q is None
    want = np.concatenate([plain.rms_norm(d32[:, q_rank:q_rank + rank], wkv, eps),
                           plain.rotate_half(d32[:, q_rank + rank:], positions, rot_config)], axis=1)
    table = view.block_table[0].tolist()
    stored = torch.stack([cache.keys[table[p // 64], 0, p % 64] for p in positions])
    close(stored, want, T, "the cache rows")
    # a slice of every head, rotated in place
    heads, plain_dim = 3, 10
    x = rng.standard_normal((n, heads, plain_dim + rot))
    xd = dev(x.reshape(n, -1), T)
    before = xd.float().cpu().numpy().astype(np.float64).reshape(n, heads, -1)
    ops.rotate_heads(xd, plain_dim + rot, plain_dim, heads, rot, step.positions, part.cos, part.sin)
    want = np.concatenate([before[..., :plain_dim],
                           plain.rotate_half(before[..., plain_dim:], positions, rot_config)], axis=-1)
    close(xd.view(n, heads, -1), want, T, "rotated heads")


# -- the mixture ----------------------------------------------------------------------------------

def plain_mixture(h, t, experts, top, limit, weight_input=True):
    m = {"router": {"experts": experts, "top": top}, "expert": {"ff": 0, "limit": limit}}
    return plain.moe(h, t, "", m)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,width,experts,top,ff", [
    (1, 64, 2, 1, 96), (77, 96, 6, 2, 48), (5, 100, 3, 3, 50), (200, 64, 40, 4, 24),
    (33, 72, 7, 1, 130), (300, 200, 5, 2, 72), (9, 36, 4, 2, 20)])
def test_routed_experts_against_the_plain_mixture(dtype, n, width, experts, top, ff):
    T = TYPES[dtype]
    rng = np.random.default_rng(n + experts)
    limit, alpha = 1.1, 1.702
    h = rounded(rng.standard_normal((n, width)), T)
    t = {"router": rng.standard_normal((experts, width)) * 0.3}
    if experts > 4:
        t["router"][1] = -10.0 * np.abs(t["router"][1])      # hardly ever chosen ...
        t["router"][1][0] = 0.0
        h[:, 0] = np.abs(h[:, 0])
    for e in range(experts):
        t[f"e{e}.gate"] = rounded(rng.standard_normal((ff, width)) * 0.2, T)
        t[f"e{e}.up"] = rounded(rng.standard_normal((ff, width)) * 0.2, T)
        t[f"e{e}.down"] = rounded(rng.standard_normal((width, ff)) * 0.2, T)
    logits = mixture.router_logits(dev(h, T), dev(t["router"]))
    z = logits.cpu().numpy().astype(np.float64)
    exact = h @ dev(t["router"]).cpu().numpy().astype(np.float64).T
    assert np.abs(z - exact).max() <= 1e-5 * np.abs(exact).max()
    routing = mixture.route(logits, experts, top)
    chosen = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    assert np.array_equal(routing.chosen.cpu().numpy(), chosen)
    assert np.allclose(routing.weights.cpu().numpy(), plain.sigmoid(np.take_along_axis(z, chosen, -1)),
                       rtol=1e-6)
    offsets = routing.offsets.cpu().numpy()
    assert offsets[0] == 0 and offsets[-1] == n * top
    assert np.array_equal(np.diff(offsets), np.bincount(chosen.ravel(), minlength=experts))
    slots = routing.slot_of.cpu().numpy() if False else None
    rows = mixture.gather_rows(dev(h, T), routing, True)
    slot_of = routing.slot_of.cpu().numpy()
    assert sorted(slot_of.ravel().tolist()) == list(range(n * top))      # every row once
    for e in range(experts):                                            # ... sorted by expert
        mine = slot_of[chosen == e]
        assert ((mine >= offsets[e]) & (mine < offsets[e + 1])).all()
    stack = lambda name: dev(np.stack([t[f"e{e}.{name}"] for e in range(experts)]), T)
    act = mixture.grouped_product(rows, routing, stack("gate"), stack("up"), limit, alpha)
    products = mixture.grouped_product(act, routing, stack("down"), None)
    out = mixture.combine(products, routing, False)
    # the plain mixture on what the device computed with: w h rounded once to the type
    want = np.zeros((n, width))
    w = routing.weights.cpu().numpy().astype(np.float64)
    for i in range(n):
        for k in range(top):
            x = rounded(w[i, k] * h[i:i + 1], T)
            want[i] += plain.expert(x, t, f"e{chosen[i, k]}.", limit)[0]
    close(out, want, T, "the routed experts")
    # with a shared expert and its gate
    shared = rng.standard_normal((n, width))
    gate = rng.standard_normal((n, 3))
    both = mixture.combine(products, routing, False, dev(shared), dev(gate)[:, 1])
    close(both, want + shared * plain.sigmoid(gate[:, 1:2]), T, "with the shared expert")
    again = mixture.route(logits, experts, top)         # the counts were left clean
    assert torch.equal(again.offsets, routing.offsets)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_activation(dtype):
    T = TYPES[dtype]
    rng = np.random.default_rng(3)
    both = rounded(3.0 * rng.standard_normal((9, 2 * 37)), T)
    got = mixture.clamped_act(dev(both, T), 1.5, 1.702)
    g = np.minimum(both[:, :37], 1.5)
    u = np.clip(both[:, 37:], -1.5, 1.5)
    close(got, g * plain.sigmoid(1.702 * g) * (u + 1), T)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_product_a_head(dtype):
    T = TYPES[dtype]
    rng = np.random.default_rng(4)
    n, heads, k, m = 19, 3, 24, 40
    x = rounded(rng.standard_normal((n, heads, k + 8)), T)
    w = rounded(rng.standard_normal((heads, m, k)), T)
    out = torch.zeros((n, heads, m + 5), dtype=T, device=DEV)
    ops.per_head(dev(x, T)[:, :, 8:], dev(w, T), out[:, :, :m])
    want = np.einsum("nhk,hmk->nhm", x[:, :, 8:], w)
    close(out[:, :, :m], want, T)
    assert float(out[:, :, m:].abs().max()) == 0.0
