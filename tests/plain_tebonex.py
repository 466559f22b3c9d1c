"""A plain, slow Tebonex in NumPy float64: whole sequences only, no cache, no batching, no
step function. One function for each mechanism of the design, written from its equations;
nothing here imports the package under test.

Notation: n tokens, W the model's width, H heads, G key/value heads, D a head's key size,
Dv its value size, S streams. Linear weights are [out, in] and applied as `x @ w.T`.
"""

from __future__ import annotations

import numpy as np

from plain_model import read_model_folder      # the tests' own safetensors reader

__all__ = ["read_model_folder", "rms", "sigmoid", "gelu_tanh", "token_shift", "streams_read",
           "streams_write", "decay", "delta_rule_scan", "delta_rule_mixer", "distance_scores",
           "log_distance_attention", "dense_mlp", "forward", "generate"]

DECAY_SCALE = np.exp(-0.5)
KEY_EPS = 1e-6


def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def token_shift(h, shift, before=None):
    """Row i blended with row i - 1 as both were BEFORE the blend; the row before the first
    is `before` (zeros at the start of a sequence)."""
    first = np.zeros((1, h.shape[1])) if before is None else np.asarray(before)[None, :]
    prev = np.concatenate([first, h[:-1]])
    return h + (prev - h) * shift


def streams_read(xs, w_in):
    """xs: [S, n, W]; the sublayer's input before its norm."""
    return np.einsum("s,snw->nw", w_in, xs)


def streams_write(xs, y, w_mix, w_out):
    """Every new stream t from all the old ones: sum_s mix[s, t] x_s + out[t] y."""
    return np.einsum("st,snw->tnw", w_mix, xs) + w_out[:, None, None] * y[None]


def decay(h, w1, w2, w0):
    """The per-channel decay in (exp(-exp(-1/2)), 1): exp(-c sigmoid(w0 + W2 tanh(W1 h)))."""
    return np.exp(-DECAY_SCALE * sigmoid(np.tanh(h @ w1.T) @ w2.T + w0))


def delta_rule_scan(r, k, v, w, a, state=None):
    """r, k, v, w, a: [n, H, D]. Returns (o [n, H, D], final state [H, D, D]); state rows are
    key channels, columns value channels. Both correction terms read the old state."""
    n, heads, dim = r.shape
    state = np.zeros((heads, dim, dim)) if state is None else state.copy()
    out = np.empty((n, heads, dim))
    for i in range(n):
        unit = k[i] / np.sqrt(np.sum(k[i] ** 2, axis=-1, keepdims=True) + KEY_EPS)
        along = np.einsum("hk,hkv->hv", unit, state)                     # u^T S
        state = (w[i][:, :, None] * state
                 - (a[i] * unit)[:, :, None] * along[:, None, :]
                 + k[i][:, :, None] * v[i][:, None, :])
        out[i] = np.einsum("hkv,hk->hv", state, r[i])
    return out, state


def delta_rule_mixer(h, t, p, heads, dim, eps):
    """`t`: tensors by name, `p`: the mixer's prefix ('l0.mix.')."""
    n = h.shape[0]
    split = lambda name: (h @ t[p + name].T).reshape(n, heads, dim)
    w = decay(h, t[p + "w1"], t[p + "w2"], t[p + "w0"]).reshape(n, heads, dim)
    a = sigmoid(h @ t[p + "a"].T + t[p + "a.b"]).reshape(n, heads, dim)
    o, _ = delta_rule_scan(split("r"), split("k"), split("v"), w, a)
    o = rms(o, eps).reshape(n, heads * dim) * t[p + "norm"] * sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T


def distance_scores(q, k, scale, slope, rate, window):
    """q [n, D], k [n, D] of one head -> scores [n, n] with -inf where j is not visible."""
    n = q.shape[0]
    dist = np.arange(n)[:, None] - np.arange(n)[None, :]
    s = q @ k.T * scale - slope * np.log1p(rate * np.maximum(dist, 0))
    seen = dist >= 0
    if window:
        seen &= dist < window
    return np.where(seen, s, -np.inf)


def log_distance_attention(h, t, p, heads, kv_heads, dim, vdim, scale, window):
    n = h.shape[0]
    q = (h @ t[p + "q"].T + t[p + "q.b"]).reshape(n, heads, dim)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).reshape(n, kv_heads, dim)
    v = (h @ t[p + "v"].T + t[p + "v.b"]).reshape(n, kv_heads, vdim)
    gate = sigmoid(h @ t[p + "g"].T)                                     # [n, H]
    out = np.empty((n, heads, vdim))
    for head in range(heads):
        group = head // (heads // kv_heads)
        s = distance_scores(q[:, head], k[:, group], scale, t[p + "r1"][head], t[p + "r2"][head],
                            window)
        e = np.exp(s - s.max(-1, keepdims=True))
        out[:, head] = (e / e.sum(-1, keepdims=True)) @ v[:, group] * gate[:, head:head + 1]
    return out.reshape(n, heads * vdim) @ t[p + "o"].T + t[p + "o.b"]


def dense_mlp(h, up, down):
    return gelu_tanh(h @ up.T) @ down.T


def forward(config: dict, t: dict, ids, layer_sums: list | None = None) -> np.ndarray:
    """float64 logits [n, vocab]; `layer_sums` receives the sum of the streams after every
    layer."""
    eps = config["norm"]["eps"]
    streams = config.get("streams")
    x = t["embed"][np.asarray(ids, dtype=np.int64)] * config["embedding"]["scale"]
    xs = np.stack([x] * (streams or 1))
    ones, eye = np.ones(streams or 1), np.eye(streams or 1)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        for q in (1, 2):
            if q == 2 and layer["mlp"] is None:
                continue
            if streams is None:
                w_in, w_mix, w_out = ones, eye, ones
            else:
                w_in, w_mix, w_out = (t[f"{p}hc{q}.{name}"] for name in ("in", "mix", "out"))
            h = rms(streams_read(xs, w_in), eps) * t[f"{p}norm{q}"]
            m = layer["mixer"]
            if q == 2:
                y = dense_mlp(h, t[p + "mlp.up"], t[p + "mlp.down"])
            else:
                h = token_shift(h, t[p + "shift"])
                if layer["type"] == "general_delta":
                    y = delta_rule_mixer(h, t, p + "mix.", m["heads"], m["dim"], eps)
                else:
                    y = log_distance_attention(
                        h, t, p + "mix.", m["heads"], m.get("kv_heads", m["heads"]), m["dim"],
                        m.get("vdim", m["dim"]), m["scale"], (m.get("mask") or {}).get("size"))
            xs = streams_write(xs, y, w_mix, w_out)
        if layer_sums is not None:
            layer_sums.append(xs.sum(0))
    return (rms(xs.sum(0), eps) * t["final.norm"]) @ t["head"].T


def generate(config, t, prompt, new_tokens: int) -> list:
    ids, out = list(prompt), []
    for _ in range(new_tokens):
        token = int(forward(config, t, ids)[-1].argmax())
        out.append(token)
        ids.append(token)
    return out
