"""A plain, slow Venanex in NumPy float64: whole sequences only, no cache, no batching, no
step function. One function for each mechanism of the design, written from its equations;
nothing here imports the package under test.

Notation: n tokens, W the model's width, H heads, G key/value heads, D a head's key size,
Dv its value size, R the rotated size, C the latent's size. Linear weights are [out, in] and
applied as `x @ w.T`.
"""

from __future__ import annotations

import math

import numpy as np

from plain_model import read_model_folder      # the tests' own safetensors reader

__all__ = ["read_model_folder", "layer_norm", "rms_norm", "sigmoid", "yarn_frequencies",
           "rotate_half", "softmax_rows", "latent_attention", "differential_attention",
           "expert", "routed_experts", "router_margins", "moe", "layer", "run_order", "forward", "generate"]


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis; var is the mean squared deviation."""
    mean = x.mean(-1, keepdims=True)
    var = ((x - mean) ** 2).mean(-1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) (* w): eps inside the root."""
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return y if w is None else y * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def yarn_frequencies(rot):
    """(frequencies [dims / 2], magnitude) of a rotation `rot` = {base, dims, scaling?}. With
    scaling {factor, original, fast, slow} the frequencies whose wavelength is long against
    the original context are divided by factor, the short ones stay, a linear ramp over the
    pair index lies between; cos and sin are both multiplied by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], float(rot["base"])
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor = float(sc["factor"])

    def pair_of(turns):       # the pair index whose wavelength makes `turns` turns in `original`
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, rot):
    """x: [n, ..., dims]; pair (i, i + dims/2) turned by the angle position * f_i."""
    f, mag = yarn_frequencies(rot)
    half = rot["dims"] // 2
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (half,)
    cos, sin = (np.cos(a) * mag).reshape(shape), (np.sin(a) * mag).reshape(shape)
    u, v = x[..., :half], x[..., half:2 * half]
    return np.concatenate([u * cos - v * sin, v * cos + u * sin, x[..., 2 * half:]], axis=-1)


def softmax_rows(s, visible):
    s = np.where(visible, s, -np.inf)
    e = np.exp(s - s.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def latent_attention(h, t, p, m, eps):
    """`t`: tensors by name, `p`: the mixer's prefix ('l0.mix.'), `m`: its config entry."""
    n = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(n)
    if m.get("q_rank"):
        cq = rms_norm(h @ t[p + "dq"].T, t[p + "dq.norm"], eps)
        q = (cq @ t[p + "uq"].T).reshape(n, H, D + R)
    else:                                     # no query latent: straight from the input
        q = (h @ t[p + "q"].T).reshape(n, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_half(q[..., D:], pos, m["rot"])
    down = h @ t[p + "dkv"].T
    c = rms_norm(down[:, :C], t[p + "dkv.norm"], eps)
    k_rot = rotate_half(down[:, C:], pos, m["rot"])                  # [n, R], shared by heads
    k_plain = (c @ t[p + "uk"].T).reshape(n, H, D)
    v = (c @ t[p + "uv"].T).reshape(n, H, Dv)
    visible = pos[:, None] >= pos[None, :]
    out = np.empty((n, H, Dv))
    for i in range(H):
        s = (q_plain[:, i] @ k_plain[:, i].T + q_rot[:, i] @ k_rot.T) * m["scale"]
        out[:, i] = softmax_rows(s, visible) @ v[:, i]
    return out.reshape(n, H * Dv) @ t[p + "o"].T


def differential_attention(h, t, p, m, eps):
    """Two softmax maps a head over the same values, o = a1 - lambda a2, unit norm a head,
    (1 - diff), an output gate from the mixer's own input."""
    n = h.shape[0]
    H, D = m["heads"], m["dim"]
    G, Dv = m.get("kv_heads", H), m.get("vdim", D)
    q = (h @ t[p + "q"].T).reshape(n, H, 2, D)
    k = (h @ t[p + "k"].T).reshape(n, G, 2, D)
    v = (h @ t[p + "v"].T).reshape(n, G, Dv)
    pos = np.arange(n)
    visible = pos[:, None] >= pos[None, :]
    mask = m.get("mask")
    if mask:
        visible &= (pos[:, None] // mask["size"]) == (pos[None, :] // mask["size"])
    lam = (math.exp(float(np.sum(t[p + "lq1"] * t[p + "lk1"])))
           - math.exp(float(np.sum(t[p + "lq2"] * t[p + "lk2"]))) + m["diff"])
    out = np.empty((n, H, Dv))
    for i in range(H):
        g = i // (H // G)
        a = [softmax_rows(q[:, i, j] @ k[:, g, j].T * m["scale"], visible) @ v[:, g]
             for j in (0, 1)]
        out[:, i] = rms_norm(a[0] - lam * a[1], None, eps) * (1.0 - m["diff"])
    gated = out.reshape(n, H * Dv) * sigmoid(h @ t[p + "g"].T)
    return gated @ t[p + "o"].T


def expert(h, t, p, limit):
    g = np.minimum(h @ t[p + "gate"].T, limit)
    u = np.clip(h @ t[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ t[p + "down"].T


def routed_experts(h, t, p, experts, top):
    """(chosen [n, top], weights [n, top]): the `top` largest sigmoid scores, as they are."""
    s = sigmoid(h @ t[p + "router"].T)
    chosen = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, -1)


def router_margins(h, t, p, experts, top):
    """For each token, how far the last chosen expert's logit lies above the best one left
    out (inf when every expert is chosen): a small margin is a close call that rounding may
    turn."""
    z = np.sort(h @ t[p + "router"].T, axis=-1)[:, ::-1]
    return z[:, top - 1] - z[:, top] if top < experts else np.full(h.shape[0], np.inf)


def moe(h, t, p, m, margins=None):
    n = h.shape[0]
    chosen, weights = routed_experts(h, t, p, m["router"]["experts"], m["router"]["top"])
    if margins is not None:
        margins.append(router_margins(h, t, p, m["router"]["experts"], m["router"]["top"]))
    out = np.zeros((n, t[p + "e0.down"].shape[0]))
    for i in range(n):
        for e, w in zip(chosen[i], weights[i]):       # the weight multiplies the expert's INPUT
            out[i] += expert(w * h[i:i + 1], t, f"{p}e{e}.", m["expert"]["limit"])[0]
    if m.get("shared"):
        out += expert(h, t, p + "shared.", m["shared"]["limit"]) * sigmoid(h @ t[p + "shared.sg"].T)
    return out


def layer(x, t, i, entry, eps, margins=None):
    p = f"l{i}."
    h = layer_norm(x, t[p + "norm1"], eps)
    if entry["type"] == "latent_attention":
        y = latent_attention(h, t, p + "mix.", entry["mixer"], eps)
    elif entry["type"] == "attention":
        y = differential_attention(h, t, p + "mix.", entry["mixer"], eps)
    else:
        raise ValueError(entry["type"])
    x = x + layer_norm(y, t[p + "norm1b"], eps)
    if entry.get("mlp") is not None:
        y = moe(layer_norm(x, t[p + "norm2"], eps), t, p + "mlp.", entry["mlp"], margins)
        x = x + layer_norm(y, t[p + "norm2b"], eps)
    return x


def run_order(config):
    """[(layer, first of a pass?)]: layers start..stop-1 run `times` times in a row."""
    n, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def forward(config, t, ids, layers_out=None, margins=None):
    """Logits [n, vocab] of a whole sequence; `layers_out` (a list) receives the residual
    stream after every layer run, `margins` (a list) every routed layer run's
    `router_margins`."""
    eps = config["norm"]["eps"]
    x0 = t["embed"][np.asarray(ids)]
    x = x0.copy()
    for i, first in run_order(config):
        if first:
            x = np.concatenate([x, x0], axis=-1) @ t["loop.in"].T
        x = layer(x, t, i, config["layers"][i], eps, margins)
        if layers_out is not None:
            layers_out.append(x.copy())
    return layer_norm(x, t["final.norm"], eps) @ t["embed"].T


def generate(config, t, prompt, new_tokens):
    ids = list(prompt)
    for _ in range(new_tokens):
        ids.append(int(np.argmax(forward(config, t, ids)[-1])))
    return ids[len(prompt):]
