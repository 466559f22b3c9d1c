"""Small Tebonex configurations for the tests: every size differs between them and from
layer to layer, and some take the values that make branches coincide elsewhere (one stream,
one head, a window of one token, a window of exactly a cache block, values wider or narrower
than keys, a layer without a feed-forward, no `streams` key at all)."""


def delta(heads, dim, rank, ff):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def attention(heads, kv_heads, dim, vdim, scale, window, ff):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer,
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


MIXED = {"architecture": "Tebonex", "vocab": 211, "width": 96, "streams": 3,
         "embedding": {"scale": 12.0}, "norm": {"eps": 1e-5}, "initializer_range": 0.08,
         "layers": [attention(4, 2, 16, 24, 0.3, 37, 160), delta(3, 16, 8, 128),
                    attention(2, 2, 32, 16, 0.2, None, None), delta(2, 48, 5, 72)]}
PLAIN = {"architecture": "Tebonex", "vocab": 150, "width": 64,
         "embedding": {"scale": 7.0}, "norm": {"eps": 1e-6}, "initializer_range": 0.1,
         "layers": [delta(1, 64, 16, 96), attention(1, 1, 64, 64, 0.125, 64, 96),
                    attention(3, 1, 8, 8, 0.5, 1, None), delta(4, 8, 3, 40)]}
SINGLE = {"architecture": "Tebonex", "vocab": 97, "width": 128, "streams": 1,
          "embedding": {"scale": 3.0}, "norm": {"eps": 3e-6}, "initializer_range": 0.06,
          "layers": [delta(4, 32, 4, 200), attention(8, 4, 16, 32, 0.25, 130, 136)]}
# sizes that no vector access divides: a width of 100, heads of 24 and 40, four streams.
# (Its seed is one whose first tokens are well conditioned: after one token a head's state is
# k v^T, so its normed output is v / rms(v) times the SIGN of r.k, and a seed that draws r.k
# next to zero for some token turns rounding into a flipped sign, in any implementation.)
ODD = {"architecture": "Tebonex", "vocab": 131, "width": 100, "streams": 4,
       "embedding": {"scale": 9.0}, "norm": {"eps": 1e-5}, "initializer_range": 0.09,
       "layers": [delta(5, 24, 7, 50), attention(5, 5, 24, 40, 0.2, 3, 90),
                  attention(6, 2, 12, 20, 0.3, 100, None), delta(1, 100, 2, 33)]}
CONFIGS = {"mixed": (MIXED, 11), "plain": (PLAIN, 12), "single": (SINGLE, 13), "odd": (ODD, 15)}
