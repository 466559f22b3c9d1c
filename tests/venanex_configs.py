"""Small Venanex configurations for the tests. Every size differs between them and from layer
to layer, and some take the values that make branches coincide elsewhere: one expert a token
and several, as many choices as experts, no shared expert, a layer without a feed-forward, no
repeated run at all, a run that starts after the first layer, a run of one pass, chunks of one
cache block, of fewer and of more positions, no chunks, as many key/value heads as heads,
values wider and narrower than keys, a rotation with and without stretched wavelengths, no
query latent, sizes that no vector access divides, and the widths of a large model's heads."""


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, scaling, mlp):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
             "scale": scale, "rot": rot}
    if q_rank is not None:
        mixer["q_rank"] = q_rank
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, scale, diff, chunk, mlp):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
             "diff": diff}
    if chunk is not None:
        mixer["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top},
           "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


MIXED = {"architecture": "Venanex", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
         "initializer_range": 0.12, "loop": {"start": 1, "stop": 3, "times": 3},
         "layers": [latent(4, 16, 8, 24, 40, 24, 0.2, 10000.0, (4.0, 64, 8.0, 2.0),
                           moe(6, 2, 48, 1.0, (32, 3.0))),
                    attention(4, 2, 16, 24, 0.25, 0.5, 37, None),
                    latent(3, 24, 16, 16, 56, None, 0.16, 500.0, None, moe(5, 5, 40, 0.7)),
                    attention(2, 2, 32, 16, 0.18, 0.3, None, moe(3, 1, 64, 2.5, (80, 0.9)))]}
PLAIN = {"architecture": "Venanex", "vocab": 150, "width": 64, "norm": {"eps": 1e-6},
         "initializer_range": 0.08,
         "layers": [attention(1, 1, 64, 64, 0.125, 0.4, 64, moe(2, 1, 96, 1.2, (16, 1.0))),
                    latent(1, 8, 32, 8, 16, 48, 0.3, 100.0, (2.0, 32, 16.0, 1.0), None)]}
ODD = {"architecture": "Venanex", "vocab": 131, "width": 100, "norm": {"eps": 3e-6},
       "initializer_range": 0.1, "loop": {"start": 0, "stop": 1, "times": 1},
       "layers": [latent(5, 12, 6, 20, 36, 28, 0.25, 777.0, (1.5, 40, 4.0, 0.5),
                         moe(3, 2, 50, 1.5, (30, 2.0))),
                  attention(6, 2, 20, 12, 0.22, 0.45, 3, moe(7, 3, 22, 0.8)),
                  attention(3, 3, 24, 36, 0.2, 0.6, 100, None)]}
WIDE = {"architecture": "Venanex", "vocab": 97, "width": 128, "norm": {"eps": 1e-6},
        "initializer_range": 0.06, "loop": {"start": 0, "stop": 2, "times": 2},
        "layers": [latent(2, 128, 64, 128, 512, 96, 0.07, 10000.0, (40.0, 4096, 32.0, 1.0),
                          moe(4, 2, 128, 7.0, (64, 7.0))),
                   attention(4, 1, 128, 320, 0.088, 0.2, 128, None),
                   attention(2, 1, 64, 256, 0.125, 0.35, 70, moe(9, 4, 32, 1.0))]}
CONFIGS = {"mixed": (MIXED, 21), "plain": (PLAIN, 22), "odd": (ODD, 23), "wide": (WIDE, 24)}
