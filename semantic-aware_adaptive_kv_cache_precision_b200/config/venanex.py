"""Venanex: a decoder whose layers are listed one by one in config.json, some of them run
several times in a row.

    {"architecture": "Venanex", "vocab": V, "width": W, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads": H, "dim": D, "rot_dim": R, "vdim": Dv, "kv_rank": C,
                           "q_rank": Q, "scale": s,
                           "rot": {"base": b, "dims": R,
                                   "scaling": {"factor": f, "original": n, "fast": x, "slow": y}}},
                 "mlp": {"kind": "moe", "router": {"experts": E, "top": k},
                         "expert": {"ff": F, "limit": l}, "shared": {"ff": Fs, "limit": ls}}},
                {"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": s,
                           "diff": d, "mask": {"size": c}},
                 "mlp": null}, ...]}

Every layer has a layer norm before and after each sublayer (`SandwichBlockSpec`). Its mixer
is attention over a cached latent with a rotated key part that all heads share
(`LatentAttentionSpec`) or two-map differential attention inside chunks of positions
(`DifferentialAttentionSpec`); its feed-forward is a mixture of clamped gated experts with a
shared one (`RoutedExpertsSpec`) or absent. Layers `start .. stop-1` run `times` times in a
row with the same weights, every pass with a cache of its own, and before the first layer of
each pass the stream becomes `W [x; x0]` (`loop.in`, x0 the embedding's output). The output
head is the embedding table. Tensors: `embed`, `loop.in`, `l<i>.norm1`, `l<i>.norm1b`,
`l<i>.norm2`, `l<i>.norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .specs import (ClampedExpertSpec, ConfigError, DifferentialAttentionSpec, LatentAttentionSpec,
                    LayerCall, ModelSpec, NormSpec, RampScaling, RotarySpec, RoutedExpertsSpec,
                    SandwichBlockSpec)

#: positions the rotation's table may be asked for; a sequence is bounded by the cache
MAX_POSITIONS = 1 << 22
#: the activation's constant in an expert: y = g * sigmoid(ALPHA * g) * (u + 1)
EXPERT_ALPHA = 1.702
#: cosines and sines of a stretched rotation are multiplied by SLOPE * ln(factor) + 1
MAGNITUDE_SLOPE = 0.1


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@dataclass(frozen=True)
class VenanexLayer:
    type: str                       # "latent_attention" | "attention"
    mixer: dict                     # the entry's own keys, checked
    mlp: Optional[dict]             # None: no feed-forward


@dataclass(frozen=True)
class VenanexConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    loop: Optional[tuple]           # (start, stop, times) or None
    initializer_range: float = 0.05

    architecture = "Venanex"

    @classmethod
    def from_dict(cls, raw: dict) -> "VenanexConfig":
        problems = []

        def positive_int(where, holder, key):
            v = holder.get(key) if isinstance(holder, dict) else None
            if not _is_int(v) or v <= 0:
                problems.append(f"{where}{key}: expected a positive integer, config.json has {v!r}")
                return 1
            return v

        def number(where, holder, key, low=None):
            v = holder.get(key) if isinstance(holder, dict) else None
            if not _is_number(v) or (low is not None and v <= low):
                problems.append(f"{where}{key}: expected a number"
                                + (f" above {low}" if low is not None else "")
                                + f", config.json has {v!r}")
                return 1.0
            return float(v)

        vocab = positive_int("", raw, "vocab")
        width = positive_int("", raw, "width")
        eps = (raw.get("norm") or {}).get("eps")
        if not _is_number(eps) or eps < 0:
            problems.append(f"norm.eps: expected a number >= 0, config.json has {eps!r}")
            eps = 0.0
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            problems.append("layers: expected a list of layers")
            listed = []
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                problems.append(f"{where}mixer: expected an object with the mixer's sizes")
                continue
            kind, m = entry.get("type"), entry["mixer"]
            mw = where + "mixer."
            if kind == "latent_attention":
                mixer = {k: positive_int(mw, m, k) for k in ("heads", "dim", "rot_dim", "vdim",
                                                             "kv_rank")}
                mixer["q_rank"] = None if m.get("q_rank") is None else positive_int(mw, m, "q_rank")
                mixer["scale"] = number(mw, m, "scale")
                rot = m.get("rot")
                if not isinstance(rot, dict):
                    problems.append(f"{mw}rot: expected an object with base and dims")
                    rot = {}
                dims = positive_int(mw + "rot.", rot, "dims")
                if dims != mixer["rot_dim"] or dims % 2:
                    problems.append(f"{mw}rot.dims: {dims} must be even and equal rot_dim "
                                    f"{mixer['rot_dim']}")
                turned = {"base": number(mw + "rot.", rot, "base", 0.0), "dims": dims}
                sc = rot.get("scaling")
                if sc is not None:
                    sw = mw + "rot.scaling."
                    turned["scaling"] = {k: number(sw, sc, k, 0.0)
                                         for k in ("factor", "original", "fast", "slow")}
                    if turned["base"] == 1.0:
                        problems.append(f"{mw}rot.base: 1 leaves the ramp of the scaling undefined")
                mixer["rot"] = turned
                if mixer["kv_rank"] + mixer["rot_dim"] > 640 or mixer["kv_rank"] > 512:
                    problems.append(f"{mw}kv_rank + rot_dim up to 640 and kv_rank up to 512 are "
                                    "what the attention kernel takes")
            elif kind == "attention":
                mixer = {k: positive_int(mw, m, k) for k in ("heads", "dim")}
                mixer["kv_heads"] = mixer["heads"] if m.get("kv_heads") is None \
                    else positive_int(mw, m, "kv_heads")
                mixer["vdim"] = mixer["dim"] if m.get("vdim") is None else positive_int(mw, m, "vdim")
                if mixer["heads"] % mixer["kv_heads"]:
                    problems.append(f"{mw}{mixer['heads']} heads are not a multiple of "
                                    f"{mixer['kv_heads']} kv_heads")
                mixer["scale"] = number(mw, m, "scale")
                mixer["diff"] = number(mw, m, "diff")
                mask = m.get("mask")
                mixer["mask"] = None if mask is None else \
                    {"size": positive_int(mw + "mask.", mask, "size")}
                if mixer["dim"] > 256 or mixer["vdim"] > 512:
                    problems.append(f"{mw}dim up to 256 and vdim up to 512 are what the "
                                    "attention kernel takes")
            else:
                problems.append(f"{where}type: {kind!r} is neither 'latent_attention' nor "
                                "'attention'")
                continue
            mlp = entry.get("mlp")
            if mlp is not None:
                lw = where + "mlp."
                if not isinstance(mlp, dict) or mlp.get("kind", "moe") != "moe":
                    problems.append(f"{lw}kind: only 'moe' is built, config.json has {mlp!r}")
                    mlp = None
                else:
                    router, exp, shared = mlp.get("router"), mlp.get("expert"), mlp.get("shared")
                    out = {"kind": "moe",
                           "router": {"experts": positive_int(lw + "router.", router, "experts"),
                                      "top": positive_int(lw + "router.", router, "top")},
                           "expert": {"ff": positive_int(lw + "expert.", exp, "ff"),
                                      "limit": number(lw + "expert.", exp, "limit", 0.0)}}
                    if out["router"]["top"] > out["router"]["experts"]:
                        problems.append(f"{lw}router.top is more than router.experts")
                    if out["router"]["top"] > 32 or out["router"]["experts"] > 1024:
                        problems.append(f"{lw}router: up to 1024 experts and top 32 are built")
                    if shared is not None:
                        out["shared"] = {"ff": positive_int(lw + "shared.", shared, "ff"),
                                         "limit": number(lw + "shared.", shared, "limit", 0.0)}
                    mlp = out
            layers.append(VenanexLayer(kind, mixer, mlp))
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict) or not all(_is_int(loop.get(k)) for k in
                                                     ("start", "stop", "times")):
                problems.append("loop: expected integers start, stop and times")
                loop = None
            else:
                loop = (loop["start"], loop["stop"], loop["times"])
                if not (0 <= loop[0] < loop[1] <= max(len(layers), len(listed))) or loop[2] < 1:
                    problems.append(f"loop: start {loop[0]}, stop {loop[1]}, times {loop[2]} do "
                                    f"not name a run of the {len(listed)} layers")
        if problems:
            raise ConfigError("config.json cannot describe a Venanex model:\n    "
                              + "\n    ".join(problems))
        return cls(vocab=vocab, width=width, eps=float(eps), layers=tuple(layers), loop=loop,
                   initializer_range=float(raw.get("initializer_range", 0.05)))

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        layers = []
        for layer in self.layers:
            mixer = {k: v for k, v in layer.mixer.items() if v is not None}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": layer.mlp})
        raw = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.eps}, "layers": layers,
               "initializer_range": self.initializer_range}
        if self.loop is not None:
            raw["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return raw

    def run_order(self) -> tuple:
        """Every layer run as a `LayerCall` with a cache entry of its own; the first call of
        each pass of the repeated run takes the input up again."""
        n = len(self.layers)
        if self.loop is None:
            runs = [(i, False) for i in range(n)]
        else:
            start, stop, times = self.loop
            runs = [(i, False) for i in range(start)]
            for _ in range(times):
                runs += [(i, i == start) for i in range(start, stop)]
            runs += [(i, False) for i in range(stop, n)]
        return tuple(LayerCall(block=i, cache=c, mix_input=first)
                     for c, (i, first) in enumerate(runs))

    def model_spec(self) -> ModelSpec:
        norm = NormSpec(size=self.width, eps=self.eps, kind="layer_norm", suffix="")
        blocks, ignore = [], []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "latent_attention":
                sc = m["rot"].get("scaling")
                position = RotarySpec(
                    head_dim=m["rot_dim"], rotary_dim=m["rot"]["dims"], theta=m["rot"]["base"],
                    max_positions=MAX_POSITIONS,
                    scaling=None if sc is None else RampScaling(
                        factor=sc["factor"], original=sc["original"], fast=sc["fast"],
                        slow=sc["slow"], magnitude_slope=MAGNITUDE_SLOPE))
                mixer = LatentAttentionSpec(
                    hidden=self.width, heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
                    value_dim=m["vdim"], kv_rank=m["kv_rank"], q_rank=m["q_rank"],
                    scale=m["scale"], eps=self.eps, position=position)
            else:
                mixer = DifferentialAttentionSpec(
                    hidden=self.width, heads=m["heads"], kv_heads=m["kv_heads"],
                    head_dim=m["dim"], value_dim=m["vdim"], scale=m["scale"],
                    chunk=None if m["mask"] is None else m["mask"]["size"], diff=m["diff"],
                    eps=self.eps)
            ffn = None
            if layer.mlp is not None:
                shared = layer.mlp.get("shared")
                ffn = RoutedExpertsSpec(
                    hidden=self.width, experts=layer.mlp["router"]["experts"],
                    top=layer.mlp["router"]["top"],
                    expert=ClampedExpertSpec(layer.mlp["expert"]["ff"], layer.mlp["expert"]["limit"],
                                             EXPERT_ALPHA),
                    shared=None if shared is None else ClampedExpertSpec(
                        shared["ff"], shared["limit"], EXPERT_ALPHA))
            else:      # a checkpoint may still carry the absent sublayer's norms
                ignore += [f"l{i}.norm2", f"l{i}.norm2b"]
            blocks.append(SandwichBlockSpec(prefix=f"l{i}.", mixer=mixer, ffn=ffn, norm=norm))
        order = self.run_order()
        mixes = any(call.mix_input for call in order)
        if not mixes:
            ignore.append("loop.in")
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden=self.width,
            blocks=tuple(blocks), run_order=order, final_norm=norm, tie_head=True,
            max_positions=MAX_POSITIONS, embed_name="embed", final_norm_name="final.norm",
            stored_dtype="bfloat16", init_std=self.initializer_range,
            ignore_tensors=tuple(ignore), input_mix_name="loop.in" if mixes else None)


register_architecture(VenanexConfig.architecture, VenanexConfig)
