"""Tebonex: a decoder whose layers are listed one by one in config.json.

    {"architecture": "Tebonex", "vocab": V, "width": W, "streams": S,
     "embedding": {"scale": c}, "norm": {"eps": e},
     "layers": [{"type": "general_delta", "mixer": {"heads": H, "dim": D},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv,
                                                "scale": s, "mask": {"size": w}},
                 "mlp": null}, ...]}

Every layer is a pre-norm block over `streams` copies of the residual stream
(`StreamBlockSpec`; without a `streams` key the plain residual sum), its mixer reads
its input blended with the previous token's (token shift), and the mixer is either
the delta-rule recurrence (`DeltaRuleSpec`) or windowed attention with a logarithmic
distance penalty (`LogDistanceAttentionSpec`). Tensors are named `embed`,
`l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.hc1.*`, `l<i>.shift`, `final.norm`,
`head`. The inner size of the decay's low-rank pair is not in config.json: it is the
first size of the tensor `l<i>.mix.w1` (a model written from a configuration alone
gives it as `decay_rank`).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .specs import (ConfigError, DeltaRuleSpec, DenseMLPSpec, LayerCall, LogDistanceAttentionSpec,
                    ModelSpec, NormSpec, StreamBlockSpec)

DEFAULT_DECAY_RANK = 16
#: the design has no table of positions; this bounds a sequence only through the cache
MAX_POSITIONS = 1 << 22


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@dataclass(frozen=True)
class TebonexLayer:
    type: str                       # "general_delta" | "attention"
    heads: int
    dim: int
    kv_heads: int = 0               # attention only
    vdim: int = 0
    scale: float = 0.0
    window: Optional[int] = None
    ff: Optional[int] = None        # None: no feed-forward
    decay_rank: int = 0             # general_delta only


@dataclass(frozen=True)
class TebonexConfig:
    vocab: int
    width: int
    streams: Optional[int]          # None: one stream, plain residual sum
    embedding_scale: float
    eps: float
    layers: tuple
    initializer_range: float = 0.05

    architecture = "Tebonex"
    needs_tensor_shapes = True

    @classmethod
    def from_dict(cls, raw: dict, tensor_shapes: dict | None = None) -> "TebonexConfig":
        problems = []

        def positive_int(where, holder, key, default=None):
            v = holder.get(key, default) if isinstance(holder, dict) else default
            if not _is_int(v) or v <= 0:
                problems.append(f"{where}{key}: expected a positive integer, config.json has {v!r}")
                return 1
            return v

        vocab = positive_int("", raw, "vocab")
        width = positive_int("", raw, "width")
        streams = raw.get("streams")
        if streams is not None:
            streams = positive_int("", raw, "streams")
            if streams > 16:
                problems.append(f"streams: {streams} is more than the 16 the kernels take")
        scale = (raw.get("embedding") or {}).get("scale", 1.0)
        if not _is_number(scale):
            problems.append(f"embedding.scale: expected a number, config.json has {scale!r}")
            scale = 1.0
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
            heads = positive_int(where + "mixer.", m, "heads")
            dim = positive_int(where + "mixer.", m, "dim")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                    problems.append(f"{where}mlp: only kind 'dense' is built, config.json has "
                                    f"{mlp!r}")
                else:
                    ff = positive_int(where + "mlp.", mlp, "ff")
            if kind == "general_delta":
                rank = m.get("decay_rank")
                shape = (tensor_shapes or {}).get(f"l{i}.mix.w1")
                if shape is not None and len(shape) == 2:
                    rank = int(shape[0])
                if rank is None:
                    rank = DEFAULT_DECAY_RANK
                if not _is_int(rank) or rank <= 0:
                    problems.append(f"{where}mixer.decay_rank: expected a positive integer")
                    rank = 1
                if dim > 256:
                    problems.append(f"{where}mixer.dim: {dim} is more than the 256 the "
                                    "recurrence kernel takes")
                layers.append(TebonexLayer("general_delta", heads, dim, ff=ff, decay_rank=rank))
            elif kind == "attention":
                kv_heads = positive_int(where + "mixer.", m, "kv_heads", heads)
                vdim = positive_int(where + "mixer.", m, "vdim", dim)
                if heads % kv_heads:
                    problems.append(f"{where}mixer: {heads} heads are not a multiple of "
                                    f"{kv_heads} kv_heads")
                s = m.get("scale")
                if not _is_number(s):
                    problems.append(f"{where}mixer.scale: expected a number, config.json has {s!r}")
                    s = 1.0
                mask, window = m.get("mask"), None
                if mask is not None:
                    window = positive_int(where + "mixer.mask.", mask, "size")
                if max(dim, vdim) > 512:
                    problems.append(f"{where}mixer: dim {dim} / vdim {vdim} are more than the "
                                    "512 the attention kernel takes")
                layers.append(TebonexLayer("attention", heads, dim, kv_heads, vdim, float(s),
                                           window, ff))
            else:
                problems.append(f"{where}type: {kind!r} is neither 'general_delta' nor 'attention'")
        if problems:
            raise ConfigError("config.json cannot describe a Tebonex model:\n    "
                              + "\n    ".join(problems))
        return cls(vocab=vocab, width=width, streams=streams, embedding_scale=float(scale),
                   eps=float(eps), layers=tuple(layers),
                   initializer_range=float(raw.get("initializer_range", 0.05)))

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        layers = []
        for layer in self.layers:
            if layer.type == "general_delta":
                mixer = {"heads": layer.heads, "dim": layer.dim, "decay_rank": layer.decay_rank}
            else:
                mixer = {"heads": layer.heads, "kv_heads": layer.kv_heads, "dim": layer.dim,
                         "vdim": layer.vdim, "scale": layer.scale}
                if layer.window is not None:
                    mixer["mask"] = {"size": layer.window}
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
        raw = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps},
               "layers": layers, "initializer_range": self.initializer_range}
        if self.streams is not None:
            raw["streams"] = self.streams
        return raw

    def model_spec(self) -> ModelSpec:
        norm = NormSpec(size=self.width, eps=self.eps, suffix="")
        blocks, ignore = [], []
        for i, layer in enumerate(self.layers):
            if layer.type == "general_delta":
                mixer = DeltaRuleSpec(hidden=self.width, heads=layer.heads, head_dim=layer.dim,
                                      decay_rank=layer.decay_rank, eps=self.eps)
            else:
                mixer = LogDistanceAttentionSpec(
                    hidden=self.width, heads=layer.heads, kv_heads=layer.kv_heads,
                    head_dim=layer.dim, value_dim=layer.vdim, scale=layer.scale,
                    window=layer.window)
            ffn = None if layer.ff is None else DenseMLPSpec(hidden=self.width,
                                                             intermediate=layer.ff)
            if ffn is None:      # a checkpoint may still carry the unused sublayer's constants
                ignore += [f"l{i}.norm2", f"l{i}.hc2.*"]
            blocks.append(StreamBlockSpec(
                prefix=f"l{i}.", mixer=mixer, mixer_norm=norm, ffn=ffn,
                ffn_norm=None if ffn is None else norm, streams=self.streams or 1,
                connections=self.streams is not None, token_shift=True))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden=self.width,
            blocks=tuple(blocks),
            run_order=tuple(LayerCall(block=i, cache=i) for i in range(len(blocks))),
            final_norm=norm, tie_head=False, max_positions=MAX_POSITIONS, embed_name="embed",
            final_norm_name="final.norm", head_name="head", stored_dtype="bfloat16",
            init_std=self.initializer_range, embed_scale=self.embedding_scale,
            ignore_tensors=tuple(ignore), streams=self.streams or 1)


register_architecture(TebonexConfig.architecture, TebonexConfig)
