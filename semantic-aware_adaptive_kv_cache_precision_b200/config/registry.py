"""One registry from an architecture's name (config.json `architectures[0]`) to
the class that reads its configuration. The model itself is always built by
`engine.model.DecoderModel` from the `ModelSpec` that class produces."""

from __future__ import annotations

import json
from pathlib import Path

from .specs import ConfigError

_ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_class: type) -> None:
    """Make `name` loadable. `config_class` needs `from_dict(raw) -> config`,
    and the config needs `model_spec() -> ModelSpec` and `to_dict()`."""
    _ARCHITECTURES[name] = config_class


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_name(raw: dict) -> str:
    """The model class a config.json names: the first entry of its `architectures` list, or
    the string under `architecture`."""
    if isinstance(raw.get("architecture"), str) and "architectures" not in raw:
        return raw["architecture"]
    names = raw.get("architectures")
    if not isinstance(names, (list, tuple)) or not names or not isinstance(names[0], str):
        raise ConfigError("config.json has neither an `architectures` list nor an "
                          "`architecture` string naming the model class; "
                          f"known architectures: {', '.join(known_architectures())}")
    return names[0]


def config_from_dict(raw: dict, tensor_shapes: dict | None = None):
    """`tensor_shapes` (tensor name -> shape, from a checkpoint's header): for architectures
    whose config.json leaves a size to the tensors (`needs_tensor_shapes` on the class)."""
    name = architecture_name(raw)
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered; known architectures: "
                          f"{', '.join(known_architectures())}")
    cls = _ARCHITECTURES[name]
    if getattr(cls, "needs_tensor_shapes", False):
        return cls.from_dict(raw, tensor_shapes)
    return cls.from_dict(raw)


def config_from_folder(folder):
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist: a model folder holds config.json and "
                          "model.safetensors")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not JSON: {exc}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    shapes = None
    try:
        cls = _ARCHITECTURES.get(architecture_name(raw))
    except ConfigError:
        cls = None
    if getattr(cls, "needs_tensor_shapes", False):
        from ..weights.loader import Checkpoint
        from ..weights.safetensors_io import WeightError
        try:
            checkpoint = Checkpoint(folder)
            shapes = {n: tuple(checkpoint.info(n).shape) for n in checkpoint.names()}
        except WeightError:
            shapes = None          # the loader will say what is wrong with the folder
    return config_from_dict(raw, shapes)
