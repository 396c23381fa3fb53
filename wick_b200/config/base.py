"""Typed model configuration and the architecture registry.

A configuration is a frozen dataclass whose fields are read from the
architecture's own ``config.json`` keys.  The registry maps the architecture
name found in ``config.json`` (``architectures[0]``, else ``model_type``) to an
:class:`Architecture`: the configuration class and the function that turns a
configuration into a :class:`~wick_b200.models.spec.ModelSpec`.

Reference behaviour: wick ``src/config.rs:55-68`` (name lookup and the error
for an unknown architecture) and ``src/config.rs:135-151`` (``config.json`` plus
the extra stop tokens of ``generation_config.json``).
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Callable, Dict, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A ``config.json`` that cannot be turned into a model."""


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.

    ``architecture`` is the registry key the configuration was loaded under.
    Subclasses add their own fields and implement :meth:`from_json` and
    :meth:`to_json`; ``to_json`` must write keys that ``from_json`` reads back to
    an equal configuration (the random-weights mode relies on it).
    """

    architecture: str

    @classmethod
    def from_json(cls, j: Mapping[str, Any], architecture: str) -> "ModelConfig":
        raise NotImplementedError

    def to_json(self) -> Dict[str, Any]:
        raise NotImplementedError

    # Sizes every engine component may ask for, whatever the architecture.
    @property
    def vocab(self) -> int:
        raise NotImplementedError

    @property
    def max_position(self) -> int:
        raise NotImplementedError

    @property
    def stop_token_ids(self) -> Tuple[int, ...]:
        return ()


@dataclasses.dataclass(frozen=True)
class Architecture:
    """One registry entry.

    names:      every string of ``config.json`` that selects this entry.
    config_cls: the :class:`ModelConfig` subclass.
    build_spec: ``config -> ModelSpec`` (layers, their parts, the run order and
                the tensor names); the only architecture-specific code.
    """

    names: Tuple[str, ...]
    config_cls: type
    build_spec: Callable[[ModelConfig], Any]


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    for n in arch.names:
        _REGISTRY[n] = arch
    return arch


def architecture_names() -> Tuple[str, ...]:
    return tuple(sorted(_REGISTRY))


def get_architecture(name: str) -> Architecture:
    try:
        return _REGISTRY[name]
    except KeyError:
        raise ConfigError(
            f"unsupported architecture {name} (supported: {', '.join(architecture_names())})"
        ) from None


def architecture_name_of(j: Mapping[str, Any]) -> str:
    """``architectures[0]`` if present, else ``model_type`` (config.rs:56-62)."""
    archs = j.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    mt = j.get("model_type")
    if isinstance(mt, str):
        return mt
    raise ConfigError("config.json has no architectures")


def config_from_json(j: Mapping[str, Any]) -> ModelConfig:
    name = architecture_name_of(j)
    arch = get_architecture(name)
    return arch.config_cls.from_json(j, name)


def _token_ids(v: Any) -> Tuple[int, ...]:
    """An int or a list of ints (config.rs:46-52); anything else is no id."""
    if isinstance(v, bool):
        return ()
    if isinstance(v, int):
        return (v,)
    if isinstance(v, list):
        return tuple(int(x) for x in v if isinstance(x, int) and not isinstance(x, bool))
    return ()


def load_config(model_dir: str) -> ModelConfig:
    """Read ``<model_dir>/config.json`` and merge the stop tokens that
    ``generation_config.json`` lists (config.rs:135-151)."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            j = json.load(f)
    except OSError as e:
        raise ConfigError(f"{path}: {e.strerror or e}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: {e}") from None
    if not isinstance(j, dict):
        raise ConfigError(f"{path}: not a JSON object")
    cfg = config_from_json(j)
    gpath = os.path.join(model_dir, "generation_config.json")
    extra: Tuple[int, ...] = ()
    try:
        with open(gpath, "r", encoding="utf-8") as f:
            g = json.load(f)
        if isinstance(g, dict):
            extra = _token_ids(g.get("eos_token_id"))
    except (OSError, json.JSONDecodeError):
        pass
    if extra and hasattr(cfg, "eos_token_ids"):
        merged = list(cfg.eos_token_ids)
        for t in extra:
            if t not in merged:
                merged.append(t)
        cfg = dataclasses.replace(cfg, eos_token_ids=tuple(merged))
    return cfg


# helpers for from_json implementations -------------------------------------

def need_int(j: Mapping[str, Any], key: str) -> int:
    v = j.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or v < 0:
        raise ConfigError(f"config.json: missing {key}")
    return int(v)


def opt_int(j: Mapping[str, Any], key: str, default: Optional[int]) -> Optional[int]:
    v = j.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or v < 0:
        return default
    return int(v)


def opt_float(j: Mapping[str, Any], key: str, default: float) -> float:
    v = j.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        return default
    return float(v)


def opt_bool(j: Mapping[str, Any], key: str, default: bool) -> bool:
    v = j.get(key)
    return v if isinstance(v, bool) else default


token_ids = _token_ids
