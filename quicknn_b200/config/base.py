"""Typed configuration base and the architecture registry.

A configuration is a frozen dataclass whose fields are the keys of the
architecture's own ``config.json``.  Every size and constant the model uses comes
from here; nothing downstream carries a default of its own.

The reference reads its values ad hoc with ``Config.GetValue<T>(key, default)``
and raises one combined "Invalid Gemma 2 geometry/configuration" error
(src/models/QuickNN.Models.Gemma2.pas:76-95) and dispatches on the
``model_type`` string with an if/else chain (src/models/QuickNN.Models.LLM.pas:153-188).
Here each violated rule is reported by name and the dispatch is a table.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Callable, Dict, List, Optional, Tuple, Type


class ConfigError(ValueError):
    """Raised with every violated rule listed, one per line."""

    def __init__(self, problems: List[str], where: str = "config"):
        self.problems = list(problems)
        super().__init__(f"invalid {where}:\n  - " + "\n  - ".join(self.problems))


_MISSING = object()


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of all typed configurations.

    Subclasses declare fields; a field with ``metadata={"key": "json_key"}`` reads
    that key, otherwise the field's own name.  ``metadata={"required": True}`` makes
    absence an error even if the dataclass needs a placeholder default.
    """

    @classmethod
    def architecture_names(cls) -> Tuple[str, ...]:  # pragma: no cover - abstract
        raise NotImplementedError

    # ---- reading -------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        problems: List[str] = []
        values: Dict[str, Any] = {}
        known = set()
        for f in dataclasses.fields(cls):
            key = f.metadata.get("key", f.name)
            known.add(key)
            v = raw.get(key, _MISSING)
            if v is _MISSING:
                if f.metadata.get("required", False):
                    problems.append(f"missing required key '{key}'")
                    continue
                if f.default is not dataclasses.MISSING:
                    v = f.default
                elif f.default_factory is not dataclasses.MISSING:  # type: ignore[misc]
                    v = f.default_factory()  # type: ignore[misc]
                else:
                    problems.append(f"missing required key '{key}'")
                    continue
            else:
                conv = f.metadata.get("convert")
                try:
                    v = conv(v) if conv is not None else v
                except (TypeError, ValueError) as e:
                    problems.append(f"key '{key}': {e}")
                    continue
            values[f.name] = v
        if problems:
            raise ConfigError(problems)
        cfg = cls(**values)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "ModelConfig":
        with open(path, "r", encoding="utf-8") as fh:
            raw = json.load(fh)
        if not isinstance(raw, dict):
            raise ConfigError(["config.json is not a JSON object"], where=path)
        return cls.from_dict(raw)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        for f in dataclasses.fields(self):
            v = getattr(self, f.name)
            if isinstance(v, tuple):
                v = list(v)
            out[f.metadata.get("key", f.name)] = v
        return out

    def validate(self) -> None:
        problems = self.problems()
        if problems:
            raise ConfigError(problems)

    def problems(self) -> List[str]:
        return []


# ---- converters used in field metadata ----------------------------------------

def as_int(v: Any) -> int:
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise TypeError(f"expected an integer, got {v!r}")
    if isinstance(v, float):
        if v != int(v):
            raise ValueError(f"expected an integer, got {v!r}")
        v = int(v)
    return v


def as_float(v: Any) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise TypeError(f"expected a number, got {v!r}")
    return float(v)


def as_opt_float(v: Any) -> Optional[float]:
    return None if v is None else as_float(v)


def as_bool(v: Any) -> bool:
    if not isinstance(v, bool):
        raise TypeError(f"expected true/false, got {v!r}")
    return v


def as_id_tuple(v: Any) -> Tuple[int, ...]:
    """``eos_token_id`` may be one id or a list of ids (LLM.pas:105-122)."""
    if v is None:
        return ()
    if isinstance(v, (list, tuple)):
        return tuple(as_int(x) for x in v)
    return (as_int(v),)


def as_str_tuple(v: Any) -> Tuple[str, ...]:
    if v is None:
        return ()
    if isinstance(v, str):
        return (v,)
    if isinstance(v, (list, tuple)) and all(isinstance(x, str) for x in v):
        return tuple(v)
    raise TypeError(f"expected a list of strings, got {v!r}")


# ---- registry -----------------------------------------------------------------

@dataclasses.dataclass(frozen=True)
class Architecture:
    """One entry of the registry: how to read the config and lay the model out."""

    name: str
    config_cls: Type[ModelConfig]
    # config -> quicknn_b200.parts.spec.ModelSpec
    build_spec: Callable[[ModelConfig], Any]
    aliases: Tuple[str, ...] = ()


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> Architecture:
    for n in (arch.name,) + tuple(arch.aliases):
        if n in _REGISTRY and not replace and _REGISTRY[n] is not arch:
            raise KeyError(f"architecture name '{n}' is already registered")
        _REGISTRY[n] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _REGISTRY.get(name)
    if arch is None:
        return
    for n in (arch.name,) + tuple(arch.aliases):
        if _REGISTRY.get(n) is arch:
            del _REGISTRY[n]


def registered_architectures() -> List[str]:
    return sorted(_REGISTRY)


def find_architecture(raw: Dict[str, Any]) -> Architecture:
    """Pick the architecture from ``architectures[0]`` and then ``model_type``."""
    tried: List[str] = []
    archs = raw.get("architectures")
    if isinstance(archs, (list, tuple)):
        for a in archs:
            if isinstance(a, str):
                tried.append(a)
                if a in _REGISTRY:
                    return _REGISTRY[a]
    mt = raw.get("model_type")
    if isinstance(mt, str):
        tried.append(mt)
        if mt in _REGISTRY:
            return _REGISTRY[mt]
    raise ConfigError(
        [f"no registered architecture for {tried or 'a config without architectures/model_type'}; "
         f"registered: {registered_architectures()}"])


def load_config(model_dir_or_file: str) -> Tuple[Architecture, ModelConfig]:
    path = model_dir_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path, "r", encoding="utf-8") as fh:
        raw = json.load(fh)
    if not isinstance(raw, dict):
        raise ConfigError(["config.json is not a JSON object"], where=path)
    arch = find_architecture(raw)
    return arch, arch.config_cls.from_dict(raw)
