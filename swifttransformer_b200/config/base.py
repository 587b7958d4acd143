"""Typed model configurations read from a model folder's ``config.json``.

Every architecture declares one frozen dataclass whose fields are the keys of
its own ``config.json``.  A field without a default is required; a missing key
is an error that names the key.  No size lives anywhere else in the code: parts
receive their sizes from these objects.

The reference has no file-based configuration (sizes are constructor integers,
src/csrc/model/gpt/opt/optop.cc:9-36, or a name->table lookup,
src/examples/lib/common_gpt_hyper_params.h:10-68); the struct it fills is
src/csrc/model/gpt/gpt_hyper_param.h:8-28.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Callable, ClassVar, Dict, Type


class ConfigError(ValueError):
    """A config.json that cannot describe a model of its architecture."""


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of all typed configurations.

    Subclasses set ``ARCHITECTURE`` (the string in ``architectures[0]``) and
    may give ``KEY_ALIASES`` (config.json key -> field name) for keys whose
    spelling in the file differs from the field.
    """

    ARCHITECTURE: ClassVar[str] = ""
    KEY_ALIASES: ClassVar[Dict[str, str]] = {}

    def validate(self) -> None:  # pragma: no cover - overridden
        pass

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        fields = {f.name: f for f in dataclasses.fields(cls)}
        values: Dict[str, Any] = {}
        for key, val in raw.items():
            name = cls.KEY_ALIASES.get(key, key)
            if name in fields:
                values[name] = val
        missing = [
            n for n, f in fields.items()
            if n not in values
            and f.default is dataclasses.MISSING
            and f.default_factory is dataclasses.MISSING  # type: ignore[misc]
        ]
        if missing:
            raise ConfigError(
                f"config.json for {cls.ARCHITECTURE} lacks required key(s): {', '.join(missing)}")
        for name, val in list(values.items()):
            values[name] = _coerce(cls.ARCHITECTURE, name, fields[name].type, val)
        cfg = cls(**values)
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out = dataclasses.asdict(self)
        inverse = {v: k for k, v in self.KEY_ALIASES.items()}
        out = {inverse.get(k, k): v for k, v in out.items()}
        out["architectures"] = [self.ARCHITECTURE]
        return out


def _coerce(arch: str, name: str, typ: Any, val: Any) -> Any:
    tname = typ if isinstance(typ, str) else getattr(typ, "__name__", str(typ))
    if tname == "int":
        if isinstance(val, bool) or not isinstance(val, int):
            raise ConfigError(f"{arch}: key '{name}' must be an integer, got {val!r}")
        return val
    if tname == "float":
        if isinstance(val, bool) or not isinstance(val, (int, float)):
            raise ConfigError(f"{arch}: key '{name}' must be a number, got {val!r}")
        return float(val)
    if tname == "bool":
        if not isinstance(val, bool):
            raise ConfigError(f"{arch}: key '{name}' must be true or false, got {val!r}")
        return val
    if tname == "str":
        if not isinstance(val, str):
            raise ConfigError(f"{arch}: key '{name}' must be a string, got {val!r}")
        return val
    return val


_CONFIGS: Dict[str, Type[ModelConfig]] = {}


def register_config(cls: Type[ModelConfig]) -> Type[ModelConfig]:
    """Class decorator: make ``cls`` the configuration of ``cls.ARCHITECTURE``."""
    if not cls.ARCHITECTURE:
        raise ValueError("a configuration class must name its ARCHITECTURE")
    _CONFIGS[cls.ARCHITECTURE] = cls
    return cls


def known_architectures() -> list:
    return sorted(_CONFIGS)


def config_class(architecture: str) -> Type[ModelConfig]:
    try:
        return _CONFIGS[architecture]
    except KeyError:
        raise ConfigError(
            f"unknown architecture '{architecture}'; known: {', '.join(known_architectures()) or '(none)'}"
        ) from None


def config_from_dict(raw: Dict[str, Any]) -> ModelConfig:
    archs = raw.get("architectures")
    if not archs or not isinstance(archs, list):
        raise ConfigError("config.json lacks 'architectures' (a list with the model class name)")
    return config_class(archs[0]).from_dict(raw)


def load_config(model_dir: str) -> ModelConfig:
    """Read ``<model_dir>/config.json`` into the typed configuration of its architecture."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in '{model_dir}'")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(raw)


def save_config(cfg: ModelConfig, model_dir: str) -> None:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg.to_dict(), f, indent=2, sort_keys=True)
        f.write("\n")
