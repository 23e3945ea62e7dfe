"""One loader for every component's configuration dataclass: dict / JSON / YAML file, then environment
overrides, then the class's own ``validate()``.

The reference has no central flag system: each component carries a config class with defaults, a
``Validate()`` method and sometimes a builder or presets (src/MLFramework/Distributed/FSDP/FSDPConfig.cs:23-58,
src/MLFramework/Pipeline/PipelineConfig.cs:10-79), and only the visualizer reads a JSON file with environment
overrides (src/MLFramework.Visualization/Configuration/ConfigurationLoader.cs:26-231). Here the same per-component
dataclasses (``FSDPConfig``, ``PipelineConfig``, ``ExecutorConfig``, ``EngineConfig``, ...) all load through
``load_config``; an environment variable ``<PREFIX>_<FIELD>`` (upper case) overrides field ``field``.
"""
from __future__ import annotations

import dataclasses
import enum
import json
import os
import typing
from pathlib import Path
from typing import Any, Mapping, Optional, Type, TypeVar, Union

T = TypeVar("T")


def _coerce(value: Any, ftype: Any) -> Any:
    """Turn a JSON / YAML / environment value into the field's declared type."""
    origin = typing.get_origin(ftype)
    if origin is Union:                                   # Optional[X] and unions: first member that accepts the value
        args = [a for a in typing.get_args(ftype) if a is not type(None)]
        if value is None or (isinstance(value, str) and value.lower() in ("none", "null", "")):
            return None
        for a in args:
            try:
                return _coerce(value, a)
            except (TypeError, ValueError):
                continue
        return value
    if isinstance(ftype, type) and issubclass(ftype, enum.Enum):
        if isinstance(value, ftype):
            return value
        try:
            return ftype[str(value).upper()] if isinstance(value, str) and str(value).upper() in ftype.__members__ else ftype(value)
        except ValueError:
            return ftype(type(next(iter(ftype)).value)(value))
    if dataclasses.is_dataclass(ftype) and isinstance(value, Mapping):
        return from_dict(ftype, value)
    if ftype is bool:
        if isinstance(value, str):
            if value.lower() in ("1", "true", "yes", "on"):
                return True
            if value.lower() in ("0", "false", "no", "off"):
                return False
            raise ValueError(f"not a boolean: {value!r}")
        return bool(value)
    if ftype in (int, float, str):
        return ftype(value)
    if origin in (list, tuple) and isinstance(value, str):
        inner = (typing.get_args(ftype) or (str,))[0]
        items = [_coerce(v.strip(), inner) for v in value.split(",") if v.strip()]
        return tuple(items) if origin is tuple else items
    if origin in (list, tuple) and isinstance(value, (list, tuple)):
        inner = (typing.get_args(ftype) or (Any,))[0]
        items = [_coerce(v, inner) if inner is not Any else v for v in value]
        return tuple(items) if origin is tuple else items
    return value


def from_dict(cls: Type[T], data: Mapping[str, Any], strict: bool = True) -> T:
    """Build dataclass ``cls`` from a mapping; unknown keys raise unless ``strict`` is False."""
    if not dataclasses.is_dataclass(cls):
        raise TypeError(f"{cls!r} is not a dataclass")
    hints = typing.get_type_hints(cls)
    names = {f.name for f in dataclasses.fields(cls) if f.init}
    unknown = set(data) - names
    if unknown and strict:
        raise KeyError(f"unknown {cls.__name__} field(s): {sorted(unknown)}")
    kwargs = {k: _coerce(v, hints.get(k, Any)) for k, v in data.items() if k in names}
    return cls(**kwargs)


def to_dict(cfg: Any) -> dict:
    """Plain-JSON view of a config dataclass (enums by value)."""
    def enc(v):
        if isinstance(v, enum.Enum):
            return v.value
        if dataclasses.is_dataclass(v):
            return {f.name: enc(getattr(v, f.name)) for f in dataclasses.fields(v)}
        if isinstance(v, (list, tuple)):
            return [enc(x) for x in v]
        if isinstance(v, dict):
            return {k: enc(x) for k, x in v.items()}
        return v
    return enc(cfg)


def read_file(path: Union[str, Path]) -> dict:
    p = Path(path)
    text = p.read_text()
    if p.suffix.lower() in (".yaml", ".yml"):
        import yaml
        return yaml.safe_load(text) or {}
    return json.loads(text)


def apply_env(cls: Type[T], data: dict, prefix: str, environ: Optional[Mapping[str, str]] = None) -> dict:
    """``<PREFIX>_<FIELD>`` overrides ``field``; the value is parsed by the field's type."""
    env = os.environ if environ is None else environ
    out = dict(data)
    for f in dataclasses.fields(cls):
        key = f"{prefix}_{f.name}".upper()
        if key in env:
            out[f.name] = env[key]
    return out


def load_config(cls: Type[T], source: Union[None, str, Path, Mapping[str, Any]] = None, env_prefix: Optional[str] = None,
                environ: Optional[Mapping[str, str]] = None, strict: bool = True) -> T:
    """Defaults < file or mapping < environment; then ``validate()`` if the class has one."""
    data: dict = {}
    if isinstance(source, Mapping):
        data = dict(source)
    elif source is not None:
        data = read_file(source)
    if env_prefix:
        data = apply_env(cls, data, env_prefix, environ)
    cfg = from_dict(cls, data, strict)
    v = getattr(cfg, "validate", None)
    if callable(v):
        v()
    return cfg


def save_config(cfg: Any, path: Union[str, Path]) -> None:
    p = Path(path)
    d = to_dict(cfg)
    if p.suffix.lower() in (".yaml", ".yml"):
        import yaml
        p.write_text(yaml.safe_dump(d, sort_keys=False))
    else:
        p.write_text(json.dumps(d, indent=1))
