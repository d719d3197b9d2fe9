"""Dataclass-backed configuration: YAML file + ``a.b=c`` command-line overrides.

Same behaviour as the OmegaConf-based helpers in lingua/args.py (dataclass_from_dict :38,
dataclass_to_dict :48, load_config_file :60, dump_config :65, flatten_dict :27) and the
``structured(Args()) <- yaml <- cli`` merge of apps/main/train.py:644-651, implemented on
plain dicts so that it has no dependency beyond PyYAML:

* unknown keys are errors in strict mode (the "struct" flag),
* values are coerced to the annotated field type (``3e-4`` given as a string becomes a
  float, ints are accepted for floats, nested dataclasses / Optional / List / Dict / Any
  are handled recursively),
* the resolved config round-trips through ``dump_config`` / ``load_config_file``.
"""
from __future__ import annotations

import dataclasses
import logging
import re
import typing
from enum import Enum
from typing import Any, Dict, List, Optional, Type, TypeVar, Union, get_args, get_origin

import yaml

logger = logging.getLogger()
T = TypeVar("T")

_FLOAT_RE = re.compile(r"^[-+]?(\d[\d_]*)?(\.\d*)?([eE][-+]?\d+)?$")


class ConfigError(ValueError):
    pass


# ----------------------------------------------------------------------------- parsing
def parse_scalar(text: str) -> Any:
    """Parse one command-line value with YAML rules, plus floats such as ``3e-4``."""
    try:
        v = yaml.safe_load(text)
    except yaml.YAMLError:
        return text
    if isinstance(v, str):
        s = v.strip()
        if s and _FLOAT_RE.match(s) and any(c.isdigit() for c in s):
            try:
                return float(s.replace("_", ""))
            except ValueError:
                return v
    return v


def from_cli(argv: Optional[List[str]] = None) -> Dict[str, Any]:
    """``["a.b=1", "c=[x,y]"]`` -> ``{"a": {"b": 1}, "c": ["x", "y"]}``."""
    import sys

    argv = sys.argv[1:] if argv is None else argv
    out: Dict[str, Any] = {}
    for item in argv:
        if "=" not in item:
            raise ConfigError(f"expected key=value, got {item!r}")
        key, val = item.split("=", 1)
        node = out
        parts = key.strip().split(".")
        for p in parts[:-1]:
            nxt = node.setdefault(p, {})
            if not isinstance(nxt, dict):
                raise ConfigError(f"{key}: {p} is already a leaf")
            node = nxt
        node[parts[-1]] = parse_scalar(val)
    return out


def load_yaml(path: str) -> Dict[str, Any]:
    with open(path) as f:
        data = yaml.safe_load(f)
    return data or {}


def merge_dicts(base: Dict[str, Any], override: Dict[str, Any]) -> Dict[str, Any]:
    """Recursive merge; values of ``override`` win, dicts merge key by key."""
    out = dict(base)
    for k, v in override.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = merge_dicts(out[k], v)
        else:
            out[k] = v
    return out


# ----------------------------------------------------------------------------- typing
def _is_dataclass_type(t) -> bool:
    return isinstance(t, type) and dataclasses.is_dataclass(t)


def _coerce(value: Any, tp: Any, path: str, strict: bool) -> Any:
    if tp is Any or tp is typing.Any or tp is None:
        return value
    origin = get_origin(tp)
    if origin is Union:
        args = get_args(tp)
        if value is None:
            if type(None) in args:
                return None
            raise ConfigError(f"{path}: None is not allowed")
        errors = []
        for a in args:
            if a is type(None):
                continue
            try:
                return _coerce(value, a, path, strict)
            except (ConfigError, TypeError, ValueError) as e:  # try the next alternative
                errors.append(str(e))
        raise ConfigError(f"{path}: {value!r} matches no alternative of {tp}: {errors}")
    if origin in (list, List):
        (et,) = get_args(tp) or (Any,)
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{path}: expected a list, got {value!r}")
        return [_coerce(v, et, f"{path}[{i}]", strict) for i, v in enumerate(value)]
    if origin in (dict, Dict):
        kt, vt = get_args(tp) or (Any, Any)
        if not isinstance(value, dict):
            raise ConfigError(f"{path}: expected a mapping, got {value!r}")
        return {k: _coerce(v, vt, f"{path}.{k}", strict) for k, v in value.items()}
    if origin is tuple:
        return tuple(value)
    if _is_dataclass_type(tp):
        if dataclasses.is_dataclass(value) and not isinstance(value, type):
            return value
        if value is None:
            raise ConfigError(f"{path}: None given for {tp.__name__}")
        if not isinstance(value, dict):
            raise ConfigError(f"{path}: expected a mapping for {tp.__name__}, got {value!r}")
        return _build(tp, value, path, strict)
    if isinstance(tp, type) and issubclass(tp, Enum):
        if isinstance(value, tp):
            return value
        try:
            return tp(value)
        except ValueError:
            try:
                return tp[str(value)]
            except KeyError:
                raise ConfigError(f"{path}: {value!r} is not a {tp.__name__}")
    if tp is bool:
        if isinstance(value, bool):
            return value
        if isinstance(value, str) and value.lower() in ("true", "false"):
            return value.lower() == "true"
        raise ConfigError(f"{path}: expected bool, got {value!r}")
    if tp is int:
        if isinstance(value, bool):
            raise ConfigError(f"{path}: expected int, got bool")
        if isinstance(value, int):
            return value
        if isinstance(value, float) and value.is_integer():
            return int(value)
        if isinstance(value, str):
            try:
                return int(value.replace("_", ""))
            except ValueError:
                pass
        raise ConfigError(f"{path}: expected int, got {value!r}")
    if tp is float:
        if isinstance(value, bool):
            raise ConfigError(f"{path}: expected float, got bool")
        if isinstance(value, (int, float)):
            return float(value)
        if isinstance(value, str):
            try:
                return float(value.replace("_", ""))
            except ValueError:
                pass
        raise ConfigError(f"{path}: expected float, got {value!r}")
    if tp is str:
        if isinstance(value, (dict, list)):
            raise ConfigError(f"{path}: expected str, got {value!r}")
        return value if isinstance(value, str) else str(value)
    return value


def _build(cls: Type[T], data: Dict[str, Any], path: str, strict: bool) -> T:
    hints = typing.get_type_hints(cls)
    fields = {f.name: f for f in dataclasses.fields(cls)}
    unknown = [k for k in data if k not in fields]
    if unknown and strict:
        raise ConfigError(
            f"{path or cls.__name__}: unknown key(s) {unknown}; valid keys: {sorted(fields)}"
        )
    obj = cls()
    for name, f in fields.items():
        if name not in data:
            continue
        sub = f"{path}.{name}" if path else name
        tp = hints.get(name, Any)
        value = data[name]
        cur = getattr(obj, name, None)
        # a mapping merged into a dataclass default keeps the default's other fields
        if isinstance(value, dict) and dataclasses.is_dataclass(cur) and not isinstance(cur, type):
            value = merge_dicts(dataclass_to_dict(cur), value)
            setattr(obj, name, _coerce(value, type(cur), sub, strict))
        else:
            setattr(obj, name, _coerce(value, tp, sub, strict))
    return obj


# ----------------------------------------------------------------------------- public
def dataclass_from_dict(cls: Type[T], data: Dict[str, Any], strict: bool = True) -> T:
    """Instantiate ``cls`` with its defaults overridden by ``data`` (recursively)."""
    return _build(cls, dict(data or {}), "", strict)


def dataclass_to_dict(obj: Any) -> Any:
    """Nested plain-container copy of a dataclass instance (enums become their value)."""
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: dataclass_to_dict(getattr(obj, f.name)) for f in dataclasses.fields(obj)}
    if isinstance(obj, dict):
        return {k: dataclass_to_dict(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [dataclass_to_dict(v) for v in obj]
    if isinstance(obj, Enum):
        return obj.value
    return obj


def flatten_dict(d: Dict[str, Any], parent_key: str = "", sep: str = "_") -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    for k, v in d.items():
        key = f"{parent_key}{sep}{k}" if parent_key else str(k)
        if isinstance(v, dict):
            out.update(flatten_dict(v, key, sep))
        else:
            out[key] = v
    return out


def to_yaml(obj: Any) -> str:
    return yaml.safe_dump(dataclass_to_dict(obj), sort_keys=False, default_flow_style=False)


def load_config_file(path: str, cls: Type[T]) -> T:
    return dataclass_from_dict(cls, load_yaml(path))


def dump_config(config: Any, path: str, log_config: bool = True) -> None:
    text = to_yaml(config)
    if log_config:
        logger.info("Using the following config for this run:")
        logger.info(text)
    with open(path, "w") as f:
        f.write(text)


def config_from_cli(cls: Type[T], argv: Optional[List[str]] = None, strict: bool = True) -> T:
    """``defaults <- yaml named by config=... <- remaining key=value overrides``."""
    cli = from_cli(argv)
    file_cfg: Dict[str, Any] = {}
    path = cli.pop("config", None)
    if path is not None:
        file_cfg = load_yaml(path)
    return dataclass_from_dict(cls, merge_dicts(file_cfg, cli), strict=strict)
