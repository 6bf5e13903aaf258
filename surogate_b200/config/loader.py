"""Load a YAML config (local path or http(s) URL), expand ``${ENV}`` references, build a config object.

Parity: surogate/core/config/loader.py:24-76.
"""
from __future__ import annotations

import os
import re
from typing import Any, Dict, Type, TypeVar

import yaml

T = TypeVar("T")
_ENV = re.compile(r"\$\{([A-Za-z_][A-Za-z0-9_]*)(?::-([^}]*))?\}")


class DictDefault(dict):
    """dict whose missing keys read as None and whose keys are also attributes."""

    def __getattr__(self, k):
        v = self.get(k)
        return DictDefault(v) if isinstance(v, dict) and not isinstance(v, DictDefault) else v

    def __setattr__(self, k, v):
        self[k] = v

    def __missing__(self, k):
        return None


def expand_env(obj: Any) -> Any:
    """Recursively replace ``${VAR}`` / ``${VAR:-default}`` in strings; an unset VAR without default is an error."""
    if isinstance(obj, str):
        def sub(m):
            val = os.environ.get(m.group(1), m.group(2))
            if val is None:
                raise KeyError(f"config references ${{{m.group(1)}}} but it is not set")
            return val
        return _ENV.sub(sub, obj)
    if isinstance(obj, dict):
        return {k: expand_env(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [expand_env(v) for v in obj]
    return obj


def coerce_fields(cls, kw: Dict[str, Any]) -> Dict[str, Any]:
    """Convert string values to the scalar type a dataclass field declares.  YAML 1.1 reads ``3e-4`` (no decimal point) as a
    string, and every ``${ENV}`` expansion yields one; without this they would reach arithmetic as text.  A value that does not
    parse raises an error naming the key."""
    import dataclasses
    import typing

    hints = typing.get_type_hints(cls)
    out = dict(kw)
    for f in dataclasses.fields(cls):
        v = out.get(f.name)
        if not isinstance(v, (str, int)) or isinstance(v, bool):
            continue
        t = hints.get(f.name)
        args = [a for a in typing.get_args(t) if a is not type(None)] if typing.get_origin(t) is typing.Union else [t]
        if str in args and isinstance(v, str):
            continue
        try:
            if isinstance(v, str):
                if bool in args and v.strip().lower() in ("true", "false", "yes", "no", "on", "off", "1", "0"):
                    out[f.name] = v.strip().lower() in ("true", "yes", "on", "1")
                elif int in args and re.fullmatch(r"[+-]?\d+", v.strip()):
                    out[f.name] = int(v)
                elif float in args:
                    out[f.name] = float(v)
                elif int in args:
                    fv = float(v)
                    if fv != int(fv):
                        raise ValueError(v)
                    out[f.name] = int(fv)
            elif float in args and int not in args:
                out[f.name] = float(v)
        except ValueError:
            raise ValueError(f"[E100] config key '{f.name}': cannot read '{v}' as {getattr(t, '__name__', t)}") from None
    return out


def read_yaml(path: str) -> Dict[str, Any]:
    if path.startswith(("http://", "https://")):
        import requests

        r = requests.get(path, timeout=30)
        r.raise_for_status()
        text = r.text
    else:
        with open(path) as f:
            text = f.read()
    data = yaml.safe_load(text) or {}
    if not isinstance(data, dict):
        raise ValueError(f"{path}: top level of a config must be a mapping")
    return expand_env(data)


def load_config(cls: Type[T], path_or_dict, **overrides) -> T:
    data = dict(path_or_dict) if isinstance(path_or_dict, dict) else read_yaml(path_or_dict)
    data.update({k: v for k, v in overrides.items() if v is not None})
    return cls.from_dict(DictDefault(data))
