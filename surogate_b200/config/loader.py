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
