"""What every architecture's configuration reader shares: the error type, typed access to a
key of config.json, token-id lists, and the reading of a model folder's config files
(crates/hi-mlx/src/config.rs:485-520, 809-823 for the end-of-sequence ids and their merge
with generation_config.json)."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model; the message names the key."""


def get_key(raw: Dict[str, Any], key: str, kind, default=None, required=False):
    if key not in raw or raw[key] is None:
        if required:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    value = raw[key]
    try:
        if kind is bool:
            if isinstance(value, (bool, int)):
                return bool(value)
            raise TypeError
        if kind is int:
            if isinstance(value, bool) or (isinstance(value, float) and value != int(value)):
                raise TypeError
            return int(value)
        if kind is float:
            if isinstance(value, bool):
                raise TypeError
            return float(value)
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: key '{key}' has value {value!r}, expected {kind.__name__}")
    return value


def token_ids(raw: Dict[str, Any], key: str) -> List[int]:
    value = raw.get(key)
    if isinstance(value, bool):
        return []
    if isinstance(value, int):
        return [value] if value >= 0 else []
    if isinstance(value, list):
        return [int(v) for v in value if isinstance(v, int) and not isinstance(v, bool) and v >= 0]
    return []


def read_config_files(model_dir: str):
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})")
    gen = None
    gpath = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gpath):
        try:
            with open(gpath, "r", encoding="utf-8") as f:
                gen = json.load(f)
        except json.JSONDecodeError:
            gen = None
    return raw, gen
