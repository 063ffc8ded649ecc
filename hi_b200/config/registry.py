"""One registry from an architecture's name to its model.

An :class:`Architecture` knows how to read its config.json (a typed configuration), how to
turn that into a :class:`~hi_b200.parts.spec.ModelSpec`, and how checkpoint tensor names map
to the names its parts ask for. Lookup is by ``architectures[0]`` first, then ``model_type``
(the reference routes by substring of model_type: crates/hi-mlx/src/config.rs:535-643,
crates/hi-mlx/src/models.rs:373-375).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

from .base import ConfigError, read_config_files


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any], Optional[Dict[str, Any]]], Any]
    build_spec: Callable[[Any], Any]                       # typed config -> ModelSpec
    normalize_tensor_name: Callable[[str], Optional[str]]  # checkpoint name -> part name, None = not ours
    # other layouts of the same weights: {normalised name: shape} of the checkpoint -> {part name:
    # DerivedTensor} for tensors that have to be made from others (split, transposed); optional
    derive_tensors: Optional[Callable[[Dict[str, tuple]], Dict[str, Any]]] = None


_BY_NAME: Dict[str, Architecture] = {}


def register_architecture(names: List[str], arch: Architecture) -> None:
    for n in names:
        _BY_NAME[n] = arch


def registered_architectures() -> List[str]:
    _load_builtin()
    return sorted(_BY_NAME)


_builtin_loaded = False


def _load_builtin() -> None:
    """The architectures this package brings register themselves when their module is imported."""
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        import importlib

        importlib.import_module("hi_b200.architectures")


def lookup(raw_config: Dict[str, Any]) -> Architecture:
    _load_builtin()
    archs = raw_config.get("architectures") or []
    if isinstance(archs, str):
        archs = [archs]
    for name in list(archs) + [raw_config.get("model_type")]:
        if isinstance(name, str) and name in _BY_NAME:
            return _BY_NAME[name]
    raise ConfigError(
        f"config.json: no model is registered for architectures {list(archs)!r} / model_type "
        f"{raw_config.get('model_type')!r}; registered: {registered_architectures()}")


def load_architecture(model_dir: str):
    """(architecture, typed config, raw config) of a model folder."""
    raw, gen = read_config_files(model_dir)
    arch = lookup(raw)
    return arch, arch.parse_config(raw, gen), raw
