"""Bind checkpoint tensors to a model's parts by name, or fill them from a seeded generator.

Floating tensors stored as BF16 stay bfloat16 (F16 is converted to bfloat16); a tensor
stored in 32-bit stays 32-bit; integer tables become int32. In the float32 path every
floating tensor is widened to float32. One error lists every missing tensor, every
unexpected tensor and every wrong shape (the reference stops at the first missing name:
crates/hi-mlx/src/models.rs:10723, crates/hi-mlx/src/weights.rs:94-103).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, List, Optional

import torch

from . import random_values
from .safetensors_io import Checkpoint, SafetensorsError, write_safetensors


class WeightError(ValueError):
    """The checkpoint does not fit the model; ``missing``, ``unexpected`` and ``wrong_shape`` say how."""

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)


def check_names(specs, available: Dict[str, tuple], where: str) -> None:
    """Compare what the parts ask for with what the checkpoint holds ({name: shape})."""
    expected = {s.name: s for s in specs}
    missing = sorted(n for n, s in expected.items() if n not in available and not s.optional)
    unexpected = sorted(n for n in available if n not in expected)
    wrong = sorted((n, tuple(available[n]), tuple(s.shape)) for n, s in expected.items()
                   if n in available and tuple(available[n]) != tuple(s.shape))
    if missing or unexpected or wrong:
        lines = [f"{where}: the checkpoint does not fit the model"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " +
                         ", ".join(f"{n} is {list(a)}, expected {list(e)}" for n, a, e in wrong))
        raise WeightError("\n".join(lines), missing, unexpected, wrong)


class DerivedTensor:
    """A tensor the parts ask for that the checkpoint holds in another layout: ``make`` builds it
    (on the device) from the tensors named ``sources``, which count as used."""

    def __init__(self, sources, shape, make):
        self.sources, self.shape, self.make = list(sources), tuple(shape), make


def _to_engine(t: torch.Tensor, engine_dtype: torch.dtype, device) -> torch.Tensor:
    if t.dtype in (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8, torch.bool):
        return t.to(device=device, dtype=torch.int32)
    if engine_dtype == torch.float32:
        return t.to(device=device).to(torch.float32)
    if t.dtype == torch.float16:
        return t.to(device=device).to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(device=device).to(torch.float32)
    return t.to(device=device)        # BF16 stays bfloat16, F32 stays float32


def load_from_dir(model, model_dir: str, normalize: Callable[[str], Optional[str]], derive=None) -> None:
    """Fill ``model`` (a :class:`hi_b200.parts.model.Model`) from the safetensors of ``model_dir``.
    ``derive({name: shape}) -> {name: DerivedTensor}``: tensors to be made from others the
    checkpoint stores in another layout."""
    try:
        ckpt = Checkpoint(model_dir)
    except SafetensorsError as e:
        raise WeightError(str(e)) from e
    by_part_name: Dict[str, str] = {}
    clashes = []
    for original in ckpt.names():
        name = normalize(original)
        if name is None:
            continue
        if name in by_part_name:
            clashes.append(name)
        by_part_name[name] = original
    if clashes:
        raise WeightError(f"{model_dir}: tensors that map to the same name: {sorted(set(clashes))}")
    shapes = {name: ckpt.describe(orig)[1] for name, orig in by_part_name.items()}
    bad_dtype = sorted(f"{n} ({ckpt.describe(o)[0]})" for n, o in by_part_name.items()
                       if ckpt.describe(o)[0] not in ("F32", "BF16", "F16", "F64", "I32", "I64", "I16", "I8", "U8"))
    if bad_dtype:
        raise WeightError(f"{model_dir}: quantized or packed tensors are not supported: " + ", ".join(bad_dtype))
    derived: Dict[str, DerivedTensor] = derive(dict(shapes)) if derive is not None else {}
    for name, d in derived.items():
        shapes[name] = d.shape
        for src in d.sources:
            shapes.pop(src, None)
    check_names(model.tensor_specs(), shapes, model_dir)

    def fetch(name: str):
        if name in derived:
            d = derived[name]
            return d.make([_to_engine(ckpt.tensor(by_part_name[src]), model.dtype, model.device) for src in d.sources])
        original = by_part_name.get(name)
        if original is None:
            return None
        return _to_engine(ckpt.tensor(original), model.dtype, model.device)

    model.load(fetch)


# --------------------------------------------------------------------------- random weights
def random_tensor(spec, seed: int, std: float, device="cpu", dtype=torch.bfloat16) -> torch.Tensor:
    """The seeded value of one tensor: N(0, std) or ones/zeros, keyed by (seed, name, element
    index). The numbers come from a counter-based generator in integer arithmetic
    (:mod:`hi_b200.weights.random_values`), so a tensor made on the host and the same tensor made
    on the device by ``hb_random_normal`` hold the same bits."""
    if spec.dtype == "int32":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "ones":
        return torch.ones(spec.shape, dtype=dtype, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    key = random_values.tensor_key(seed, spec.name)
    if torch.device(device).type == "cuda":
        from ..kernels import ops

        out = torch.empty(spec.shape, dtype=dtype, device=device)
        ops.random_normal(out, key, float(random_values.scale_for(std)))
        return out
    n = 1
    for d in spec.shape:
        n *= int(d)
    values = torch.from_numpy(random_values.normal_values(key, 0, n, std))
    return values.view(tuple(spec.shape)).to(dtype)


def load_random(model, seed: int, std: float = 0.02) -> None:
    """Fill ``model`` on its device from the seeded generator (no files): used for large models."""
    specs = {s.name: s for s in model.tensor_specs()}

    def fetch(name: str):
        spec = specs[name]
        if spec.init == "absent":
            return None
        store = torch.bfloat16 if model.dtype == torch.bfloat16 else torch.float32
        t = random_tensor(spec, seed, std, device=model.device, dtype=torch.bfloat16)
        return t.to(store) if t.dtype.is_floating_point else t

    model.load(fetch)


def write_random_model(config: dict, out_dir: str, seed: int, std: float = 0.02,
                       overrides: Optional[Dict[str, torch.Tensor]] = None) -> str:
    """Write a model folder (config.json, model.safetensors) for ``config`` with seeded random
    weights: N(0, std) matrices, norm weights 1, all stored as BF16. ``overrides`` replaces
    named tensors (tests use it to make one key or one expert stand out)."""
    from ..config.registry import lookup
    from ..parts.model import Model

    arch = lookup(config)
    typed = arch.parse_config(config, None)
    model = Model(arch.build_spec(typed), torch.bfloat16, "cpu")
    tensors = {}
    for spec in model.tensor_specs():
        if spec.init == "absent":
            continue
        tensors[spec.name] = random_tensor(spec, seed, std)
    for name, value in (overrides or {}).items():
        if name not in tensors:
            raise WeightError(f"override for unknown tensor '{name}'")
        if tuple(value.shape) != tuple(tensors[name].shape):
            raise WeightError(f"override for '{name}' has shape {list(value.shape)}, expected {list(tensors[name].shape)}")
        tensors[name] = value.to(tensors[name].dtype)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed), "std": str(std)})
    return out_dir
