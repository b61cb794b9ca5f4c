"""Binds a checkpoint's tensors to a model's parts by name.

Every part names the tensors it reads (`tensor_specs`). The loader checks the
whole list against the checkpoint first and raises ONE `WeightError` that
lists every missing tensor, every unexpected tensor and every wrong shape;
the reference stops at the first missing name (mynah-slm src/model.c:129-135)
and checks shapes only in its tests (tests/test_model.c:116-127).

Kept types: matrices in the run's compute type (bfloat16, or float32 for the
32-bit path); gains that are stored in 32-bit stay 32-bit, others follow the
compute type; integer tables become int32. bf16 widens to fp32 exactly and
fp32 narrows to bf16 by round-to-nearest-even (what the reference's container
library does, third_party/ingot/src/dtype.c:270-284).
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..parts.base import Part, TensorSpec
from .safetensors_io import Checkpoint

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)


class WeightError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = ["the checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  {name}: shape {list(got)}, expected {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  {name}: dtype {got} cannot be used here")
        super().__init__("\n".join(lines))


def kept_dtype(role: str, stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if role == "table":
        return torch.int32
    if role == "gain" and stored == torch.float32:
        return torch.float32
    return run_dtype


def check(specs: list[tuple[Part, TensorSpec]], ckpt: Checkpoint) -> None:
    wanted: dict[str, TensorSpec] = {}
    for _, ts in specs:
        if ts.name in wanted and wanted[ts.name].shape != ts.shape:
            raise ValueError(f"two parts ask for {ts.name} with different shapes")
        if ts.name not in wanted or not ts.ignorable:
            wanted[ts.name] = ts
    have = ckpt.entries
    missing = [n for n, ts in wanted.items() if n not in have and not ts.ignorable]
    unexpected = [n for n in have if n not in wanted]
    wrong_shape, wrong_dtype = [], []
    for n, ts in wanted.items():
        if n in have and not ts.ignorable:
            e = have[n]
            if tuple(e.shape) != tuple(ts.shape):
                wrong_shape.append((n, e.shape, ts.shape))
            is_float = e.dtype in ("F32", "BF16", "F16", "F64")
            if (ts.role == "table") == is_float:
                wrong_dtype.append((n, e.dtype))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype)


def load_into(parts_and_specs: list[tuple[Part, TensorSpec]], ckpt: Checkpoint, runtime) -> None:
    """Check, move each tensor to the device in its kept type, and bind."""
    check(parts_and_specs, ckpt)
    on_device: dict[str, torch.Tensor] = {}
    by_part: dict[int, tuple[Part, dict[str, torch.Tensor]]] = {}
    for part, ts in parts_and_specs:
        entry = by_part.setdefault(id(part), (part, {}))
        if ts.ignorable:
            continue
        if ts.name not in on_device:
            src = ckpt.tensor(ts.name)
            on_device[ts.name] = src.to(device=runtime.device, dtype=kept_dtype(ts.role, src.dtype, runtime.act_dtype))
        entry[1][ts.name] = on_device[ts.name]
    for part, tensors in by_part.values():
        part.bind(tensors, runtime)
