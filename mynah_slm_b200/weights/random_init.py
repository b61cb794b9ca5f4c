"""Random-weights mode: a model from a typed configuration and a seed, with no
checkpoint.

The reference has no such mode: its tests need a real checkpoint and its CI
says so (mynah-slm .github/workflows/build.yml:10-13). Matrices and the
embedding are N(0, 0.02), norm gains 1 + N(0, 0.1) (each part states its own
in its `TensorSpec`).

Every element is a function of (seed, tensor name, element index): a
counter-based generator (splitmix64's output function, Box-Muller in exactly
rounded double arithmetic; `include/mynah_random_normal.h`). So a tensor does
not depend on the order of writing, on the other tensors or on where it is
made. Two makers evaluate the one function: the native host runtime, for
writing a model folder (config.json, model.safetensors) where there is no
device, and a kernel, which fills an engine's weights in place
(`Engine.random`): a model of the 8-billion-parameter shape then starts
without a 16 GB file. Both give the same bits, and so does a folder that was
written and read back.
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch

from ..engine.model import Model
from ..parts.base import TensorSpec
from .safetensors_io import write_safetensors

MASK64 = (1 << 64) - 1


def tensor_key(name: str) -> int:
    """FNV-1a (64-bit) of the tensor's name: what tells one tensor's numbers from another's."""
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & MASK64
    return h


def _mean_std(ts: TensorSpec) -> tuple[float, float]:
    if ts.init == "zeros":
        return 0.0, 0.0
    if ts.init == "gain":
        return 1.0, float(ts.std)
    if ts.init == "normal":
        return 0.0, float(ts.std)
    raise ValueError(f"{ts.name}: unknown init {ts.init!r}")


def _wanted(model: Model) -> list[TensorSpec]:
    seen, out = set(), []
    for _, ts in model.tensor_specs():
        if ts.ignorable or ts.name in seen:
            continue
        seen.add(ts.name)
        out.append(ts)
    return out


def host_tensor(ts: TensorSpec, seed: int, dtype: torch.dtype) -> torch.Tensor:
    """One tensor of the random model, made by the native host runtime."""
    from ..cache.pages import host_library
    if ts.role == "table":
        return torch.zeros(ts.shape, dtype=torch.int32)
    if dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"random weights are written as float32 or bfloat16, not {dtype}")
    n = int(np.prod(ts.shape)) if len(ts.shape) else 1
    mean, std = _mean_std(ts)
    buf = np.empty((n,), dtype=np.float32 if dtype == torch.float32 else np.uint16)
    lib = host_library()
    rc = lib.mynah_randn_fill_host(buf.ctypes.data, 0 if dtype == torch.float32 else 1, n, int(seed) & MASK64,
                                   tensor_key(ts.name), mean, std)
    if rc != 0:
        raise ValueError(lib.mynah_host_last_error().decode(errors="replace"))
    t = torch.from_numpy(buf)
    if dtype == torch.bfloat16:
        t = t.view(torch.int16).view(torch.bfloat16)
    return t.reshape(ts.shape)


def random_tensors(typed_config, seed: int, dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    model = Model(typed_config.model_spec())
    return {ts.name: host_tensor(ts, seed, dtype) for ts in _wanted(model)}


def write_random_model(folder: str, typed_config, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    os.makedirs(folder, exist_ok=True)
    cfg = typed_config.to_dict()
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[dtype]
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_tensors(typed_config, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder


def device_tensor(ts: TensorSpec, seed: int, dtype: torch.dtype, device) -> torch.Tensor:
    """One tensor of the random model, made on the device by `mynah_randn_fill`."""
    from ..ops.lib import call, code, ptr, stream_ptr
    if ts.role == "table":
        return torch.zeros(ts.shape, dtype=torch.int32, device=device)
    t = torch.empty(ts.shape, dtype=dtype, device=device)
    mean, std = _mean_std(ts)
    call("mynah_randn_fill", ptr(t), code(dtype), t.numel(), int(seed) & MASK64, tensor_key(ts.name), mean, std, stream_ptr())
    return t


class RandomWeights:
    """Stands where a checkpoint stands when an engine is built: the weights are made on the device from
    `seed`, as a folder written by `write_random_model(..., seed, stored_dtype)` would hold them."""

    def __init__(self, seed: int, stored_dtype: torch.dtype = torch.bfloat16):
        self.seed, self.stored_dtype = int(seed), stored_dtype

    def close(self) -> None:
        pass


def fill_into(parts_and_specs, source: RandomWeights, runtime) -> None:
    """What `loader.load_into` does for a checkpoint: each tensor once, in its kept type, bound to its parts."""
    from .loader import kept_dtype
    made: dict[str, torch.Tensor] = {}
    by_part: dict[int, tuple] = {}
    for part, ts in parts_and_specs:
        entry = by_part.setdefault(id(part), (part, {}))
        if ts.ignorable:
            continue
        if ts.name not in made:
            t = device_tensor(ts, source.seed, source.stored_dtype, runtime.device)
            made[ts.name] = t.to(kept_dtype(ts.role, t.dtype, runtime.act_dtype))
        entry[1][ts.name] = made[ts.name]
    for part, tensors in by_part.values():
        part.bind(tensors, runtime)
