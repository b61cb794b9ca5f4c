"""Random-weights mode: writes a model folder (config.json, model.safetensors)
from a typed configuration and a seed.

The reference has no such mode: its tests need a real checkpoint and its CI
says so (mynah-slm .github/workflows/build.yml:10-13). Matrices and the
embedding are N(0, 0.02), norm gains 1 + N(0, 0.1) (each part states its own
in its `TensorSpec`). Tensor i of the model's list is drawn from a generator
seeded with (seed, i), on the CPU, so a folder is reproducible anywhere and
does not depend on the order of writing.
"""
from __future__ import annotations

import json
import os

import torch

from ..engine.model import Model
from .safetensors_io import write_safetensors


def random_tensors(typed_config, seed: int, dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    model = Model(typed_config.model_spec())
    out: dict[str, torch.Tensor] = {}
    idx = 0
    for _, ts in model.tensor_specs():
        if ts.ignorable or ts.name in out:
            continue
        gen = torch.Generator(device="cpu")
        gen.manual_seed((int(seed) * 1_000_003 + idx) & 0x7FFFFFFFFFFFFFFF)
        idx += 1
        if ts.role == "table":
            out[ts.name] = torch.zeros(ts.shape, dtype=torch.int32)
            continue
        if ts.init == "zeros":
            t = torch.zeros(ts.shape, dtype=torch.float32)
        else:
            t = torch.randn(ts.shape, generator=gen, dtype=torch.float32) * ts.std
            if ts.init == "gain":
                t += 1.0
        out[ts.name] = t.to(dtype)
    return out


def write_random_model(folder: str, typed_config, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    os.makedirs(folder, exist_ok=True)
    cfg = typed_config.to_dict()
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_tensors(typed_config, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
