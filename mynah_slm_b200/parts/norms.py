"""RMSNorm with a plain gain.

out = x * (1 / sqrt(mean(x^2) + eps)) * w, the reference's form (mynah-slm
src/kernels.c:118-128); the gain multiplies as it is, it is not 1 + w
(src/kernels.h:29-33: a (1+w) norm is a different function, not a flag of
this one). Parameters: eps, dim, and the gain's tensor name.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..ops import kernels
from .base import Norm, Residual, TensorSpec, register_norm


class RMSNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.eps = float(spec["eps"])
        self.dim = int(spec["dim"])
        self.name = str(spec["name"])
        self.gain: Optional[torch.Tensor] = None
        self.act_dtype = torch.float32

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.dim,), role="gain", init="gain", std=0.1)]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.gain = tensors[self.name]
        self.act_dtype = runtime.act_dtype

    def apply(self, stream: Residual, rows: Optional[torch.Tensor] = None, lazy: bool = False):
        delta, stream.pending = stream.pending, None
        if lazy and rows is None:
            return kernels.NormedInput(stream, delta, self.gain, self.eps, self.act_dtype)
        return kernels.rmsnorm(stream.x, self.gain, self.eps, self.act_dtype, delta=delta, rows=rows)


register_norm("rmsnorm", RMSNorm)
