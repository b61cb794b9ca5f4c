"""Dense gated feed-forward (SwiGLU).

x -> W_down . (silu(W_gate . x) * (W_up . x)), no bias (mynah-slm
src/arch_qwen3.c:229-234, src/kernels.c:193-205). Parameters: hidden_size,
intermediate_size, activation (only "silu" is built), prefix. Gate and up are
kept as one fused matrix [2 * intermediate, hidden], gate rows first, so a
step is two products instead of three.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.keys import ConfigError
from ..ops import kernels
from .base import FeedForward, TensorSpec, register_ffn


class SwiGLUDense(FeedForward):
    accepts_normed = True        # its first product can compute the norm on its way

    def __init__(self, spec):
        super().__init__(spec)
        self.D = int(spec["hidden_size"])
        self.F = int(spec["intermediate_size"])
        self.prefix = str(spec["prefix"])
        act = spec.get("activation", "silu")
        if act != "silu":
            raise ConfigError(f"swiglu_dense: activation {act!r} is not supported (only 'silu')")
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> list[TensorSpec]:
        p = self.prefix
        return [TensorSpec(p + "gate_proj.weight", (self.F, self.D)),
                TensorSpec(p + "up_proj.weight", (self.F, self.D)),
                TensorSpec(p + "down_proj.weight", (self.D, self.F))]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        p = self.prefix
        self.w_gate_up = torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors[p + "down_proj.weight"]

    def streamed_tensors(self) -> list:
        return [self.w_gate_up, self.w_down]

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return kernels.linear(kernels.linear_swiglu(h, self.w_gate_up), self.w_down)


register_ffn("swiglu_dense", SwiGLUDense)
