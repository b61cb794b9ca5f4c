"""Position encodings that a mixer applies to its queries and keys.

`rope_neox`: rotary embedding in the split-half ("NeoX") pairing, element i
with element i + rotary_dim/2, not the interleaved pairing (mynah-slm
src/kernels.c:173-189; docs/qwen3-arch.md:49-53). Parameters: theta and
rotary_dim (the reference rotates the whole head: rotary_dim = head_dim). The
cos/sin table is built once per (theta, rotary_dim) in double precision and
stored as float, like the reference's (src/kernels.c:141-164), and is shared
by every layer that asks for the same pair.

`none`: no position encoding (the mixer then only norms and stores).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import kernels
from .base import PositionEncoding, register_position


class RopeNeox(PositionEncoding):
    fusable = True

    def __init__(self, spec):
        super().__init__(spec)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            from ..config.keys import ConfigError
            raise ConfigError(f"rope_neox: rotary_dim {self.rotary_dim} must be positive and even")
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def prepare(self, runtime) -> None:
        key = ("rope_neox", self.theta, self.rotary_dim)
        if key not in runtime.tables:
            runtime.tables[key] = kernels.rope_table(runtime.max_positions, self.rotary_dim, self.theta, runtime.device)
        self.cos, self.sin = runtime.tables[key]

    def fused_tables(self):
        return self.cos, self.sin, self.rotary_dim


class NoPosition(PositionEncoding):
    fusable = True

    def fused_tables(self):
        return None, None, 0


register_position("rope_neox", RopeNeox)
register_position("none", NoPosition)
