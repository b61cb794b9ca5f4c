"""Matrix products of the bfloat16 path: y = x . w^T, bf16 operands, fp32
accumulation, output bf16 or fp32.

The reference hands its matrix products to a library (its vendored `ingot`,
mynah-slm src/arch_qwen3.c:39-49), and so may this path: shapes that no
hand-written kernel takes go to cuBLAS through `torch.mm`. Hand-written
kernels register themselves in `ROUTES`; each gets the shape first and may
decline it.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

# Each route: f(x, w, out_dtype, out) -> Tensor or None (declined).
ROUTES: list[Callable[..., Optional[torch.Tensor]]] = []

# Launch count of hand-written matrix-product kernels (read by the benchmark).
counters = {"own": 0, "library": 0}


def linear_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    for route in ROUTES:
        y = route(x, w, out_dtype, out)
        if y is not None:
            counters["own"] += 1
            return y
    counters["library"] += 1
    if out_dtype == torch.bfloat16:
        if out is None:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out=out)
    if out_dtype == torch.float32:
        if out is None:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    raise ValueError(f"linear_bf16: unsupported output dtype {out_dtype}")
