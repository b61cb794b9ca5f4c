"""Matrix products of the bfloat16 path: y = x . w^T, bf16 operands, fp32
accumulation, output bf16 or fp32.

The reference hands its matrix products to a library (its vendored `ingot`,
mynah-slm src/arch_qwen3.c:39-49), and so may this path: shapes that no
hand-written kernel takes go to cuBLAS through `torch.mm`. Hand-written
kernels register themselves in `ROUTES`; each gets the shape first and may
decline it.
"""
from __future__ import annotations

import os
from typing import Callable, Optional

import torch

from . import lib
from .lib import call, ptr, stream_ptr

# Each route: f(x, w, out_dtype, out) -> Tensor or None (declined).
ROUTES: list[Callable[..., Optional[torch.Tensor]]] = []

# Switch for the hand-written tcgen05 product (tests compare it with the library's).
USE_TCGEN05 = True
# The SwiGLU epilogue of the tcgen05 product.
USE_TCGEN05_SWIGLU = True
# Rows from which the tcgen05 tiles (128 rows each) are worth their launch: with one tile of rows or less a
# product has N / 128 CTAs (8 for the narrow matrices), and the library's split-K kernels are faster.
TCGEN05_MIN_ROWS = 129

_STATUS: dict = {}


def status_word(device) -> torch.Tensor:
    """Status word that the tcgen05 kernel reports a timed-out wait through."""
    key = str(device)
    if key not in _STATUS:
        _STATUS[key] = torch.zeros((1,), dtype=torch.int32, device=device)
    return _STATUS[key]


_SMS: dict = {}


def _sm_count(device) -> int:
    key = str(device)
    if key not in _SMS:
        _SMS[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SMS[key]


def tcgen05_supported(M: int, N: int, K: int) -> bool:
    return bool(lib.load().mynah_gemm_tcgen05_supported(M, N, K))


def splits_k(M: int, N: int, K: int, device) -> bool:
    """Whether the bf16-rows product of this shape runs as two halves of K on two CTAs a tile."""
    return bool(lib.load().mynah_gemm_tcgen05_splits_k(M, N, K, _sm_count(device)))


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, N: int, epilogue: int, out: torch.Tensor) -> torch.Tensor:
    """epilogue 0: bf16 rows, 1: fp32 rows, 2: SwiGLU (w = N gate rows then N up rows)."""
    M, K = x.shape
    call("mynah_gemm_tcgen05", ptr(x), ptr(w), ptr(out), M, N, K, out.shape[1], epilogue, _sm_count(x.device),
         ptr(status_word(x.device)), stream_ptr())
    return out


def _tcgen05_route(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, out: Optional[torch.Tensor]):
    M, K = x.shape
    N = w.shape[0]
    if not USE_TCGEN05 or M < TCGEN05_MIN_ROWS or N % 8 or not tcgen05_supported(M, N, K):
        return None
    if not (x.is_contiguous() and w.is_contiguous()) or (out is not None and not out.is_contiguous()):
        return None
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    return gemm_tcgen05(x, w, N, 0 if out_dtype == torch.bfloat16 else 1, out)


ROUTES.append(_tcgen05_route)

# Switch for the q/k/v product with norm, rotation and cache write in its epilogue. Off: with a token's head of
# 128 accumulators in a thread's registers the rotation's table reads (32 vectors a head, a different table row
# in every lane) run one after the other, and the epilogue takes as long as the separate pass it replaces
# (36.5 us against 19.5 + 15 us for 2,048 tokens of the 0.6B shape). The kernel test covers it.
USE_QKV_EPILOGUE = os.environ.get("MYNAH_QKV_EPILOGUE", "0") != "0"


def qkv_rope_supported(x: torch.Tensor, w: torch.Tensor, H: int, KV: int, HD: int) -> bool:
    M, K = x.shape
    return (USE_TCGEN05 and USE_QKV_EPILOGUE and M >= TCGEN05_MIN_ROWS and x.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous() and w.shape[1] == K
            and bool(lib.load().mynah_gemm_qkv_rope_supported(M, H, KV, HD, K)))


def gemm_qkv_rope(x: torch.Tensor, w: torch.Tensor, H: int, KV: int, HD: int, q_gain, k_gain, eps: float,
                  cos, sin, tok_seq: torch.Tensor, tok_pos: torch.Tensor, pages, k_cache, v_cache) -> torch.Tensor:
    """q [M, H * HD] (normed, rotated), and k, v written into the paged cache, from one product. `w` holds the
    q rows, then (with a cache given) the k and v rows. `pages` is the group's PageTableView."""
    from .lib import code
    M, K = x.shape
    q = torch.empty((M, H * HD), dtype=torch.bfloat16, device=x.device)
    call("mynah_gemm_qkv_rope", ptr(x), ptr(w), M, H, KV, HD, K,
         ptr(q_gain), ptr(k_gain), code(q_gain.dtype) if q_gain is not None else 0, float(eps),
         ptr(cos), ptr(sin), cos.shape[0] if cos is not None else 0,
         ptr(tok_seq), ptr(tok_pos),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         ptr(q), q.shape[1], ptr(k_cache), ptr(v_cache),
         _sm_count(x.device), ptr(status_word(x.device)), stream_ptr())
    counters["own"] += 1
    return q

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
