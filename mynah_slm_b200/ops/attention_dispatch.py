"""Chooses the attention kernel of a step.

The tensor-core kernel takes bfloat16 with the head sizes it was built for;
everything else (the whole 32-bit path, other head sizes) runs the general
kernel. Both read the same paged cache and give the same result up to
rounding.
"""
from __future__ import annotations

import torch

from . import kernels


def prefill(qkv: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int,
            k_cache: torch.Tensor, v_cache: torch.Tensor, pages, window: int) -> None:
    if kernels.attn_prefill_tc_supported(qkv.dtype, H, KV, HD):
        kernels.attn_prefill_tc(qkv, out, ctx.B, ctx.max_q_len, H, KV, HD, k_cache, v_cache,
                                ctx.cu_q, ctx.kv_len, pages, window, ctx.status)
        return
    kernels.attn_prefill_generic(qkv, out, ctx.B, ctx.max_q_len, H, KV, HD, k_cache, v_cache,
                                 ctx.cu_q, ctx.kv_len, pages, window, ctx.status)


def decode(qkv: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int, k_cache: torch.Tensor,
           v_cache: torch.Tensor, pages, window: int, scratch: torch.Tensor) -> None:
    """One query per sequence. Both kernels split a sequence page by page and
    combine in page order, so either gives a sequence the same bits whatever
    the batch."""
    if kernels.attn_decode_tc_supported(qkv.dtype, H, KV, HD):
        kernels.attn_decode_tc(qkv, out, ctx.B, H, KV, HD, k_cache, v_cache, ctx.kv_len, pages, window,
                               ctx.decode_splits, scratch, ctx.status)
    else:
        kernels.attn_decode(qkv, out, ctx.B, H, KV, HD, k_cache, v_cache, ctx.kv_len, pages, window,
                            ctx.decode_splits, scratch, ctx.status)
