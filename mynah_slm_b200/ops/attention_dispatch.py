"""Chooses the attention kernel of a step.

The tensor-core kernel takes bfloat16 with the head sizes it was built for;
everything else (the whole 32-bit path, other head sizes) runs the general
kernel. Both read the same paged cache and give the same result up to
rounding.
"""
from __future__ import annotations

import os

import torch

from . import kernels


# Switch for the tcgen05 prompt attention (tests compare it with the mma.sync kernel).
USE_TCGEN05_PREFILL = os.environ.get("MYNAH_TCGEN05_ATTN", "1") != "0"


def prefill(qkv: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int,
            k_cache: torch.Tensor, v_cache: torch.Tensor, pages, window: int) -> None:
    if USE_TCGEN05_PREFILL and kernels.attn_prefill_tcgen05_supported(qkv.dtype, H, KV, HD):
        kernels.attn_prefill_tcgen05(qkv, out, ctx.B, ctx.max_q_len, H, KV, HD, k_cache, v_cache,
                                     ctx.cu_q, ctx.kv_len, pages, window, ctx.status)
        return
    if kernels.attn_prefill_tc_supported(qkv.dtype, H, KV, HD):
        kernels.attn_prefill_tc(qkv, out, ctx.B, ctx.max_q_len, H, KV, HD, k_cache, v_cache,
                                ctx.cu_q, ctx.kv_len, pages, window, ctx.status)
        return
    kernels.attn_prefill_generic(qkv, out, ctx.B, ctx.max_q_len, H, KV, HD, k_cache, v_cache,
                                 ctx.cu_q, ctx.kv_len, pages, window, ctx.status)


# The one-launch decode attention (norm, rotation, cache write, pages, merge) saves two launches but repeats
# the query's preparation in every page's CTA, so it pays while a step has few CTAs. Both routes give a
# sequence the same bits, so the choice may depend on the batch. 0 switches it off.
FUSED_DECODE_MAX_CTAS = int(os.environ.get("MYNAH_FUSED_ATTN_MAX_CTAS", "1100"))
# Floats of shared memory that the merge of a (sequence, kv head) has for its pages' weights.
_MERGE_FLOATS = 2048


def _tc_fits(H: int, KV: int, n_splits: int) -> bool:
    return (H // KV) * n_splits <= _MERGE_FLOATS


# Larger steps can still let the pages' kernel prepare the queries and write the new key and value itself (no
# rotation/cache-write launch before it) and merge with a launch of its own. 1: do so.
FUSED_PREP_LARGE = os.environ.get("MYNAH_FUSED_ATTN_PREP", "0") == "1"


def decode_fused_ok(dtype: torch.dtype, H: int, KV: int, HD: int, rotary_dim: int, cos, B: int, n_splits: int) -> bool:
    """Whether the one-launch decode attention takes this layer in this step: the tensor-core sizes, a rotation
    of the whole head or none, and few enough CTAs."""
    if not kernels.attn_decode_tc_supported(dtype, H, KV, HD):
        return False
    if B * KV * n_splits > FUSED_DECODE_MAX_CTAS and not FUSED_PREP_LARGE:
        return False
    return _tc_fits(H, KV, n_splits) and (cos is None or rotary_dim == HD)


def decode_fused_merges(B: int, KV: int, n_splits: int) -> bool:
    """Whether the one-launch form also merges (small steps), or leaves the merge to a launch of its own."""
    return B * KV * n_splits <= FUSED_DECODE_MAX_CTAS


# Whether the pages' kernel of the tensor-core decode attention also merges (the CTA that finishes a sequence's
# kv head last), instead of a merge launch of its own with a CTA per head. The bits are the same; the launch of its
# own measured faster (batch 8: 1.37 against 1.48 ms a step; batch 64: 3.92 against 4.60), so this is off.
MERGE_IN_PAGES_KERNEL = os.environ.get("MYNAH_ATTN_MERGE_IN_PAGES", "0") == "1"


def decode(qkv: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int, k_cache: torch.Tensor,
           v_cache: torch.Tensor, pages, window: int, scratch: torch.Tensor, counters=None) -> None:
    """One query per sequence. Both kernels split a sequence page by page and
    combine in page order, so either gives a sequence the same bits whatever
    the batch."""
    if kernels.attn_decode_tc_supported(qkv.dtype, H, KV, HD) and _tc_fits(H, KV, ctx.decode_splits):
        kernels.attn_decode_tc(qkv, out, ctx.B, H, KV, HD, k_cache, v_cache, ctx.kv_len, pages, window,
                               ctx.decode_splits, scratch, ctx.status,
                               counters if MERGE_IN_PAGES_KERNEL else None)
    else:
        kernels.attn_decode(qkv, out, ctx.B, H, KV, HD, k_cache, v_cache, ctx.kv_len, pages, window,
                            ctx.decode_splits, scratch, ctx.status)
