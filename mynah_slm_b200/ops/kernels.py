"""Tensor-level wrappers of the kernel entry points.

Each function checks what the kernel cannot (device, dtype, contiguity,
shapes) and launches on the current CUDA stream. Matrix products of the
bfloat16 path go to the library (`torch.mm`, i.e. cuBLAS) here unless a
hand-written kernel takes the shape; everything else is this package's own
CUDA.
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import Optional

import torch

from ..cache.pages import PAGE_TOKENS
from . import lib
from .lib import KernelError, call, code, ptr, stream_ptr

MAX_HEAD_DIM = 256

ST_PAGE_RANGE, ST_POS_RANGE, ST_TOKEN_RANGE, ST_SPLIT_RANGE = 1, 2, 4, 8


def _chk(t: torch.Tensor, name: str, dtype=None, dim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name} has {t.dim()} dimensions, expected {dim}")


@dataclass
class PageTableView:
    """A cache group's page lists for the sequences of one step (device)."""
    indptr: torch.Tensor      # int32 [B+1]
    ids: torch.Tensor         # int32 [>= indptr[B]]
    base: torch.Tensor        # int32 [B]
    n_pages: int


def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(table, "embedding table", dim=2)
    _chk(tokens, "tokens", torch.int32, 1)
    T, (V, D) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    call("mynah_embed_gather", ptr(table), code(table.dtype), ptr(tokens), ptr(out), T, D, V, stream_ptr())
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, act_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h = RMSNorm(x (+ delta)) * gain. Without `rows`, x is updated in place when delta is given; with `rows`
    (which may name a row more than once) x is only read."""
    _chk(x, "residual", torch.float32, 2)
    _chk(gain, "norm gain", dim=1)
    T, D = x.shape
    if gain.numel() != D:
        raise KernelError(f"norm gain has {gain.numel()} elements, the rows have {D}")
    if delta is not None:
        _chk(delta, "delta", act_dtype, 2)
        if delta.shape != x.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match the residual {tuple(x.shape)}")
    n = T
    if rows is not None:
        _chk(rows, "rows", torch.int32, 1)
        n = rows.numel()
    if out is None:
        out = torch.empty((n, D), dtype=act_dtype, device=x.device)
    call("mynah_rmsnorm", ptr(x), ptr(delta), ptr(gain), code(gain.dtype), ptr(rows), ptr(out), code(act_dtype),
         n, D, float(eps), stream_ptr())
    return out


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    _chk(x, "residual", torch.float32)
    _chk(delta, "delta")
    if delta.shape != x.shape:
        raise KernelError("residual_add: shapes differ")
    call("mynah_residual_add", ptr(x), ptr(delta), code(delta.dtype), x.numel(), stream_ptr())


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(gate_up, "gate_up", dim=2)
    T, F2 = gate_up.shape
    if F2 % 2:
        raise KernelError("swiglu: the input must hold gate and up side by side")
    if out is None:
        out = torch.empty((T, F2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    call("mynah_swiglu", ptr(gate_up), ptr(out), code(gate_up.dtype), T, F2 // 2, stream_ptr())
    return out


class NormedInput:
    """A norm that has not been run yet: the residual rows, the pending add and
    the gain. A matrix product that can compute the norm on its way takes it as
    it is (`linear`, `linear_swiglu`); anything else calls `materialize`."""

    def __init__(self, stream, delta, gain: torch.Tensor, eps: float, act_dtype: torch.dtype):
        self.stream, self.delta, self.gain, self.eps, self.act_dtype = stream, delta, gain, float(eps), act_dtype
        self.shape = stream.x.shape
        self.dtype = act_dtype
        self._h: Optional[torch.Tensor] = None

    def materialize(self) -> torch.Tensor:
        if self._h is None:
            self._h = rmsnorm(self.stream.x, self.gain, self.eps, self.act_dtype, delta=self.delta)
            self.delta = None
        return self._h


_SM_COUNT: dict = {}


def _sm_count(device) -> int:
    if device not in _SM_COUNT:
        _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[device]


def gemv_decode_mode(mode: int) -> int:
    """How the decode products read their weights: 0 straight into registers, 1 through a ring of asynchronous copies
    in shared memory, 2 (the default) whichever the shape does better with. Returns the mode set before; a row's
    sums are the same bits either way."""
    return int(lib.load().mynah_gemv_decode_mode(int(mode)))


def gemv_decode_supported(M: int, N: int, K: int) -> bool:
    return bool(lib.load().mynah_gemv_decode_supported(M, N, K))


def _gemv_decode(x, w: torch.Tensor, N: int, epilogue: int, out: torch.Tensor) -> torch.Tensor:
    """x: bf16 rows [M, K] or a NormedInput. epilogue 0: bf16, 1: SwiGLU (w holds N gate rows then N up rows), 2: fp32."""
    K = w.shape[1]
    if isinstance(x, NormedInput) and x._h is None and (x.shape[0] > FUSED_NORM_MAX_ROWS or not _norm_prologue_fits(x.shape[0], K)):
        x.materialize()
    if isinstance(x, NormedInput) and x._h is None:
        st = x.stream
        M = st.x.shape[0]
        new_x = torch.empty_like(st.x) if x.delta is not None else None
        call("mynah_gemv_decode", ptr(w), N, K, M, None, ptr(st.x), ptr(x.delta), ptr(new_x),
             ptr(x.gain), code(x.gain.dtype), x.eps, ptr(out), out.shape[1], epilogue, _sm_count(w.device), stream_ptr())
        if new_x is not None:
            st.x = new_x                       # the residual with the add done, written by the kernel
            x.delta = None
        return out
    if isinstance(x, NormedInput):
        x = x._h
    call("mynah_gemv_decode", ptr(w), N, K, x.shape[0], ptr(x), None, None, None, None, 0, 0.0,
         ptr(out), out.shape[1], epilogue, _sm_count(w.device), stream_ptr())
    return out


# Many outputs of long rows (the q/k/v and gate/up products of the 4B and 8B shapes): the library's kernels stream such
# matrices at 5.4 to 5.6 TB/s where gemv_decode reaches 2.8 to 4.4 (`python bench.py --only products --shape 8b`), so
# they are left to it, as the reference leaves its products to a library. 0 rows: never.
GEMV_LIBRARY_FROM_ROWS = int(os.environ.get("MYNAH_GEMV_LIBRARY_FROM_ROWS", "6144"))
GEMV_LIBRARY_FROM_K = 2048
# From nine rows on (the second half of the tensor cores' sixteen rows is then in use) the library also does better
# on every large matrix of long rows: 8B down 4,096 x 12,288 at 16 rows takes 21.8 us there against 32.2, 8B o 9.8
# against 13.6, 4B down 15.3 against 17.3; at 8 rows the own kernels are level or ahead. 0 elements: never.
GEMV_LIBRARY_FROM_ELEMENTS_9_ROWS = int(os.environ.get("MYNAH_GEMV_LIBRARY_FROM_ELEMENTS_9_ROWS", str(1 << 23)))


def _fusable(x, w: torch.Tensor, N: int) -> bool:
    if w.dtype != torch.bfloat16 or not w.is_contiguous():
        return False
    if GEMV_LIBRARY_FROM_ROWS and w.shape[0] >= GEMV_LIBRARY_FROM_ROWS and w.shape[1] >= GEMV_LIBRARY_FROM_K:
        return False
    if isinstance(x, NormedInput):
        if x.act_dtype != torch.bfloat16:
            return False
        M, K = x.shape
        if x._h is None and (x.gain.numel() != K or not x.stream.x.is_contiguous()):
            return False
    else:
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            return False
        M, K = x.shape
    if (GEMV_LIBRARY_FROM_ELEMENTS_9_ROWS and M > 8 and K >= GEMV_LIBRARY_FROM_K
            and w.shape[0] * w.shape[1] >= GEMV_LIBRARY_FROM_ELEMENTS_9_ROWS):
        return False
    return K == w.shape[1] and N <= GEMV_MAX_OUT_ROWS and gemv_decode_supported(M, N, K)


# Rows up to which the norm runs as the product's prologue. 0: never. Since the products spread over up to four
# CTAs an SM, every CTA recomputing the norm costs as much as the separate norm kernel at one row (0.985 vs
# 0.980 ms a step at batch 1) and more from two rows on (1.155 vs 1.045 ms at batch 2), so it is off; the
# prologue stays in the kernel and in the tests.
FUSED_NORM_MAX_ROWS = int(os.environ.get("MYNAH_FUSED_NORM_MAX_ROWS", "0"))
def _norm_prologue_fits(M: int, K: int) -> bool:
    """The norm prologue keeps its rows (8 or 16 of them, padded) in shared memory beside the 80 KB ring of weights."""
    return (16 if M > 8 else 8) * (K + 32) * 2 + 80 * 1024 <= 200 * 1024
GEMV_MAX_OUT_ROWS = 32768   # wider products (the output head) stream better through the library for now


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x . w^T with w [out, in] row-major (no bias). float32 runs the
    package's FFMA kernel (true 32-bit); bfloat16 accumulates in fp32. `x` may
    be a NormedInput: a few bf16 rows then take the fused norm+product kernel."""
    _chk(w, "linear weight", dim=2)
    out_dtype = out_dtype or (x.dtype if not isinstance(x, NormedInput) else x.act_dtype)
    N = w.shape[0]
    if out_dtype in (torch.bfloat16, torch.float32) and _fusable(x, w, N):
        if out is None:
            out = torch.empty((x.shape[0], N), dtype=out_dtype, device=w.device)
        from . import gemm_bf16
        gemm_bf16.counters["own"] += 1
        return _gemv_decode(x, w, N, 0 if out_dtype == torch.bfloat16 else 2, out)
    if isinstance(x, NormedInput):
        x = x.materialize()
    _chk(x, "linear input", dim=2)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or x.dtype != w.dtype:
        raise KernelError(f"linear: input [{M},{K}] {x.dtype} does not fit weight [{N},{K2}] {w.dtype}")
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise KernelError("linear: the 32-bit path writes float32")
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        call("mynah_gemm_f32", ptr(x), ptr(w), ptr(out), M, N, K, K, K, N, stream_ptr())
        return out
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported dtype {x.dtype}")
    from . import gemm_bf16
    return gemm_bf16.linear_bf16(x, w, out_dtype, out)


def linear_swiglu(x, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) with w_gate_up = [Wg; Wu] ([2F, K]); one kernel for a few bf16 rows."""
    F = w_gate_up.shape[0] // 2
    if _fusable(x, w_gate_up, F):
        out = torch.empty((x.shape[0], F), dtype=torch.bfloat16, device=w_gate_up.device)
        from . import gemm_bf16
        gemm_bf16.counters["own"] += 1
        return _gemv_decode(x, w_gate_up, F, 1, out)
    from . import gemm_bf16
    if isinstance(x, NormedInput):
        x = x.materialize()
    if (x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and gemm_bf16.USE_TCGEN05 and gemm_bf16.USE_TCGEN05_SWIGLU
            and x.shape[0] >= gemm_bf16.TCGEN05_MIN_ROWS and F % 8 == 0 and x.is_contiguous()
            and w_gate_up.is_contiguous() and gemm_bf16.tcgen05_supported(x.shape[0], F, x.shape[1])):
        out = torch.empty((x.shape[0], F), dtype=torch.bfloat16, device=x.device)
        gemm_bf16.counters["own"] += 1
        return gemm_bf16.gemm_tcgen05(x, w_gate_up, F, 2, out)      # the activation runs on the accumulator
    return swiglu(linear(x, w_gate_up))


def rope_table(n_pos: int, rotary_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    half = rotary_dim // 2
    cos = torch.empty((n_pos, half), dtype=torch.float32, device=device)
    sin = torch.empty((n_pos, half), dtype=torch.float32, device=device)
    # theta is a float in the reference's table builder (mynah-slm src/kernels.c:141)
    theta32 = float(torch.tensor(theta, dtype=torch.float32))
    call("mynah_rope_table", ptr(cos), ptr(sin), n_pos, rotary_dim, theta32, stream_ptr())
    return cos, sin


def qk_norm_rope_store(qkv: torch.Tensor, H: int, KV: int, HD: int,
                       q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                       tok_seq: torch.Tensor, tok_pos: torch.Tensor, pages: PageTableView,
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       status: torch.Tensor) -> None:
    _chk(qkv, "qkv", dim=2)
    T, ld = qkv.shape
    if (q_gain is None) != (k_gain is None):
        raise KernelError("qk_norm_rope_store: q and k gains go together")
    gd = 0
    if q_gain is not None:
        if q_gain.dtype != k_gain.dtype or q_gain.numel() != HD or k_gain.numel() != HD:
            raise KernelError("qk_norm_rope_store: the head gains must both have head_dim elements of one dtype")
        gd = code(q_gain.dtype)
    n_pos = 0
    if cos is not None:
        _chk(cos, "cos table", torch.float32, 2)
        n_pos = cos.shape[0]
        if cos.shape[1] * 2 != rotary_dim:
            raise KernelError("qk_norm_rope_store: the rotation table does not match rotary_dim")
    if k_cache is not None:
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_store: the cache and the activations differ in dtype")
        if tuple(k_cache.shape[1:]) != (KV, PAGE_TOKENS, HD):
            raise KernelError(f"qk_norm_rope_store: cache pages are {tuple(k_cache.shape[1:])}, expected {(KV, PAGE_TOKENS, HD)}")
    call("mynah_qk_norm_rope_store", ptr(qkv), code(qkv.dtype), T, H, KV, HD, ld,
         ptr(q_gain), ptr(k_gain), gd, float(eps),
         ptr(cos), ptr(sin), rotary_dim, n_pos,
         ptr(tok_seq), ptr(tok_pos),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         ptr(k_cache), ptr(v_cache), ptr(status), stream_ptr())


def attn_prefill_generic(qkv: torch.Tensor, out: torch.Tensor, B: int, max_q_len: int, H: int, KV: int, HD: int,
                         k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                         pages: PageTableView, window: int, status: torch.Tensor) -> None:
    """q is read from the first H*HD columns of `qkv` (row stride qkv.shape[1])."""
    _chk(qkv, "q", dim=2)
    _chk(out, "attention output", qkv.dtype, 2)
    call("mynah_attn_prefill_generic", ptr(qkv), ptr(out), code(qkv.dtype), qkv.shape[0], B, max_q_len, H, KV, HD,
         qkv.shape[1], out.shape[1], ptr(k_cache), ptr(v_cache), ptr(cu_q), ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages, window or 0, ptr(status), stream_ptr())


def attn_prefill_tc_supported(dtype: torch.dtype, H: int, KV: int, HD: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib.load().mynah_attn_prefill_tc_supported(H, KV, HD))


def attn_prefill_tc(qkv: torch.Tensor, out: torch.Tensor, B: int, max_q_len: int, H: int, KV: int, HD: int,
                    k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                    pages: PageTableView, window: int, status: torch.Tensor) -> None:
    """The tensor-core prompt attention (bfloat16, head_dim 64 or 128); same contract as attn_prefill_generic."""
    _chk(qkv, "q", torch.bfloat16, 2)
    _chk(out, "attention output", torch.bfloat16, 2)
    call("mynah_attn_prefill_tc", ptr(qkv), ptr(out), qkv.shape[0], B, max_q_len, H, KV, HD, qkv.shape[1], out.shape[1],
         ptr(k_cache), ptr(v_cache), ptr(cu_q), ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages, window or 0, ptr(status), stream_ptr())


def attn_prefill_tcgen05_supported(dtype: torch.dtype, H: int, KV: int, HD: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib.load().mynah_attn_prefill_tcgen05_supported(H, KV, HD))


def attn_prefill_tcgen05(qkv: torch.Tensor, out: torch.Tensor, B: int, max_q_len: int, H: int, KV: int, HD: int,
                         k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                         pages: PageTableView, window: int, status: torch.Tensor) -> None:
    """The prompt attention on tcgen05 (bfloat16, head_dim 64 or 128); same contract as attn_prefill_generic."""
    _chk(qkv, "q", torch.bfloat16, 2)
    _chk(out, "attention output", torch.bfloat16, 2)
    _chk(k_cache, "K cache", torch.bfloat16)
    _chk(v_cache, "V cache", torch.bfloat16)
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError("attn_prefill_tcgen05: the cache tensors must be contiguous")
    call("mynah_attn_prefill_tcgen05", ptr(qkv), ptr(out), qkv.shape[0], B, max_q_len, H, KV, HD, qkv.shape[1], out.shape[1],
         ptr(k_cache), ptr(v_cache), ptr(cu_q), ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages, window or 0, ptr(status), stream_ptr())


def attn_prefill_tcgen05_stages(mode: int) -> None:
    """0: the prompt attention chooses its form by the number of CTAs; 1: one stage of K, V and scores, two CTAs an
    SM; 2: two stages, one CTA an SM. Both give the same bits."""
    call("mynah_attn_prefill_tcgen05_stages", int(mode))


def attn_decode_scratch_floats(B: int, H: int, HD: int, n_splits: int) -> int:
    return int(lib.load().mynah_attn_decode_scratch_floats(B, H, HD, n_splits))


def attn_decode(qkv: torch.Tensor, out: torch.Tensor, B: int, H: int, KV: int, HD: int,
                k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len: torch.Tensor, pages: PageTableView,
                window: int, n_splits: int, scratch: torch.Tensor, status: torch.Tensor) -> None:
    _chk(qkv, "q", dim=2)
    _chk(out, "attention output", qkv.dtype, 2)
    _chk(scratch, "scratch", torch.float32)
    need = B * H * n_splits * (HD + 2)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode: scratch holds {scratch.numel()} floats, {need} are needed")
    call("mynah_attn_decode", ptr(qkv), ptr(out), code(qkv.dtype), B, H, KV, HD, qkv.shape[1], out.shape[1],
         ptr(k_cache), ptr(v_cache), ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         window or 0, n_splits, ptr(scratch), ptr(status), stream_ptr())


def attn_decode_tc_supported(dtype: torch.dtype, H: int, KV: int, HD: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib.load().mynah_attn_decode_tc_supported(H, KV, HD))


def attn_decode_stream_mode(mode: int) -> int:
    """How the tensor-core decode attention walks a step's pages: 0 one page a CTA, 2 persistent CTAs fed by TMA
    wherever that can run, 1 (the default) whichever pays. Returns the mode set before; the results are the same
    bits either way."""
    return int(lib.load().mynah_attn_decode_stream_mode(int(mode)))


def attn_decode_tc(qkv: torch.Tensor, out: torch.Tensor, B: int, H: int, KV: int, HD: int,
                   k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len: torch.Tensor, pages: PageTableView,
                   window: int, n_splits: int, scratch: torch.Tensor, status: torch.Tensor,
                   counters: Optional[torch.Tensor] = None) -> None:
    """The tensor-core decode attention (bfloat16, head_dim 64 or 128); same contract as attn_decode. With
    `counters` (B * KV zeroed int32 words, left zero) the pages' kernel also merges and no second launch is made;
    the result is the same."""
    _chk(qkv, "q", torch.bfloat16, 2)
    if counters is not None:
        _chk(counters, "counters", torch.int32, 1)
        if counters.numel() < B * KV:
            raise KernelError(f"attn_decode_tc: {counters.numel()} counters, {B * KV} are needed")
    _chk(out, "attention output", torch.bfloat16, 2)
    _chk(scratch, "scratch", torch.float32)
    need = B * H * n_splits * (HD + 2)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode_tc: scratch holds {scratch.numel()} floats, {need} are needed")
    call("mynah_attn_decode_tc", ptr(qkv), ptr(out), B, H, KV, HD, qkv.shape[1], out.shape[1],
         ptr(k_cache), ptr(v_cache), ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         window or 0, n_splits, ptr(scratch), ptr(counters), ptr(status), stream_ptr())


def attn_decode_fused(qkv: torch.Tensor, out: torch.Tensor, B: int, H: int, KV: int, HD: int,
                      q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], qk_eps: float,
                      cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], tok_pos: torch.Tensor,
                      k_cache: torch.Tensor, v_cache: torch.Tensor, write_kv: bool, kv_len: torch.Tensor,
                      pages: PageTableView, window: int, n_splits: int, scratch: torch.Tensor,
                      counters: Optional[torch.Tensor], status: torch.Tensor) -> None:
    """Per-head norm, rotation, cache write and attention of a decode step in one launch (bfloat16, head_dim 64
    or 128, whole-head rotation or none). `qkv` holds the projection's rows; with write_kv False only q is read."""
    _chk(qkv, "qkv", torch.bfloat16, 2)
    _chk(out, "attention output", torch.bfloat16, 2)
    _chk(scratch, "scratch", torch.float32)
    # counters None: the pages' CTAs do not merge, the merge follows as a launch of its own (the same bits)
    need = B * H * n_splits * (HD + 2)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode_fused: scratch holds {scratch.numel()} floats, {need} are needed")
    if counters is not None:
        _chk(counters, "counters", torch.int32)
        if counters.numel() < B * KV:
            raise KernelError(f"attn_decode_fused: {counters.numel()} counters, {B * KV} are needed")
    if cos is not None and cos.shape[1] * 2 != HD:
        raise KernelError("attn_decode_fused: the rotation must cover the whole head")
    call("mynah_attn_decode_fused", ptr(qkv), ptr(out), B, H, KV, HD, qkv.shape[1], out.shape[1],
         ptr(q_gain), ptr(k_gain), code(q_gain.dtype) if q_gain is not None else 0, float(qk_eps),
         ptr(cos), ptr(sin), cos.shape[0] if cos is not None else 0, ptr(tok_pos),
         ptr(k_cache), ptr(v_cache), 1 if write_kv else 0, ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         window or 0, n_splits, ptr(scratch), ptr(counters), ptr(status), stream_ptr())


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(logits, "logits", torch.float32, 2)
    B, V = logits.shape
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    call("mynah_argmax", ptr(logits), B, V, V, ptr(out), stream_ptr())
    return out


def sample(logits: torch.Tensor, params: torch.Tensor, rng: torch.Tensor, slots: Optional[torch.Tensor],
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Overwrites `logits`. params: float32 [7] on the device (temp, top_p,
    min_p, top_k, repeat, freq, presence); rng: int64 generator state per slot."""
    _chk(logits, "logits", torch.float32, 2)
    _chk(rng, "rng states", torch.int64, 1)
    _chk(params, "sampling parameters", torch.float32, 1)
    B, V = logits.shape
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    pv = pi = None
    if V >= SAMPLE_TWO_STEP_MIN_VOCAB:
        pv, pi = _sample_scratch(logits.device, B)
    call("mynah_sample", ptr(logits), B, V, V, ptr(params), ptr(rng), ptr(slots), ptr(out), ptr(pv), ptr(pi), stream_ptr())
    return out


# From this vocabulary size on a row's maximum is found by several CTAs first (one CTA reads a long row slowly).
SAMPLE_TWO_STEP_MIN_VOCAB = 16384
_SAMPLE_SCRATCH: dict = {}


def _sample_scratch(device, B: int):
    """Scratch of the two-step maximum, kept for the life of the process (a captured step holds its address)."""
    key = (str(device), B)
    if key not in _SAMPLE_SCRATCH:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("sample: scratch memory must exist before graph capture")
        n = B * int(lib.load().mynah_argmax_parts())
        _SAMPLE_SCRATCH[key] = (torch.empty((n,), dtype=torch.float32, device=device),
                                torch.empty((n,), dtype=torch.int32, device=device))
    return _SAMPLE_SCRATCH[key]


def apply_penalties(logits: torch.Tensor, ring: torch.Tensor, ring_n: torch.Tensor, slots: Optional[torch.Tensor],
                    params: torch.Tensor) -> None:
    _chk(logits, "logits", torch.float32, 2)
    _chk(ring, "ring", torch.int32, 2)
    B, V = logits.shape
    call("mynah_apply_penalties", ptr(logits), B, V, V, ptr(ring), ptr(ring_n), ring.shape[1], ptr(slots),
         ptr(params), stream_ptr())


def sampler_accept(tokens: torch.Tensor, ring: torch.Tensor, ring_n: torch.Tensor, ring_head: torch.Tensor,
                   slots: Optional[torch.Tensor], params: torch.Tensor) -> None:
    _chk(tokens, "tokens", torch.int32, 1)
    call("mynah_sampler_accept", ptr(tokens), tokens.numel(), ptr(ring), ptr(ring_n), ptr(ring_head),
         ring.shape[1], ptr(slots), ptr(params), stream_ptr())


def decode_advance(tokens: torch.Tensor, sampled: torch.Tensor, tok_pos: torch.Tensor, kv_len: torch.Tensor,
                   slots: torch.Tensor) -> None:
    call("mynah_decode_advance", ptr(tokens), ptr(sampled), ptr(tok_pos), ptr(kv_len), ptr(slots),
         tokens.numel(), stream_ptr())


def l2_prefetch(tensors) -> None:
    """Ask the memory system to bring these tensors (contiguous, at most 8) into L2; returns at once and computes
    nothing. Meant for a second stream beside a chain of kernels that will read the tensors shortly."""
    import ctypes
    ts = [t for t in tensors if t is not None and t.is_cuda and t.is_contiguous() and t.numel()]
    for i in range(0, len(ts), 8):
        part = ts[i:i + 8]
        ptrs = (ctypes.c_void_p * len(part))(*[t.data_ptr() for t in part])
        sizes = (ctypes.c_ulonglong * len(part))(*[t.numel() * t.element_size() for t in part])
        call("mynah_l2_prefetch", ptrs, sizes, len(part), stream_ptr())
