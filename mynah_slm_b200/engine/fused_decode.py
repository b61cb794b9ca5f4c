"""The fused decode step: when every layer of the model is the standard
pre-norm block (RMSNorm, grouped-query attention with per-head RMSNorm or
none and whole-head split-half rotation or none, SwiGLU feed-forward), the run
is bfloat16 and the batch has at most 16 sequences, a decode step runs as ONE
persistent kernel (`csrc/decode_step.cu`) instead of one launch per part.

The parts stay the description of the model: this module only reads their
tensors and parameters into the table the kernel walks. Anything it does not
recognise (another mixer, another feed-forward, a run that reads another run's
cache, a part that plans on the host) makes `plan` return None and the step
goes part by part as before; the tests compare the two paths.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import lib
from ..ops.lib import call, code, ptr, stream_ptr
from ..parts.attention import GQAttention
from ..parts.block import PreNormResidual
from ..parts.feedforward import SwiGLUDense
from ..parts.norms import RMSNorm
from ..parts.position import NoPosition, RopeNeox

MAX_ROWS = 16
_SIGNATURE_DONE = False


def _declare() -> None:
    global _SIGNATURE_DONE
    if _SIGNATURE_DONE:
        return
    h = lib.load()
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    h.mynah_decode_step_supported.restype = I
    h.mynah_decode_step_supported.argtypes = [I] * 8
    h.mynah_decode_step_layer_bytes.restype = I
    h.mynah_decode_step_layer_bytes.argtypes = []
    lib.register("mynah_decode_step_fill_layer", [P, P, P, P, P, P, I, P, I, P, P, I, P, P, P, P, I, I, I])
    lib.register("mynah_decode_step", [I] * 9 + [F, F] + [P, P, P, P] + [I, P, P, P, P] + [P, P, I, P]
                 + [P] * 10 + [I, P, P, P])
    _SIGNATURE_DONE = True


@dataclass
class _Buffers:
    x0: torch.Tensor
    x1: torch.Tensor
    qkv: torch.Tensor
    attn: torch.Tensor
    delta: torch.Tensor
    act: torch.Tensor
    part: torch.Tensor
    counters: torch.Tensor
    logits: torch.Tensor


class FusedDecode:
    """The table of layers on the device, and the work buffers per batch size."""

    def __init__(self, model, cache, runtime):
        _declare()
        self.runtime = runtime
        self.device = runtime.device
        first: GQAttention = model.layers[model.schedule[0].layer].mixer
        ffn: SwiGLUDense = model.layers[model.schedule[0].layer].ffn
        self.D, self.H, self.KV, self.HD, self.F = first.D, first.H, first.KV, first.HD, ffn.F
        self.V = model.spec.vocab_size
        self.eps = model.final_norm.eps
        self.qk_eps = first.qk_eps
        self.n_layers = len(model.schedule)
        self.n_groups = len(cache.plan.groups)
        self.embed = model.embedding.table
        self.final_gain = model.final_norm.gain
        self.head = model.head.weight
        nbytes = lib.load().mynah_decode_step_layer_bytes()
        host = (ctypes.c_ubyte * (nbytes * self.n_layers))()
        for i, e in enumerate(model.schedule):
            blk = model.layers[e.layer]
            att: GQAttention = blk.mixer
            ff: SwiGLUDense = blk.ffn
            view = cache.views[i]
            cos, sin, _ = att.position.fused_tables()
            call("mynah_decode_step_fill_layer", ctypes.addressof(host) + i * nbytes,
                 ptr(att.w_qkv), ptr(att.w_o), ptr(ff.w_gate_up), ptr(ff.w_down),
                 ptr(blk.norms["mixer"].gain), code(blk.norms["mixer"].gain.dtype),
                 ptr(blk.norms["ffn"].gain), code(blk.norms["ffn"].gain.dtype),
                 ptr(att.q_gain), ptr(att.k_gain), code(att.q_gain.dtype) if att.q_gain is not None else 0,
                 ptr(view.k), ptr(view.v), ptr(cos), ptr(sin), cos.shape[0] if cos is not None else 0,
                 view.group, att.window or 0)
        self.layers_dev = torch.frombuffer(bytearray(host), dtype=torch.uint8).to(self.device)
        self.sync = torch.zeros((4,), dtype=torch.int32, device=self.device)
        self.sm_count = runtime.sm_count
        self.trace: Optional[torch.Tensor] = None      # int64 [64]: time stamps of CTA 0, when set (tuning aid)
        self._bufs: dict[tuple[int, int], _Buffers] = {}

    def supported(self, rows: int, pages: int) -> bool:
        return bool(lib.load().mynah_decode_step_supported(rows, self.D, self.H, self.KV, self.HD, self.F, self.V, pages))

    def buffers(self, rows: int, pages: int) -> _Buffers:
        key = (rows, pages)
        if key not in self._bufs:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the fused decode step's buffers must exist before capture")
            d, bf, f32 = self.device, torch.bfloat16, torch.float32
            self._bufs[key] = _Buffers(
                x0=torch.empty((rows, self.D), dtype=f32, device=d), x1=torch.empty((rows, self.D), dtype=f32, device=d),
                qkv=torch.empty((rows, (self.H + 2 * self.KV) * self.HD), dtype=bf, device=d),
                attn=torch.empty((rows, self.H * self.HD), dtype=bf, device=d),
                delta=torch.empty((rows, self.D), dtype=bf, device=d), act=torch.empty((rows, self.F), dtype=bf, device=d),
                part=torch.empty((rows * self.H * pages * (self.HD + 2),), dtype=f32, device=d),
                counters=torch.zeros((rows * self.KV,), dtype=torch.int32, device=d),
                logits=torch.empty((rows, self.V), dtype=f32, device=d))
        return self._bufs[key]

    def run(self, ctx) -> torch.Tensor:
        """One decode step for the batch that `ctx` describes; returns fp32 logits [rows, vocab]."""
        rows, pages = ctx.B, ctx.decode_splits
        b = self.buffers(rows, pages)
        PP = ctypes.c_void_p * self.n_groups
        indptr = PP(*[ctx.pages[g].indptr.data_ptr() for g in range(self.n_groups)])
        ids = PP(*[ctx.pages[g].ids.data_ptr() for g in range(self.n_groups)])
        base = PP(*[ctx.pages[g].base.data_ptr() for g in range(self.n_groups)])
        n_pages = (ctypes.c_int * self.n_groups)(*[ctx.pages[g].n_pages for g in range(self.n_groups)])
        call("mynah_decode_step", self.n_layers, rows, self.D, self.H, self.KV, self.HD, self.F, self.V, pages,
             float(self.eps), float(self.qk_eps),
             ptr(self.layers_dev), ptr(ctx.tokens), ptr(ctx.tok_pos), ptr(ctx.kv_len),
             self.n_groups, ctypes.cast(indptr, ctypes.c_void_p), ctypes.cast(ids, ctypes.c_void_p),
             ctypes.cast(base, ctypes.c_void_p), ctypes.cast(n_pages, ctypes.c_void_p),
             ptr(self.embed), ptr(self.final_gain), code(self.final_gain.dtype), ptr(self.head),
             ptr(b.x0), ptr(b.x1), ptr(b.qkv), ptr(b.attn), ptr(b.delta), ptr(b.act), ptr(b.part), ptr(b.counters),
             ptr(self.sync), ptr(b.logits), self.sm_count, ptr(ctx.status), ptr(self.trace), stream_ptr())
        return b.logits

    def reset_after_abort(self) -> None:
        self.sync.zero_()
        for b in self._bufs.values():
            b.counters.zero_()


def plan(model, cache, runtime) -> Optional[FusedDecode]:
    """A FusedDecode for this model, or None when some part is not the standard one."""
    if runtime.act_dtype != torch.bfloat16:
        return None
    sizes = None
    for e in model.schedule:
        if e.cache_from is not None:
            return None
        blk = model.layers[e.layer]
        if type(blk) is not PreNormResidual or type(blk.mixer) is not GQAttention or type(blk.ffn) is not SwiGLUDense:
            return None
        att, ff = blk.mixer, blk.ffn
        if any(type(n) is not RMSNorm for n in blk.norms.values()):
            return None
        pos = att.position
        if type(pos) is RopeNeox:
            if pos.rotary_dim != att.HD:
                return None
        elif type(pos) is not NoPosition:
            return None
        mine = (att.D, att.H, att.KV, att.HD, ff.F, ff.D, att.qk_eps if att.has_qk_norm else None, att.has_qk_norm,
                blk.norms["mixer"].eps, blk.norms["ffn"].eps, type(pos))
        if sizes is None:
            sizes = mine
        elif mine != sizes:
            return None                     # the kernel takes one set of sizes for all layers
        if att.w_qkv.dtype != torch.bfloat16 or ff.w_gate_up.dtype != torch.bfloat16:
            return None
    if sizes is None or type(model.final_norm) is not RMSNorm:
        return None
    if model.final_norm.eps != sizes[8] or sizes[8] != sizes[9] or sizes[0] != sizes[5]:
        return None
    if model.head.weight.dtype != torch.bfloat16 or model.embedding.table.dtype != torch.bfloat16:
        return None
    if len(cache.plan.groups) > 4:
        return None
    try:
        fused = FusedDecode(model, cache, runtime)
    except Exception:
        return None
    return fused if fused.supported(1, 1) else None
