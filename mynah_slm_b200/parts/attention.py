"""Grouped-query softmax attention over the paged cache.

What the reference's block does between its two norms (mynah-slm
src/arch_qwen3.c:204-224): project q, k, v; norm q and k per head (optional
part `qk_norm`); encode positions into q and k (part `position`); write k and
v to the cache; attend causally, each query head to the kv head h // (H/KV);
project the heads back to the hidden size. No bias anywhere
(src/model.h:55-61 has no bias field).

Parameters (all from the spec): hidden_size, num_heads, num_kv_heads,
head_dim, qk_norm (a norm spec or None), position (a position spec), window
(None: all keys; W: the query's own position and the W-1 before it), prefix
(tensor-name prefix).

The three projections are kept as one fused matrix [(H + 2 KV) * HD, hidden]
so that a step is one product instead of three. A run that reads the cache
another run wrote brings only q.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config.keys import ConfigError
from ..config.spec import PartSpec
from ..ops import kernels
from .base import (CacheView, KVRequest, Mixer, TensorSpec, build_part, register_mixer)


class GQAttention(Mixer):
    accepts_normed = True        # its first product can compute the norm on its way

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.D = int(spec["hidden_size"])
        self.H = int(spec["num_heads"])
        self.KV = int(spec["num_kv_heads"])
        self.HD = int(spec["head_dim"])
        self.window: Optional[int] = spec.get("window")
        self.prefix = str(spec["prefix"])
        if self.H % self.KV:
            raise ConfigError(f"attention: {self.H} heads are not a multiple of {self.KV} kv heads")
        if self.HD % 8 or self.HD > kernels.MAX_HEAD_DIM:
            raise ConfigError(f"attention: head_dim {self.HD} must be a multiple of 8 and at most "
                              f"{kernels.MAX_HEAD_DIM} for the attention kernels")
        if self.window is not None and self.window < 1:
            raise ConfigError(f"attention: window {self.window} must be positive")
        qk = spec.get("qk_norm")
        self.qk_eps = float(qk["eps"]) if qk is not None else 0.0
        self.has_qk_norm = qk is not None
        if qk is not None and qk.kind != "rmsnorm":
            raise ConfigError(f"attention: per-head norm {qk.kind!r} is not supported (only 'rmsnorm')")
        self.position = build_part("position", spec["position"])
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = None

    # ------------------------------------------------------------ weights
    def tensor_specs(self) -> list[TensorSpec]:
        p, H, KV, HD, D = self.prefix, self.H, self.KV, self.HD, self.D
        specs = [
            TensorSpec(p + "q_proj.weight", (H * HD, D)),
            TensorSpec(p + "k_proj.weight", (KV * HD, D)),
            TensorSpec(p + "v_proj.weight", (KV * HD, D)),
            TensorSpec(p + "o_proj.weight", (D, H * HD)),
        ]
        if self.has_qk_norm:
            specs += [TensorSpec(p + "q_norm.weight", (HD,), role="gain", init="gain", std=0.1),
                      TensorSpec(p + "k_norm.weight", (HD,), role="gain", init="gain", std=0.1)]
        return specs + self.position.tensor_specs()

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        p = self.prefix
        self.w_qkv = torch.cat([tensors[p + "q_proj.weight"], tensors[p + "k_proj.weight"],
                                tensors[p + "v_proj.weight"]], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.H * self.HD]
        self.w_o = tensors[p + "o_proj.weight"]
        if self.has_qk_norm:
            self.q_gain, self.k_gain = tensors[p + "q_norm.weight"], tensors[p + "k_norm.weight"]
        self.position.bind(tensors, runtime)
        self.position.prepare(runtime)
        self.runtime = runtime

    def streamed_tensors(self) -> list:
        return [self.w_qkv, self.w_o]

    # -------------------------------------------------------------- cache
    def kv_request(self) -> KVRequest:
        return KVRequest(self.KV, self.HD, self.window)

    # ------------------------------------------------------------ forward
    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        H, KV, HD = self.H, self.KV, self.HD
        T = h.shape[0]
        writes = cache.writes
        pages = ctx.pages[cache.group]
        from ..ops import attention_dispatch, gemm_bf16
        w_in = self.w_qkv if writes else self.w_q
        if not ctx.is_decode and self.position.fusable and self.runtime.act_dtype == torch.bfloat16:
            cos, sin, rot = self.position.fused_tables()
            x_in = h.materialize() if isinstance(h, kernels.NormedInput) else h
            same_gains = self.q_gain is None or self.q_gain.dtype == self.k_gain.dtype
            if ((cos is None or rot == HD) and same_gains and gemm_bf16.qkv_rope_supported(x_in, w_in, H, KV, HD)
                    and kernels.attn_prefill_tcgen05_supported(x_in.dtype, H, KV, HD)):
                # a prompt step: norm, rotation and the cache write happen in the projection's epilogue
                q = gemm_bf16.gemm_qkv_rope(x_in, w_in, H, KV, HD, self.q_gain, self.k_gain, self.qk_eps, cos, sin,
                                            ctx.tok_seq, ctx.tok_pos, pages,
                                            cache.k if writes else None, cache.v if writes else None)
                out = torch.empty((T, H * HD), dtype=q.dtype, device=q.device)
                attention_dispatch.prefill(q, out, ctx, H, KV, HD, cache.k, cache.v, pages, self.window or 0)
                return kernels.linear(out, self.w_o)
            h = x_in
        qkv = kernels.linear(h, w_in)
        out = torch.empty((T, H * HD), dtype=qkv.dtype, device=qkv.device)
        if self.position.fusable:
            cos, sin, rot = self.position.fused_tables()
            if ctx.is_decode and attention_dispatch.decode_fused_ok(qkv.dtype, H, KV, HD, rot, cos,
                                                                    ctx.B, ctx.decode_splits):
                # norm, rotation, cache write and attention in one launch
                gains_dtype_ok = self.q_gain is None or self.q_gain.dtype == self.k_gain.dtype
                if gains_dtype_ok:
                    kernels.attn_decode_fused(
                        qkv, out, ctx.B, H, KV, HD, self.q_gain, self.k_gain, self.qk_eps, cos, sin, ctx.tok_pos,
                        cache.k, cache.v, writes, ctx.kv_len, pages, self.window or 0, ctx.decode_splits,
                        self.runtime.attn_scratch(ctx.B, H, HD, ctx.decode_splits),
                        self.runtime.attn_counters(ctx.B * KV)
                        if attention_dispatch.decode_fused_merges(ctx.B, KV, ctx.decode_splits) else None, ctx.status)
                    return kernels.linear(out, self.w_o)
        else:
            q_view = qkv[:, : H * HD].view(T, H, HD)
            k_view = qkv[:, H * HD: (H + KV) * HD].view(T, KV, HD) if writes else None
            self.position.apply(q_view, k_view, ctx)
            cos = sin = None
            rot = 0
        kernels.qk_norm_rope_store(
            qkv, H, KV, HD, self.q_gain, self.k_gain, self.qk_eps, cos, sin, rot,
            ctx.tok_seq, ctx.tok_pos, pages,
            cache.k if writes else None, cache.v if writes else None, ctx.status)
        if ctx.is_decode:
            attention_dispatch.decode(qkv, out, ctx, H, KV, HD, cache.k, cache.v, pages, self.window or 0,
                                      self.runtime.attn_scratch(ctx.B, H, HD, ctx.decode_splits),
                                      self.runtime.attn_counters(ctx.B * KV))
        else:
            attention_dispatch.prefill(qkv, out, ctx, H, KV, HD, cache.k, cache.v, pages, self.window or 0)
        return kernels.linear(out, self.w_o)


register_mixer("gqa_attention", GQAttention)
