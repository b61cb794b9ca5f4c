"""Arrangements of a layer's parts around the residual stream.

`prenorm_residual`: x = x + mixer(norm_mixer(x)); x = x + ffn(norm_ffn(x)),
the reference's block (mynah-slm docs/qwen3-arch.md:33-47,
src/arch_qwen3.c:201-234). It places two norms, named "mixer" and "ffn". Each
add is left pending on the stream, so the norm that follows does it in the
same pass.
"""
from __future__ import annotations

from ..config.keys import ConfigError
from .base import Block, CacheView, Residual, register_block


class PreNormResidual(Block):
    def __init__(self, spec, mixer, ffn, norms):
        super().__init__(spec, mixer, ffn, norms)
        for need in ("mixer", "ffn"):
            if need not in self.norms:
                raise ConfigError(f"prenorm_residual: the layer gives no {need!r} norm")

    def forward(self, stream: Residual, ctx, cache: CacheView) -> None:
        h = self.norms["mixer"].apply(stream, lazy=getattr(self.mixer, "accepts_normed", False))
        stream.add(self.mixer.forward(h, ctx, cache))
        h = self.norms["ffn"].apply(stream, lazy=getattr(self.ffn, "accepts_normed", False))
        stream.add(self.ffn.forward(h, ctx))


register_block("prenorm_residual", PreNormResidual)
