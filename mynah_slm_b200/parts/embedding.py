"""Token embedding and output head.

Embedding: x = E[token], no scaling by sqrt(hidden) (mynah-slm
src/arch_qwen3.c:186). Head: logits = Head . h in fp32, where Head is the
embedding matrix when the configuration ties them and `lm_head.weight`
otherwise; the configuration decides, not the presence of the tensor
(docs/qwen3-arch.md:91-113: the official checkpoint ships a duplicate
`lm_head.weight` although it is tied).
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..ops import kernels
from .base import Embedding, Head, TensorSpec, register_embedding, register_head


class TokenEmbedding(Embedding):
    def __init__(self, spec):
        super().__init__(spec)
        self.name = str(spec["name"])
        self.V, self.D = int(spec["vocab_size"]), int(spec["dim"])
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.V, self.D))]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.table = tensors[self.name]

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return kernels.embed_gather(self.table, tokens)


class LinearHead(Head):
    def __init__(self, spec, embedding):
        super().__init__(spec)
        self.tied = bool(spec["tied"])
        self.name = str(spec["name"])
        self.V, self.D = int(spec["vocab_size"]), int(spec["dim"])
        self.embedding = embedding
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        # tied: a stored copy is tolerated and left unread
        return [TensorSpec(self.name, (self.V, self.D), ignorable=self.tied)]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        if self.tied and getattr(self.embedding, "table", None) is None:
            from ..config.keys import ConfigError
            raise ConfigError("linear_head: a tied head needs an embedding part that keeps its matrix as `table`")
        self.weight = self.embedding.table if self.tied else tensors[self.name]

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return kernels.linear(h, self.weight, out_dtype=torch.float32)


register_embedding("token_embedding", TokenEmbedding)
register_head("linear_head", LinearHead)
