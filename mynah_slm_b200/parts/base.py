"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a `PartSpec` (its kind and its sizes and constants) and
knows nothing of the model it sits in. Seven families:

  mixer       mixes information along the sequence (attention here); may ask
              for key/value storage and for fixed-size per-sequence state
  feed-forward  works on each token alone (dense here; could be routed)
  norm        normalises the residual stream into a part's input
  position    position encoding that a mixer applies to its queries and keys
  block       the arrangement of norms, mixer and feed-forward around the
              residual stream
  embedding   token ids -> the first residual stream (fp32 rows)
  head        normalised rows -> fp32 logits; is handed the model's embedding
              part, whose matrix it may share

Each family has a registry from `kind` to a class; `register_*` adds to it,
from inside this package or from outside. The engine only ever talks to
these interfaces.

Interface common to all parts:
  tensor_specs() -> list[TensorSpec]   the tensors it reads from the checkpoint
  bind(tensors, runtime)               receives them on the device; may fuse
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping, Optional, Sequence

import torch

from ..config.spec import PartSpec


# ----------------------------------------------------------------- tensors

@dataclass(frozen=True)
class TensorSpec:
    """A checkpoint tensor a part binds by name.

    role decides the type it is kept in on the device:
      "matrix"  operand of a matrix product: the run's compute type
      "gain"    vector applied in fp32 arithmetic: fp32 stays fp32; otherwise
                bf16 in a bf16 run and fp32 in a 32-bit run
      "table"   integer table: int32
    init decides how the random-weights writer fills it: "normal" is
    N(0, std), "gain" is 1 + N(0, std), "zeros" is all zero.
    """
    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    std: float = 0.02
    ignorable: bool = False      # tolerated in the checkpoint but never read (a stored copy of a tied matrix)


# ------------------------------------------------------------ cache requests

@dataclass(frozen=True)
class KVRequest:
    """What a mixer keeps per position: keys of kv_heads x head_dim and, unless
    `values` is False, values of kv_heads x v_head_dim (head_dim when None). A
    mixer that keeps one vector per position (a latent that serves as key and
    value) asks for values=False. window=None keeps every position; window=W
    keeps the last W. Runs that ask for the same thing share a storage group
    and its page lists."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None
    values: bool = True

    @property
    def value_dim(self) -> int:
        return 0 if not self.values else (self.head_dim if self.v_head_dim is None else self.v_head_dim)


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size state per sequence, zeroed when a sequence starts."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheView:
    """What one run of a layer sees of the cache.

    group: id of the storage group whose page lists apply (ctx.pages[group]).
    k: this entry's keys [n_pages, kv_heads, 64, head_dim], or None.
    v: its values [n_pages, kv_heads, 64, v_head_dim], or None (also when the
       mixer asked for no values).
    writes: False when this run reads the cache another run wrote.
    state: [max_seqs + 1, *shape] fixed-size state of this entry, or None. Row
       `slot` belongs to the sequence in that slot; the last row belongs to no
       sequence: rows of a step that are padding (slot -1) may read and write
       it, so that a part can index with `where(slots >= 0, slots, max_seqs)`
       on the device and run from a captured graph.
    """
    group: Optional[int] = None
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    writes: bool = True
    state: Optional[torch.Tensor] = None


# ------------------------------------------------------------------- parts

class Part:
    def __init__(self, spec: PartSpec):
        self.spec = spec

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime: "Any") -> None:
        """`tensors` holds exactly the tensors named by tensor_specs() that the
        checkpoint has, already on the device in their kept types."""

    def streamed_tensors(self) -> list:
        """The bound tensors that every step reads from end to end (the matrices of its products). The engine
        may ask the memory system for them ahead of the part's turn; a part that names none is simply not
        helped."""
        return []


class Norm(Part):
    def apply(self, stream: "Residual", rows: Optional[torch.Tensor] = None, lazy: bool = False):
        """Fold the stream's pending delta in and return the normalised rows
        (all of them, or those that `rows` selects) in the activation type.
        With `lazy` a norm may return an object that stands for its result
        (with `.shape` and `.materialize()`), for a consumer that can compute
        the norm on its way; a part says that it can take one with
        `accepts_normed = True`."""
        raise NotImplementedError


class PositionEncoding(Part):
    #: True when the mixer's fused kernel applies it from `fused_tables`
    fusable = False

    def prepare(self, runtime: "Any") -> None:
        pass

    def fused_tables(self) -> tuple[Optional[torch.Tensor], Optional[torch.Tensor], int]:
        """(cos, sin, rotary_dim) for the fused norm+rotation+store kernel."""
        return None, None, 0

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx: "Any") -> None:
        """Unfused form: encode positions into q and k in place."""
        raise NotImplementedError


class Mixer(Part):
    def kv_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, h: torch.Tensor, ctx: "Any", cache: CacheView) -> torch.Tensor:
        """h: [T, hidden] in the activation type -> [T, hidden] likewise."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx: "Any") -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens: int32 [T] -> the first residual stream, fp32 [T, hidden]."""
        raise NotImplementedError


class Head(Part):
    """Built as Head(spec, embedding): the model's embedding part comes along, for a head that shares its matrix."""

    def forward(self, h) -> torch.Tensor:
        """h: the final norm's rows (or its unrun handle, see Norm.apply) -> fp32 logits [rows, vocab]."""
        raise NotImplementedError


class Block(Part):
    """Arrangement of a layer's parts around the residual stream."""

    def __init__(self, spec: PartSpec, mixer: Mixer, ffn: FeedForward, norms: Mapping[str, Norm]):
        super().__init__(spec)
        self.mixer, self.ffn, self.norms = mixer, ffn, dict(norms)

    def parts(self) -> list[Part]:
        return [self.mixer, self.ffn, *self.norms.values()]

    def forward(self, stream: "Residual", ctx: "Any", cache: CacheView) -> None:
        raise NotImplementedError


class Residual:
    """The residual stream of a step: fp32 [T, hidden], plus at most one
    delta that has not been added yet. A norm that follows an add takes both
    and does the add on its way (one pass over the row instead of two)."""

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending: Optional[torch.Tensor] = None

    def add(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            self.flush()
        self.pending = delta

    def flush(self) -> torch.Tensor:
        if self.pending is not None:
            from ..ops import kernels
            kernels.residual_add(self.x, self.pending)
            self.pending = None
        return self.x


# -------------------------------------------------------------- registries

_REGISTRIES: dict[str, dict[str, Callable[..., Part]]] = {
    "mixer": {}, "ffn": {}, "norm": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


def _register(family: str, kind: str, cls: Callable[..., Part], replace: bool) -> None:
    reg = _REGISTRIES[family]
    if kind in reg and not replace:
        raise ValueError(f"{family} {kind!r} is already registered")
    reg[kind] = cls


def register_mixer(kind: str, cls, replace: bool = False) -> None:
    _register("mixer", kind, cls, replace)


def register_ffn(kind: str, cls, replace: bool = False) -> None:
    _register("ffn", kind, cls, replace)


def register_norm(kind: str, cls, replace: bool = False) -> None:
    _register("norm", kind, cls, replace)


def register_position(kind: str, cls, replace: bool = False) -> None:
    _register("position", kind, cls, replace)


def register_block(kind: str, cls, replace: bool = False) -> None:
    _register("block", kind, cls, replace)


def register_embedding(kind: str, cls, replace: bool = False) -> None:
    _register("embedding", kind, cls, replace)


def register_head(kind: str, cls, replace: bool = False) -> None:
    _register("head", kind, cls, replace)


def build_part(family: str, spec: PartSpec, *args, **kwargs) -> Part:
    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        from ..config.keys import ConfigError
        raise ConfigError(f"unknown {family} {spec.kind!r}; known: {', '.join(sorted(reg))}")
    return reg[spec.kind](spec, *args, **kwargs)


def known_parts(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])
