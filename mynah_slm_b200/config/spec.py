"""Architecture-neutral description of a model, built from a typed config.

An architecture turns its config into a `ModelSpec`; everything below the
registry (weights, parts, cache, engine) reads only the spec. A spec names a
part by `kind` (a key of the part registries in `parts/`) and carries that
part's sizes and constants as plain parameters, layer by layer, so different
layers of one model may use different mixers, feed-forwards, norms or position
encodings.

The order in which layers run is data as well: `schedule` is a list of
`ScheduleEntry`. An entry names the layer to run; the same layer may be named
more than once (each run then has a cache of its own), and an entry may read
the cache that an earlier entry wrote instead of keeping one.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by name with its parameters (sizes, eps, theta, ...)."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged (`block`), and the parts."""
    block: PartSpec                 # arrangement, e.g. pre-norm residual block
    mixer: PartSpec                 # token mixer, e.g. grouped-query attention
    ffn: PartSpec                   # feed-forward, dense or routed
    norms: Mapping[str, PartSpec]   # named norms the block places (e.g. "mixer", "ffn")
    prefix: str                     # tensor-name prefix of this layer's weights


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                          # index into ModelSpec.layers
    cache_from: Optional[int] = None    # schedule index whose cache this run reads, or None: its own


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    embedding: PartSpec             # token embedding (tensor name in params)
    final_norm: PartSpec
    head: PartSpec                  # output head; params["tied"] selects the embedding matrix
    eos_token_ids: tuple[int, ...] = ()
    sampling_defaults: Mapping[str, Any] = field(default_factory=dict)

    def validate(self) -> None:
        from .keys import ConfigError
        if not self.schedule:
            raise ConfigError("the schedule is empty")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule[{i}] names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ConfigError(f"schedule[{i}] reads the cache of entry {e.cache_from}, which does not run before it")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ConfigError(f"schedule[{i}] reads the cache of entry {e.cache_from}, which keeps none of its own")
