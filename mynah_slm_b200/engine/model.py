"""A model put together from a `ModelSpec`: embedding, layers, final norm,
head, and the schedule in which the layers run.

The model holds no sizes of its own; every part was built from the spec's
parameters. `cache_plan` reads what each run of the schedule asks of the
cache and sorts the runs into storage groups.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..cache.pages import GroupPlan
from ..config.keys import ConfigError
from ..config.spec import ModelSpec
from ..parts import build_part
from ..parts.base import Block, KVRequest, Part, StateRequest, TensorSpec


@dataclass
class EntryPlan:
    """Cache of one run of the schedule."""
    group: Optional[int] = None          # storage group of its keys/values
    index_in_group: Optional[int] = None
    state: Optional[StateRequest] = None
    source: Optional[int] = None         # schedule index whose cache it reads instead


@dataclass
class CachePlan:
    groups: list[GroupPlan] = field(default_factory=list)
    entries: list[EntryPlan] = field(default_factory=list)


class Model:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head, self.embedding)
        self.layers: list[Block] = []
        for ls in spec.layers:
            mixer = build_part("mixer", ls.mixer)
            ffn = build_part("ffn", ls.ffn)
            norms = {k: build_part("norm", v) for k, v in ls.norms.items()}
            self.layers.append(build_part("block", ls.block, mixer, ffn, norms))
        self.schedule = spec.schedule

    def parts(self) -> list[Part]:
        out: list[Part] = [self.embedding, self.final_norm, self.head]
        for block in self.layers:
            out.append(block)
            out.extend(block.parts())
        return out

    def tensor_specs(self) -> list[tuple[Part, TensorSpec]]:
        return [(p, ts) for p in self.parts() for ts in p.tensor_specs()]

    def cache_plan(self) -> CachePlan:
        plan = CachePlan()
        keys: dict[tuple, int] = {}
        for i, e in enumerate(self.schedule):
            mixer = self.layers[e.layer].mixer
            kv, st = mixer.kv_request(), mixer.state_request()
            if e.cache_from is not None:
                src = self.schedule[e.cache_from]
                src_kv = self.layers[src.layer].mixer.kv_request()
                if kv is None or src_kv != kv:
                    raise ConfigError(f"schedule[{i}] reads the cache of entry {e.cache_from}, "
                                      f"but asks for {kv} where that entry keeps {src_kv}")
                if st is not None:
                    raise ConfigError(f"schedule[{i}] has state of its own and cannot borrow a cache")
                plan.entries.append(EntryPlan(source=e.cache_from))
                continue
            ep = EntryPlan(state=st)
            if kv is not None:
                key = (kv.kv_heads, kv.head_dim, kv.window, kv.value_dim)
                if key not in keys:
                    keys[key] = len(plan.groups)
                    plan.groups.append(GroupPlan(kv.kv_heads, kv.head_dim, kv.window, v_head_dim=kv.value_dim))
                g = keys[key]
                ep.group, ep.index_in_group = g, len(plan.groups[g].entries)
                plan.groups[g].entries.append(i)
            plan.entries.append(ep)
        if not plan.groups:
            # the page lists double as the record of each sequence's length
            plan.groups.append(GroupPlan(0, 0, None, v_head_dim=0))
        return plan
