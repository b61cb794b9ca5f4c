"""Device storage of the cache, built from a model's cache plan.

Per storage group: the keys of every entry of the group, each [n_pages,
kv_heads, 64, head_dim] in the run's type, in one allocation, and the values
likewise with their own width (a group whose mixers keep one vector per
position has none). Beside them: the fixed-size per-sequence state of the
entries that ask for one, [max_seqs + 1, *shape]: a sequence's row is zeroed
whenever its slot is handed out; the last row belongs to no sequence and is
there for a step's padding rows.

The page bookkeeping itself is on the host (`SequencePages`).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..parts.base import CacheView
from .pages import PAGE_TOKENS, CacheError, SequencePages


class Cache:
    def __init__(self, plan, n_pages: int, max_seqs: int, dtype: torch.dtype, device):
        self.plan = plan
        self.n_pages, self.max_seqs = n_pages, max_seqs
        self.pages = SequencePages(plan.groups, n_pages, max_seqs)
        self.keys: list[torch.Tensor] = []
        self.values: list[Optional[torch.Tensor]] = []
        for g in plan.groups:
            n = max(len(g.entries), 1)
            vd = g.head_dim if g.v_head_dim is None else g.v_head_dim
            self.keys.append(torch.empty((n, n_pages, g.kv_heads, PAGE_TOKENS, g.head_dim), dtype=dtype, device=device))
            self.values.append(torch.empty((n, n_pages, g.kv_heads, PAGE_TOKENS, vd), dtype=dtype, device=device) if vd else None)
        self.states: dict[int, torch.Tensor] = {}
        for i, e in enumerate(plan.entries):
            if e.state is not None:
                self.states[i] = torch.zeros((max_seqs + 1, *e.state.shape), dtype=e.state.dtype, device=device)
        self.views: list[CacheView] = []
        for i, e in enumerate(plan.entries):
            src = plan.entries[e.source] if e.source is not None else e
            k = v = None
            if src.group is not None:
                k = self.keys[src.group][src.index_in_group]
                v = self.values[src.group][src.index_in_group] if self.values[src.group] is not None else None
            self.views.append(CacheView(group=src.group if src.group is not None else 0, k=k, v=v,
                                        writes=e.source is None, state=self.states.get(i)))

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in [*self.keys, *self.values, *self.states.values()] if t is not None)

    def open(self) -> int:
        slot = self.pages.open()
        for t in self.states.values():
            t[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        self.pages.close(slot)
