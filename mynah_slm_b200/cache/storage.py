"""Device storage of the cache, built from a model's cache plan.

Per storage group: keys and values of every entry of the group, each
[n_pages, kv_heads, 64, head_dim] in the run's type, in one allocation.
Beside them: the fixed-size per-sequence state of the entries that ask for
one, [max_seqs, *shape], zeroed whenever a slot is handed out.

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
        self.kv: list[torch.Tensor] = []
        for g in plan.groups:
            n = max(len(g.entries), 1)
            self.kv.append(torch.empty((n, 2, n_pages, g.kv_heads, PAGE_TOKENS, g.head_dim), dtype=dtype, device=device))
        self.states: dict[int, torch.Tensor] = {}
        for i, e in enumerate(plan.entries):
            if e.state is not None:
                self.states[i] = torch.zeros((max_seqs, *e.state.shape), dtype=e.state.dtype, device=device)
        self.views: list[CacheView] = []
        for i, e in enumerate(plan.entries):
            src = plan.entries[e.source] if e.source is not None else e
            k = v = None
            if src.group is not None:
                k = self.kv[src.group][src.index_in_group, 0]
                v = self.kv[src.group][src.index_in_group, 1]
            self.views.append(CacheView(group=src.group if src.group is not None else 0, k=k, v=v,
                                        writes=e.source is None, state=self.states.get(i)))

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + \
            sum(t.numel() * t.element_size() for t in self.states.values())

    def open(self) -> int:
        slot = self.pages.open()
        for t in self.states.values():
            t[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        self.pages.close(slot)
