"""The description of one step's batch, on the host and on the device.

A step brings, for each of B sequences, its next tokens (one or more). The
tokens of all sequences are packed into T rows. Everything the kernels need to
know about the batch is a handful of int32 arrays, laid out in ONE buffer so
that a step costs one host-to-device copy:

  tokens  [T]    token ids
  tok_seq [T]    index of the row's sequence in this step, -1 for a padding row
  tok_pos [T]    absolute position of the row's token in its sequence
  cu_q    [B+1]  first row of each sequence
  kv_len  [B]    the sequence's length once this step is done (0: padding)
  slots   [B]    the sequence's slot (its row in per-sequence tables), -1: padding
  want    [W]    rows whose logits are wanted
  per storage group: indptr [B+1], base [B], ids [n_ids]   (the page lists)

`StepLayout` fixes the offsets for given capacities; `StepContext` is the set
of device views that parts and kernels read.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from ..ops.kernels import PageTableView


def _pad4(n: int) -> int:
    return (n + 3) & ~3


@dataclass
class StepLayout:
    T: int
    B: int
    W: int
    ids_cap: list[int]          # capacity of each group's page-id list

    def __post_init__(self):
        off = 0
        self.off = {}
        for name, n in (("tokens", self.T), ("tok_seq", self.T), ("tok_pos", self.T), ("cu_q", self.B + 1),
                        ("kv_len", self.B), ("slots", self.B), ("want", self.W)):
            self.off[name] = (off, n)
            off += _pad4(max(n, 1))
        for g, cap in enumerate(self.ids_cap):
            for name, n in ((f"indptr{g}", self.B + 1), (f"base{g}", self.B), (f"ids{g}", cap)):
                self.off[name] = (off, n)
                off += _pad4(max(n, 1))
        self.size = off
        # the same offsets as arrays, for the native packing routine (cache/pages.py: fill_step)
        names = ["tokens", "tok_seq", "tok_pos", "cu_q", "kv_len", "slots", "want"]
        for g in range(len(self.ids_cap)):
            names += [f"indptr{g}", f"base{g}", f"ids{g}"]
        self.offsets_array = np.array([self.off[n][0] for n in names], dtype=np.int32)
        self.ids_cap_array = np.array(list(self.ids_cap) or [0], dtype=np.int32)

    def view(self, buf, name: str):
        o, n = self.off[name]
        return buf[o:o + n]


@dataclass
class StepContext:
    T: int
    B: int
    tokens: torch.Tensor
    tok_seq: torch.Tensor
    tok_pos: torch.Tensor
    cu_q: torch.Tensor
    kv_len: torch.Tensor
    slots: torch.Tensor
    want: torch.Tensor
    pages: list[PageTableView]
    max_q_len: int
    is_decode: bool             # every sequence brings one token and row b is sequence b
    decode_splits: int
    status: torch.Tensor
    act_dtype: torch.dtype
    # host-side copies for parts that plan on the host (toy parts, tests)
    host_q_lens: Optional[list[int]] = None
    host_past: Optional[list[int]] = None
    host_slots: Optional[list[int]] = None


def device_context(layout: StepLayout, dev_buf: torch.Tensor, n_pages: list[int], max_q_len: int, is_decode: bool,
                   decode_splits: int, status: torch.Tensor, act_dtype: torch.dtype) -> StepContext:
    v = lambda name: layout.view(dev_buf, name)
    pages = [PageTableView(v(f"indptr{g}"), v(f"ids{g}"), v(f"base{g}"), n_pages[g]) for g in range(len(layout.ids_cap))]
    return StepContext(T=layout.T, B=layout.B, tokens=v("tokens"), tok_seq=v("tok_seq"), tok_pos=v("tok_pos"),
                       cu_q=v("cu_q"), kv_len=v("kv_len"), slots=v("slots"), want=v("want"), pages=pages,
                       max_q_len=max_q_len, is_decode=is_decode, decode_splits=decode_splits, status=status,
                       act_dtype=act_dtype)
