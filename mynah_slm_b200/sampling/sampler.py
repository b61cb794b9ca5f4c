"""Sampling parameters and the per-sequence sampler state on the device.

Parameters, their meanings and their defaults are the reference's
(mynah-slm src/sampler.h:13-26, src/sampler.c:27-36: temperature 0.6, top-k
20, top-p 0.95 from the model's generation_config.json; temp <= 0 is greedy
and skips every other filter). Order: penalties, temperature, top-k, min-p,
top-p, draw (src/sampler.c:116-187).

Per-sequence state of fixed size, one row per slot: the splitmix64 generator
state (src/sampler.c:40-46) and the ring of the last `penalty_window`
accepted tokens (src/sampler.c:73-78). A slot's state is set when its
sequence starts. The reference has one sampler for its one sequence; here
sequence number i of a call gets its own stream, derived from (seed, i), so
that what a sequence samples does not depend on which other sequences share
its batch. Stream 0 is the reference's own (seed 0 selects the constant of
src/sampler.c:55).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..ops import kernels

MASK64 = (1 << 64) - 1
SEED_ZERO = 0x853C49E6748FEA9B
_STREAM_STEP = 0xD1342543DE82EF95       # odd; separates the streams of one seed


@dataclass(frozen=True)
class SamplingParams:
    temp: float = 0.6
    top_k: int = 20
    top_p: float = 0.95
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    freq_penalty: float = 0.0
    presence_penalty: float = 0.0
    penalty_window: int = 64
    seed: int = 0

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls(temp=0.0)

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0 (0 = off), got {self.top_k}")
        if not 0.0 <= self.top_p:
            raise ValueError(f"top_p must be >= 0 (1.0 = off), got {self.top_p}")
        if self.min_p < 0.0:
            raise ValueError(f"min_p must be >= 0 (0 = off), got {self.min_p}")
        if self.penalty_window < 0:
            raise ValueError(f"penalty_window must be >= 0, got {self.penalty_window}")
        if self.repeat_penalty <= 0.0:
            raise ValueError(f"repeat_penalty must be > 0 (1.0 = off), got {self.repeat_penalty}")

    @property
    def has_penalties(self) -> bool:
        return self.penalty_window > 0 and not (self.repeat_penalty == 1.0 and self.freq_penalty == 0.0
                                                and self.presence_penalty == 0.0)


def stream_state(seed: int, index: int) -> int:
    """Initial splitmix64 state of sequence `index` under `seed`."""
    base = seed if seed else SEED_ZERO
    return (base + index * _STREAM_STEP) & MASK64


def _as_i64(u: int) -> int:
    return u - (1 << 64) if u >= (1 << 63) else u


class SamplerState:
    """Generator states and penalty rings of all slots, and the launches."""

    MAX_WINDOW = 256

    def __init__(self, max_seqs: int, device, window: int = 64):
        if not 0 <= window <= self.MAX_WINDOW:
            raise ValueError(f"penalty_window must lie in [0, {self.MAX_WINDOW}], got {window}")
        self.device = device
        self.window = window
        self.rng = torch.zeros((max_seqs,), dtype=torch.int64, device=device)
        self.ring = torch.zeros((max_seqs, max(window, 1)), dtype=torch.int32, device=device)
        self.ring_n = torch.zeros((max_seqs,), dtype=torch.int32, device=device)
        self.ring_head = torch.zeros((max_seqs,), dtype=torch.int32, device=device)
        self.params = torch.zeros((8,), dtype=torch.float32, device=device)
        self.active_window = window
        self._params_host: Optional[SamplingParams] = None
        self._to_reset: list[int] = []               # slots whose rows are set back at the next flush

    def set_params(self, p: SamplingParams) -> None:
        p.validate()
        if p.penalty_window > self.window and p.has_penalties:
            raise ValueError(f"penalty_window {p.penalty_window} exceeds the {self.window} this engine was built with")
        self.active_window = min(p.penalty_window, self.window)
        if p == self._params_host:
            return
        self.params.copy_(torch.tensor([p.temp, p.top_p, p.min_p, float(p.top_k), p.repeat_penalty,
                                        p.freq_penalty, p.presence_penalty, float(min(p.penalty_window, self.window))],
                                       dtype=torch.float32))
        self._params_host = p

    def reset_slot(self, slot: int) -> None:
        """The state a slot starts with: an empty ring and the generator of stream 0 of seed 0. A caller that
        wants another stream or the prompt in the ring calls `start_sequences` afterwards."""
        self._to_reset.append(int(slot))             # (one device operation for all of a batch's slots, not three a slot)

    def flush_resets(self) -> None:
        """Set the rows of the slots opened since the last call back; called before anything reads or writes
        the state (a draw, `start_sequences`, a captured step)."""
        if not self._to_reset:
            return
        idx = torch.tensor(self._to_reset, dtype=torch.int64).to(self.device)
        self._to_reset = []
        self.ring_n.index_fill_(0, idx, 0)
        self.ring_head.index_fill_(0, idx, 0)
        self.rng.index_fill_(0, idx, _as_i64(SEED_ZERO))

    def start_sequences(self, slots: Sequence[int], states: Sequence[int],
                        prompts: Optional[Sequence[Sequence[int]]] = None, window: Optional[int] = None) -> None:
        """Seed the slots' generators and load their rings with the prompts'
        last tokens (the reference accepts prompt tokens too, src/generate.c:25-32)."""
        self.flush_resets()
        idx = torch.tensor(list(slots), dtype=torch.int64, device=self.device)
        self.rng[idx] = torch.tensor([_as_i64(s) for s in states], dtype=torch.int64, device=self.device)
        w = self.active_window if window is None else min(window, self.window)
        rows = np.zeros((len(slots), self.ring.shape[1]), dtype=np.int32)
        ns, heads = [], []
        for i, _ in enumerate(slots):
            toks = prompts[i] if prompts is not None and w > 0 else []
            # the ring after accepting every prompt token in turn: token j lies at j % w
            n = min(len(toks), w)
            head = len(toks) % w if w > 0 else 0
            if n:
                first = len(toks) - n
                rows[i, (np.arange(first, first + n) % w)] = np.asarray(toks[first:], dtype=np.int32)
            ns.append(n)
            heads.append(head)
        self.ring[idx] = torch.from_numpy(rows).to(self.device)
        self.ring_n[idx] = torch.tensor(ns, dtype=torch.int32, device=self.device)
        self.ring_head[idx] = torch.tensor(heads, dtype=torch.int32, device=self.device)

    def sample(self, logits: torch.Tensor, slots: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Penalties, then the draw, then the accepted token into the ring.
        `logits` [B, V] fp32 is overwritten; `slots` int32 [B] (negative: padding)."""
        if not torch.cuda.is_current_stream_capturing():
            self.flush_resets()
        if self.window > 0:
            kernels.apply_penalties(logits, self.ring, self.ring_n, slots, self.params)
        out = kernels.sample(logits, self.params, self.rng, slots, out)
        if self.window > 0:
            kernels.sampler_accept(out, self.ring, self.ring_n, self.ring_head, slots, self.params)
        return out
