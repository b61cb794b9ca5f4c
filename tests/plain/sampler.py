"""Plain sampler and generation loop, written from the reference's formulas.

Citations are paths inside mynah-org/mynah-slm. Shares no code with the
product package.
"""
from __future__ import annotations

import numpy as np

MASK64 = (1 << 64) - 1
SEED_ZERO = 0x853C49E6748FEA9B      # src/sampler.c:55: seed 0 selects this constant


class SplitMix64:
    """src/sampler.c:40-46 (rng_next): state += golden; two xor-shift-multiply
    rounds; U = (z >> 11) / 2^53 in [0, 1)."""

    def __init__(self, state: int):
        self.state = state & MASK64

    def next_uniform(self) -> float:
        self.state = (self.state + 0x9E3779B97F4A7C15) & MASK64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        z = z ^ (z >> 31)
        return (z >> 11) * (1.0 / 9007199254740992.0)


class PlainSampler:
    """src/sampler.c:116-187 (mynah_slm_sample) with the penalties of :80-106
    and the ring of :73-78. Defaults of :27-36."""

    def __init__(self, temp=0.6, top_k=20, top_p=0.95, min_p=0.0, repeat_penalty=1.0,
                 freq_penalty=0.0, presence_penalty=0.0, penalty_window=64, seed=0,
                 rng_state: int | None = None):
        self.temp, self.top_k, self.top_p, self.min_p = float(temp), int(top_k), float(top_p), float(min_p)
        self.repeat_penalty = float(repeat_penalty)
        self.freq_penalty, self.presence_penalty = float(freq_penalty), float(presence_penalty)
        self.window = int(penalty_window)
        self.recent = [0] * self.window
        self.n_recent = 0
        self.head = 0
        self.rng = SplitMix64(rng_state if rng_state is not None else (seed if seed else SEED_ZERO))

    def accept(self, token: int) -> None:
        if self.window == 0:
            return
        self.recent[self.head] = int(token)
        self.head = (self.head + 1) % self.window
        if self.n_recent < self.window:
            self.n_recent += 1

    def apply_penalties(self, logits: np.ndarray) -> None:
        """In place. Walks the ring entry by entry, so a token that sits in the
        ring c times is penalised c times (src/sampler.c:86-105)."""
        if self.n_recent == 0:
            return
        if self.repeat_penalty == 1.0 and self.freq_penalty == 0.0 and self.presence_penalty == 0.0:
            return
        f32 = np.float32
        for i in range(self.n_recent):
            tok = self.recent[i]
            if tok >= len(logits):
                continue
            count = sum(1 for k in range(self.n_recent) if self.recent[k] == tok)
            l = f32(logits[tok])
            if self.repeat_penalty != 1.0:
                l = f32(l / f32(self.repeat_penalty)) if l > 0 else f32(l * f32(self.repeat_penalty))
            l = f32(l - f32(f32(self.freq_penalty) * f32(count)))
            l = f32(l - f32(self.presence_penalty))
            logits[tok] = l

    def sample(self, logits: np.ndarray) -> int:
        logits = np.asarray(logits, dtype=np.float32)
        self.apply_penalties(logits)
        V = len(logits)
        if self.temp <= 0.0:
            return int(np.argmax(logits))            # first maximum wins (:124-129)
        mx = logits.max()
        e = np.exp(((logits - mx) / np.float32(self.temp)).astype(np.float32)).astype(np.float32)  # :136
        inv = np.float32(1.0 / np.sum(e.astype(np.float64)))
        p = (e * inv).astype(np.float32)
        order = np.lexsort((np.arange(V), -p.astype(np.float64)))   # p desc, id asc (:108-114)
        ps = p[order]
        n = V
        if 0 < self.top_k < n:                       # :146-152
            n = self.top_k
        if self.min_p > 0.0 and n > 0:               # :156-161
            floor_p = np.float32(self.min_p) * ps[0]
            keep = 1
            while keep < n and ps[keep] >= floor_p:
                keep += 1
            n = keep
        if np.float32(self.top_p) < np.float32(1.0) and n > 0:   # :166-175
            acc, keep = 0.0, 0
            tp = float(np.float32(self.top_p))
            while keep < n:
                acc += float(ps[keep])
                keep += 1
                if acc >= tp:
                    break
            n = keep
        n = max(n, 1)
        total = float(np.sum(ps[:n].astype(np.float64)))
        r = self.rng.next_uniform() * total          # :178-186
        for i in range(n):
            r -= float(ps[i])
            if r <= 0.0:
                return int(order[i])
        return int(order[n - 1])


def plain_generate(model, prompt, max_new, sampler: PlainSampler, eos=()):
    """src/generate.c:13-86 without the text side: the prompt is accepted by
    the sampler token by token (:25-32); then forward, sample, accept, stop on
    any EOS id before it is emitted (:48-58). Recomputes the whole prefix each
    step, as tools/oracle/model.py:152-164 does. Returns (emitted ids, produced
    count, which includes the EOS that ended it)."""
    seq = [int(t) for t in prompt]
    for t in seq:
        sampler.accept(t)
    out, produced = [], 0
    for _ in range(max_new):
        logits = model.forward(seq)[-1].copy()
        tok = sampler.sample(logits)
        sampler.accept(tok)
        produced += 1
        if tok in eos:
            break
        out.append(tok)
        seq.append(tok)
    return out, produced
