"""The generation loop above the step function.

The reference generates one sequence (mynah-slm src/generate.c:13-86):
prompt, then forward / sample / stop-check / emit until a stop token, the
token limit or a full context. Its rules are kept per sequence:

  * a stop token ends the sequence BEFORE it is emitted; it still counts as
    produced (src/generate.c:53-55);
  * any id of the stop set stops (src/generate.c:8-11);
  * `max_new` bounds the produced tokens (:47); a full context ends the
    sequence (:48 with src/arch_qwen3.c:182);
  * a callback that returns non-zero ends the sequence (:75).

What is added is the batch: requests are taken in order, as many at a time
as the batch size and the cache allow; the prompts of a batch (of unequal
lengths) run in one step, then every live sequence goes on by one token per
step; a sequence that ends leaves the batch and gives its slot and pages
back at once, while the others go on; when a batch is done the next requests
start, in the slots and pages that were freed.

The decisions are made on the host against a small `Backend` interface, so
they can be tested without a device.

A backend that can launch a step without waiting for it (`runs_ahead`, with
`decode_launch` and `decode_collect`) is driven one step ahead: while the device runs step n + 1,
whose input tokens it takes from step n's result on the device, the host reads
step n's tokens and decides. A sequence that step n ends with a stop token or
through the callback has then run one row too many; the row is dropped, and
the sequence gives its slot and pages back one step later. Sequences that must
end with step n whatever it samples (token limit, full context) are not
launched again. The results are those of the step-by-step loop.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Protocol, Sequence

from ..cache.pages import PAGE_TOKENS


@dataclass
class Request:
    tokens: Sequence[int]
    max_new: int = 128


@dataclass
class Result:
    tokens: list[int] = field(default_factory=list)   # emitted ids (a stop token is not among them)
    produced: int = 0                                  # sampled ids, the stop token included
    finish_reason: str = ""                            # "stop" | "length" | "context" | "callback"


@dataclass
class Timing:
    """Load, prefill and decode time kept apart, and the time to the first
    token measured rather than derived (mynah-slm src/timing.h:15-28,
    src/timing.c:27-62)."""
    load_s: float = 0.0
    prefill_s: float = 0.0
    decode_s: float = 0.0
    ttft_s: float = 0.0
    n_prompt: int = 0
    n_gen: int = 0
    device_name: str = ""

    def prefill_tok_s(self) -> float:
        return self.n_prompt / self.prefill_s if self.prefill_s > 0 else 0.0

    def decode_tok_s(self) -> float:
        return self.n_gen / self.decode_s if self.decode_s > 0 else 0.0

    def format(self) -> str:
        return (f"[load {self.load_s:.2f}s | prompt {self.n_prompt} tok, prefill {self.prefill_tok_s():.1f} tok/s | "
                f"gen {self.n_gen} tok, decode {self.decode_tok_s():.1f} tok/s | TTFT {self.ttft_s * 1000.0:.0f} ms | "
                f"{self.device_name or 'gpu'}]")


class Backend(Protocol):
    max_positions: int

    def free_tokens(self) -> int: ...
    def open(self, request_index: int, prompt: Sequence[int]) -> int: ...
    def close(self, slot: int) -> None: ...
    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> list[int]: ...
    def decode(self, slots: Sequence[int], tokens: Sequence[int]) -> list[int]: ...
    # Optional, with `runs_ahead = True`:
    #   decode_launch(slots, tokens=None, feed=None) -> handle   starts a step and returns at once; the input
    #       tokens are `tokens` (host ids) or, with feed = (handle of the step before, rows), row rows[i] of that
    #       step's result, taken on the device;
    #   decode_collect(handle) -> list[int]                      waits for that step and returns its tokens.


class GenerationError(RuntimeError):
    pass


def tokens_held(prompt_len: int, max_new: int, max_positions: int) -> int:
    """Cache a request may come to hold: its positions rounded up to whole pages."""
    n = min(prompt_len + max(max_new, 0), max_positions)
    return -(-n // PAGE_TOKENS) * PAGE_TOKENS


def plan_batches(requests: Sequence[Request], max_batch: int, budget_tokens: int, max_positions: int) -> list[list[int]]:
    """Split the requests, in order, into batches that fit the batch size and
    the cache. Requests with nothing to generate are not scheduled."""
    if max_batch < 1:
        raise GenerationError(f"max_batch must be at least 1, got {max_batch}")
    batches: list[list[int]] = []
    cur: list[int] = []
    used = 0
    for i, r in enumerate(requests):
        if len(r.tokens) == 0:
            raise GenerationError(f"request {i} has an empty prompt")
        if len(r.tokens) > max_positions:
            raise GenerationError(f"request {i}: a prompt of {len(r.tokens)} tokens exceeds the model's "
                                  f"{max_positions} positions")
        if r.max_new <= 0:
            continue
        need = tokens_held(len(r.tokens), r.max_new, max_positions)
        if need > budget_tokens:
            raise GenerationError(f"request {i} may hold {need} tokens of cache, the engine has {budget_tokens}")
        if cur and (len(cur) >= max_batch or used + need > budget_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


@dataclass
class _Live:
    index: int
    slot: int
    next_token: int = 0
    length: int = 0


def generate(backend: Backend, requests: Sequence[Request], stop_ids: Sequence[int] = (), max_batch: int = 64,
             callback: Optional[Callable[[int, int], int]] = None, timing: Optional[Timing] = None,
             budget_tokens: Optional[int] = None) -> list[Result]:
    """Run every request to its end; results come back in request order."""
    stop = set(int(s) for s in stop_ids)
    results = [Result() for _ in requests]
    for i, r in enumerate(requests):
        if r.max_new <= 0:
            results[i].finish_reason = "length"
    budget = backend.free_tokens() if budget_tokens is None else budget_tokens
    t_start = time.perf_counter()

    def accept(live: _Live, tok: int) -> bool:
        """One sampled token of a live sequence. Returns True if it goes on."""
        res, req = results[live.index], requests[live.index]
        res.produced += 1
        if timing is not None:
            if timing.n_gen == 0:
                timing.ttft_s = time.perf_counter() - t_start
            timing.n_gen += 1
        if tok in stop:
            res.finish_reason = "stop"
            return False
        res.tokens.append(tok)
        if callback is not None and callback(live.index, tok):
            res.finish_reason = "callback"
            return False
        if res.produced >= req.max_new:
            res.finish_reason = "length"
            return False
        if live.length >= backend.max_positions:
            res.finish_reason = "context"       # no position left for the next input
            return False
        live.next_token = tok
        return True

    for batch in plan_batches(requests, max_batch, budget, backend.max_positions):
        live = [_Live(i, backend.open(i, requests[i].tokens)) for i in batch]
        try:
            t0 = time.perf_counter()
            prompts = [requests[l.index].tokens for l in live]
            first = backend.prefill([l.slot for l in live], prompts)
            if timing is not None:
                timing.prefill_s += time.perf_counter() - t0
                timing.n_prompt += sum(len(p) for p in prompts)
            t0 = time.perf_counter()
            for l, p in zip(live, prompts):
                l.length = len(p)
            going = []
            for l, tok in zip(live, first):
                if accept(l, int(tok)):
                    going.append(l)
                else:
                    backend.close(l.slot)
            live = going
            if getattr(backend, "runs_ahead", False):
                # one step ahead: `rows` are the sequences of the step in flight, in its row order; `dead` those
                # among them that an earlier step has ended (their rows are dropped, their slots closed below)
                def certain_end(l: _Live) -> bool:          # its next token ends it whatever it is
                    return (results[l.index].produced + 1 >= requests[l.index].max_new
                            or l.length + 1 >= backend.max_positions)
                rows = list(live)
                dead: set[int] = set()
                handle = backend.decode_launch([l.slot for l in rows], tokens=[l.next_token for l in rows]) if rows else None
                while handle is not None:
                    ahead = [(j, l) for j, l in enumerate(rows) if l.index not in dead and not certain_end(l)]
                    nxt = None
                    if ahead:
                        nxt = backend.decode_launch([l.slot for _, l in ahead], feed=(handle, [j for j, _ in ahead]))
                    toks = backend.decode_collect(handle)
                    for l, tok in zip(rows, toks):
                        if l.index in dead:                 # ended a step ago: this row was one too many
                            dead.discard(l.index)
                            live.remove(l)
                            backend.close(l.slot)
                            continue
                        l.length += 1
                        if not accept(l, int(tok)):
                            if nxt is not None and any(a is l for _, a in ahead):
                                dead.add(l.index)           # it is in the step in flight: close when that is done
                            else:
                                live.remove(l)
                                backend.close(l.slot)
                    rows = [l for _, l in ahead]
                    handle = nxt
            while live:
                toks = backend.decode([l.slot for l in live], [l.next_token for l in live])
                going = []
                for l, tok in zip(live, toks):
                    l.length += 1
                    if accept(l, int(tok)):
                        going.append(l)
                    else:
                        backend.close(l.slot)
                live = going
            if timing is not None:
                timing.decode_s += time.perf_counter() - t0
        except BaseException:
            for l in live:
                try:
                    backend.close(l.slot)
                except Exception:
                    pass
            raise
    return results
