"""The Python entry point: load a model folder, generate from token ids.

    from mynah_slm_b200 import LLM
    llm = LLM("path/to/folder", dtype="bfloat16", max_tokens=65536)
    out = llm.generate([[1, 2, 3], [4, 5]], max_new=32, temp=0.0)
    out[0].tokens

Option names and meanings are those of the reference's `run` command
(mynah-slm cli/main.c:335-356): max_new (-n), temp, top_k, top_p, min_p, seed,
repeat_penalty. Prompts are token ids: the text side (tokenizer, chat
template) is not part of this library.
"""
from __future__ import annotations

import os
import time
from typing import Callable, Optional, Sequence

import torch

from ..sampling.sampler import SamplingParams, stream_state
from .engine import Engine, StepEntry
from .generate import Request, Result, Timing, generate


class EngineBackend:
    """`generate`'s view of an engine: prompts in one step, then one sampled
    token per sequence per step, host token ids in and out."""

    def __init__(self, engine: Engine, params: SamplingParams):
        self.engine = engine
        self.params = params
        self.max_positions = engine.spec.max_positions
        engine.sampler.set_params(params)
        self._host_rows: list[torch.Tensor] = []
        self._turn = 0
        self._to_start: list[tuple] = []
        # steps fed from the device are replayed graphs; MYNAH_RUN_AHEAD=0 keeps the step-by-step loop
        self.runs_ahead = bool(engine.use_graphs and engine.graph_safe) and os.environ.get("MYNAH_RUN_AHEAD", "1") != "0"

    def free_tokens(self) -> int:
        return self.engine.free_tokens()

    def open(self, request_index: int, prompt: Sequence[int]) -> int:
        slot = self.engine.open_sequence()
        # the generators and rings of a batch's slots are set in one go, when the batch's prompts run
        self._to_start.append((slot, stream_state(self.params.seed, request_index), prompt))
        return slot

    def _start_opened(self) -> None:
        if self._to_start:
            slots, states, prompts = zip(*self._to_start)
            self._to_start = []
            self.engine.sampler.start_sequences(slots, states, prompts)

    def close(self, slot: int) -> None:
        self._to_start = [t for t in self._to_start if t[0] != slot]
        self.engine.close_sequence(slot)

    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> list[int]:
        eng = self.engine
        self._start_opened()
        logits = eng.step([StepEntry(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)])
        slots_t = torch.tensor(list(slots), dtype=torch.int32, device=eng.device)
        toks = eng.sampler.sample(logits, slots_t).cpu().tolist()
        eng.check_status()
        return toks

    def decode(self, slots: Sequence[int], tokens: Sequence[int]) -> list[int]:
        self._start_opened()
        out = self.engine.decode_sampled(slots, tokens)
        return out[:len(slots)].cpu().tolist()

    # A step that is not waited for: its tokens are copied to pinned host memory behind it on the stream, and an
    # event marks the copy's end, so that the next step can be launched (fed from this one's result on the device)
    # before the host reads them.
    def decode_launch(self, slots: Sequence[int], tokens: Optional[Sequence[int]] = None, feed=None) -> "_InFlight":
        n = len(slots)
        self._start_opened()
        out = self.engine.decode_sampled(slots, tokens, None if feed is None else (feed[0].device_tokens, feed[1]))
        if not self._host_rows or self._host_rows[0].numel() < n:
            self._host_rows = [torch.empty((max(n, 64),), dtype=torch.int32, pin_memory=True) for _ in range(3)]
        host = self._host_rows[self._turn % 3]               # (at most two steps are in flight)
        self._turn += 1
        host[:n].copy_(out[:n], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return _InFlight(out, host, done, n)

    def decode_collect(self, step: "_InFlight") -> list[int]:
        step.done.synchronize()
        return step.host[:step.n].tolist()


class _InFlight:
    __slots__ = ("device_tokens", "host", "done", "n")

    def __init__(self, device_tokens: torch.Tensor, host: torch.Tensor, done, n: int):
        self.device_tokens, self.host, self.done, self.n = device_tokens, host, done, n


class LLM:
    def __init__(self, model: str, dtype: str = "bfloat16", max_tokens: int = 65536, max_seqs: Optional[int] = None,
                 device: str = "cuda:0", use_graphs: bool = True):
        t0 = time.perf_counter()
        self.engine = Engine.from_folder(model, dtype=dtype, max_tokens=max_tokens, max_seqs=max_seqs,
                                         device=device, use_graphs=use_graphs)
        torch.cuda.synchronize()
        self.load_s = time.perf_counter() - t0
        self.last_timing: Optional[Timing] = None

    @classmethod
    def random(cls, config, seed: int = 0, dtype: str = "bfloat16", max_tokens: int = 65536,
               max_seqs: Optional[int] = None, device: str = "cuda:0", use_graphs: bool = True) -> "LLM":
        """A model with random weights made on the device from `config` (a typed configuration, a config.json
        dictionary or the path of one) and `seed`; no file is written or read."""
        t0 = time.perf_counter()
        self = cls.__new__(cls)
        self.engine = Engine.random(config, seed=seed, dtype=dtype, max_tokens=max_tokens, max_seqs=max_seqs,
                                    device=device, use_graphs=use_graphs)
        torch.cuda.synchronize()
        self.load_s = time.perf_counter() - t0
        self.last_timing = None
        return self

    @property
    def eos_token_ids(self) -> tuple[int, ...]:
        return self.engine.spec.eos_token_ids

    def generate(self, prompts: Sequence[Sequence[int]], max_new: int = 128, temp: float = 0.6, top_k: int = 20,
                 top_p: float = 0.95, min_p: float = 0.0, seed: int = 0, repeat_penalty: float = 1.0,
                 freq_penalty: float = 0.0, presence_penalty: float = 0.0, penalty_window: int = 64,
                 stop_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False, max_batch: int = 64,
                 callback: Optional[Callable[[int, int], int]] = None) -> list[Result]:
        """Generate for every prompt (a list of token ids each). `stop_ids`
        defaults to the model's stop set (config.json and generation_config.json);
        `ignore_eos` empties it. Results are in the order of the prompts."""
        params = SamplingParams(temp=temp, top_k=top_k, top_p=top_p, min_p=min_p, repeat_penalty=repeat_penalty,
                                freq_penalty=freq_penalty, presence_penalty=presence_penalty,
                                penalty_window=penalty_window, seed=seed)
        stop = () if ignore_eos else (self.eos_token_ids if stop_ids is None else tuple(stop_ids))
        backend = EngineBackend(self.engine, params)
        timing = Timing(load_s=self.load_s, device_name=torch.cuda.get_device_name(self.engine.device))
        reqs = [Request(list(p), max_new) for p in prompts]
        out = generate(backend, reqs, stop_ids=stop, max_batch=max_batch, callback=callback, timing=timing)
        self.last_timing = timing
        return out
