"""The engine: a model on the device, its cache, and the ONE step function.

`Engine.step` takes a batch of sequences that either all bring the first
tokens of their prompts (or a further piece of them) or all go on by one
token. It runs exactly the tokens it is given, as one batch, against what
earlier steps left in the cache, and returns fp32 logits at the wanted
places. It replaces the reference's `mynah_slm_forward(state, token, logits)`
(mynah-slm src/arch_qwen3.c:178-252), which takes one token of one sequence;
a loop of single-token steps here gives the same logits as one step over the
whole prompt.

A step that brings one token per sequence is replayed from a CUDA graph
(captured per batch-size bucket; unused rows of a bucket are padding rows
that read and write nothing), so a decode step costs one copy of the batch
description and one graph launch. With `sample=True` the graph also samples
and feeds each sequence's token back as its next input, so that many steps
can run without the host in between.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache.pages import PAGE_TOKENS, CacheError
from ..cache.storage import Cache
from ..config.spec import ModelSpec
from ..ops import kernels
from ..ops.lib import KernelError
from ..parts.base import Residual
from ..registry import read_config_folder
from ..sampling.sampler import SamplerState, SamplingParams
from ..weights.loader import load_into
from ..weights.safetensors_io import Checkpoint
from .context import StepContext, StepLayout, device_context
from .model import Model

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class EngineError(RuntimeError):
    pass


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()        # places among `tokens` whose logits are wanted


class Runtime:
    """Device-wide things that parts share: the compute type, lookup tables
    built once, scratch memory, and the status word kernels report through."""

    def __init__(self, device, act_dtype: torch.dtype, max_positions: int):
        self.device = device
        self.act_dtype = act_dtype
        self.max_positions = max_positions
        self.tables: dict = {}
        self.status = torch.zeros((1,), dtype=torch.int32, device=device)
        self._scratch: Optional[torch.Tensor] = None
        self._counters: Optional[torch.Tensor] = None
        # Buffers that were outgrown stay alive: a captured graph may still hold their address.
        self._retired: list[torch.Tensor] = []
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count

    def _no_capture(self, what: str) -> None:
        if torch.cuda.is_current_stream_capturing():
            raise EngineError(f"{what} would have to grow during graph capture")

    def attn_scratch(self, B: int, H: int, HD: int, splits: int) -> torch.Tensor:
        need = B * H * splits * (HD + 2)
        if self._scratch is None or self._scratch.numel() < need:
            self._no_capture("attention scratch")
            if self._scratch is not None:
                self._retired.append(self._scratch)
            self._scratch = torch.empty((need,), dtype=torch.float32, device=self.device)
        return self._scratch

    def attn_counters(self, n: int) -> torch.Tensor:
        """Zeroed words that the fused decode attention counts finished pages in (it leaves them zero)."""
        if self._counters is None or self._counters.numel() < n:
            self._no_capture("attention counters")
            if self._counters is not None:
                self._retired.append(self._counters)
            self._counters = torch.zeros((max(n, 1024),), dtype=torch.int32, device=self.device)
        return self._counters


class _Ahead:
    """A second stream beside the step's own, on which the memory system is asked for the weights of the layer
    after the running one (`kernels.l2_prefetch`). Inside a graph capture the events become edges of the graph:
    the request for layer i+1 may start when layer i starts, and the step ends only when every request has."""

    def __init__(self, device):
        self.side = torch.cuda.Stream(device=device)
        self.used = False

    def issue(self, tensors) -> None:
        if not tensors:
            return
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        self.side.wait_event(ev)
        with torch.cuda.stream(self.side):
            kernels.l2_prefetch(tensors)
        self.used = True

    def join(self) -> None:
        if self.used:
            ev = torch.cuda.Event()
            ev.record(self.side)
            torch.cuda.current_stream().wait_event(ev)
            self.used = False


class _Staging:
    """A few pinned buffers used in turn for the batch description, so that
    the host can write the next one while an earlier copy is still in flight."""

    def __init__(self, n: int = 4):
        self.bufs: list[Optional[torch.Tensor]] = [None] * n
        self.events = [torch.cuda.Event() for _ in range(n)]
        self.used = [False] * n
        self.i = 0

    def get(self, size: int) -> tuple[torch.Tensor, int]:
        i = self.i
        self.i = (self.i + 1) % len(self.bufs)
        if self.used[i]:
            self.events[i].synchronize()
        b = self.bufs[i]
        if b is None or b.numel() < size:
            b = torch.empty((max(size, 1024),), dtype=torch.int32, pin_memory=True)
            self.bufs[i] = b
        return b, i

    def sent(self, i: int) -> None:
        self.events[i].record()
        self.used[i] = True


@dataclass
class _DecodeGraph:
    bucket: int
    layout: StepLayout
    meta: torch.Tensor                 # static device copy of the batch description
    ctx: StepContext
    splits: int
    graphs: dict = field(default_factory=dict)     # mode -> (CUDAGraph, output tensor, kernels per replay)


@dataclass
class _PromptGraph:
    """A captured prompt step for one padded shape: rows, sequences, wanted rows, page-list capacity."""
    layout: StepLayout
    meta: torch.Tensor                 # static device copy of the batch description
    ctx: StepContext
    graph: object = None               # torch.cuda.CUDAGraph once captured
    logits: Optional[torch.Tensor] = None
    n_kernels: int = 0
    last_use: int = 0


# Granularity of the page splits of captured decode steps beyond this many pages (0: powers of two throughout).
# Measured at 33 pages a sequence: splits of 64 / 48 / 40 give 1.371 / 1.364 / 1.355 ms a step at batch 8 and
# 3.97 / 3.88 / 3.84 at batch 64; every new size is a capture (a step run twice), so not finer than 16.
PAGE_BUCKET_STEP = int(os.environ.get("MYNAH_PAGE_BUCKET_STEP", "16"))
# Captured decode steps of at most this many rows ask for the next layer's weights ahead of time (0: never).
# Measured at the 0.6B shape: one row 0.988 -> 0.969 ms a step; eight rows 1.355 -> 1.569 ms (the second stream's
# edges into the chain cost more than the L2 hits save, and the attention's pages push the weights out again).
L2_PREFETCH_MAX_ROWS = int(os.environ.get("MYNAH_L2_PREFETCH_MAX_ROWS", "2"))
# MYNAH_PDL_PROMPT=1: prompt steps are captured with programmatic dependent launch, so that a kernel's set-up (barriers,
# tensor memory, its first descriptor fetches) runs while the kernel before it drains. Measured on a 2,048-token
# prompt: 0.6B shape 3.983 -> 3.935 ms, 4B shape 16.14 -> 16.36 ms: within noise, so it is off.
PDL_PROMPT = os.environ.get("MYNAH_PDL_PROMPT", "0") != "0"
# Decode steps of at most this many rows are captured with programmatic dependent launch (0: none).
PDL_MAX_ROWS = int(os.environ.get("MYNAH_PDL_MAX_ROWS", "2"))


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


# Prompt steps of more rows than this are never captured: their kernels run for so long that the launches hide
# behind them (a 12,800-row step of the 4B shape: 85 ms on the device, about 2 ms of launches), while a captured step
# keeps its activations' memory for as long as the graph lives and costs a second run to record.
PROMPT_GRAPH_MAX_ROWS = int(os.environ.get("MYNAH_PROMPT_GRAPH_MAX_ROWS", "4096"))


def _prompt_rows_bucket(T: int) -> int:
    """Rows of a prompt step, padded so that a few graphs serve many lengths and at most an eighth is padding."""
    if T <= 256:
        return _round_up(T, 32)
    if T <= 1024:
        return _round_up(T, 128)
    return _round_up(T, 256)


class Engine:
    def __init__(self, spec: ModelSpec, checkpoint: Checkpoint, dtype="bfloat16", max_tokens: int = 4096,
                 max_seqs: Optional[int] = None, device="cuda:0", use_graphs: bool = True,
                 penalty_window: int = 64):
        if isinstance(dtype, str):
            if dtype not in DTYPES:
                raise EngineError(f"dtype {dtype!r} is not one of {sorted(DTYPES)}")
            dtype = DTYPES[dtype]
        if dtype not in (torch.bfloat16, torch.float32):
            raise EngineError(f"dtype {dtype} is not supported (bfloat16 or float32)")
        if not torch.cuda.is_available():
            raise EngineError("mynah_slm_b200 needs a CUDA device (B200, sm_100); there is no CPU fallback")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        from ..ops import lib
        lib.load()                                 # fails loudly when the kernels are missing
        self.spec = spec
        self.dtype = dtype
        self.model = Model(spec)
        self.runtime = Runtime(self.device, dtype, spec.max_positions)
        from ..weights.random_init import RandomWeights, fill_into
        if isinstance(checkpoint, RandomWeights):
            fill_into(self.model.tensor_specs(), checkpoint, self.runtime)
        else:
            load_into(self.model.tensor_specs(), checkpoint, self.runtime)
        self.n_pages = max(1, -(-int(max_tokens) // PAGE_TOKENS))
        self.max_seqs = int(max_seqs) if max_seqs else min(self.n_pages, 1024)
        self.cache = Cache(self.model.cache_plan(), self.n_pages, self.max_seqs, dtype, self.device)
        self.n_groups = len(self.cache.plan.groups)
        self.sampler = SamplerState(self.max_seqs, self.device, penalty_window)
        self.sampler.set_params(SamplingParams.greedy())
        self.use_graphs = use_graphs
        # a part that plans on the host (reads ctx.host_*) cannot be replayed from a graph
        self.graph_safe = all(getattr(p, "graph_safe", True) for p in self.model.parts())
        self._staging = _Staging()
        self._graphs: dict[tuple[int, int], _DecodeGraph] = {}
        # prompt steps: a shape is captured the second time it comes; a handful of graphs are kept
        self._prompt_graphs: dict[tuple, _PromptGraph] = {}
        self._prompt_seen: dict[tuple, int] = {}
        self._prompt_clock = 0
        self.max_prompt_graphs = 6
        self._ahead = _Ahead(self.device)
        self._prefetching = False                  # set while a captured decode step's launches are made
        self._layer_weights = [[t for p in self.model.layers[e.layer].parts() for t in p.streamed_tensors()]
                               for e in self.model.schedule]
        self.launches = 0                          # kernels of this package launched (see count_launches)
        self.vocab_size = spec.vocab_size

    # ------------------------------------------------------------ creation
    @classmethod
    def from_folder(cls, folder: str, **kw) -> "Engine":
        typed = read_config_folder(folder)
        ckpt = Checkpoint(folder)
        try:
            return cls(typed.model_spec(), ckpt, **kw)
        finally:
            ckpt.close()

    @classmethod
    def random(cls, config, seed: int = 0, dtype="bfloat16", stored_dtype=None, **kw) -> "Engine":
        """An engine with random weights made on the device: no file is written or read. `config` is a typed
        configuration, a config.json dictionary or the path of a config.json; the weights are those that
        `write_random_model(folder, config, seed, stored_dtype)` writes (stored_dtype: the run's type unless
        given)."""
        import json
        from ..registry import parse_config
        from ..weights.random_init import RandomWeights
        if isinstance(config, (str, os.PathLike)):
            with open(config) as f:
                config = json.load(f)
        typed = parse_config(config) if isinstance(config, dict) else config
        run = DTYPES[dtype] if isinstance(dtype, str) and dtype in DTYPES else dtype
        stored = run if stored_dtype is None else (DTYPES[stored_dtype] if isinstance(stored_dtype, str) else stored_dtype)
        return cls(typed.model_spec(), RandomWeights(seed, stored), dtype=dtype, **kw)

    # ----------------------------------------------------------- sequences
    def open_sequence(self) -> int:
        """A free slot for a new sequence. Whatever the slot's last sequence left is gone: its pages were given
        back when it closed, fixed-size state is zeroed, and the sampler's row (ring of recent tokens, generator)
        starts empty."""
        slot = self.cache.open()
        self.sampler.reset_slot(slot)
        return slot

    def close_sequence(self, slot: int) -> None:
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.pages.length[slot]

    def free_tokens(self) -> int:
        return min(p.n_free for p in self.cache.pages.pools) * PAGE_TOKENS

    # ------------------------------------------------------------- helpers
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise EngineError("a step needs at least one sequence")
        seen = set()
        V = self.spec.vocab_size
        for e in entries:
            if e.slot in seen:
                raise EngineError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if e.slot not in self.cache.pages.length:
                raise EngineError(f"slot {e.slot} is not open")
            n = len(e.tokens)
            if n < 1:
                raise EngineError(f"slot {e.slot} brings no tokens")
            toks = np.asarray(e.tokens)
            if toks.dtype.kind not in "iu":
                raise EngineError(f"the tokens of slot {e.slot} are not integers")
            if int(toks.min()) < 0 or int(toks.max()) >= V:
                bad = int(toks.min()) if int(toks.min()) < 0 else int(toks.max())
                raise EngineError(f"token id {bad} lies outside the vocabulary of {V}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise EngineError(f"wanted place {w} lies outside the {n} tokens of slot {e.slot}")
            if self.cache.pages.length[e.slot] + n > self.spec.max_positions:
                raise EngineError(f"slot {e.slot} would grow to {self.cache.pages.length[e.slot] + n} positions, "
                                  f"the model allows {self.spec.max_positions}")

    @staticmethod
    def _decode_pages(max_kv: int) -> int:
        """Page splits of a decode launch: one per page the longest sequence can see."""
        return max(1, -(-max_kv // PAGE_TOKENS))

    def _fill(self, buf_np: np.ndarray, layout: StepLayout, entries: Sequence[StepEntry], with_want: bool = True):
        """Write the batch description into a host buffer (packed by the native host runtime). Returns
        (max_q_len, want_count)."""
        return self.cache.pages.fill_step(
            buf_np, layout.offsets_array, layout.T, layout.B, layout.W, layout.ids_cap_array,
            [e.slot for e in entries], [e.tokens for e in entries],
            [e.want for e in entries] if with_want else None)

    # ------------------------------------------------------------- forward
    def _forward(self, ctx: StepContext, want_rows: Optional[torch.Tensor], taps: Optional[dict] = None) -> torch.Tensor:
        """embedding -> layers in schedule order -> final norm of the wanted
        rows -> head. Returns fp32 logits [rows, vocab]. `taps`, a dictionary,
        receives copies of the residual stream on the way (see `step`)."""
        x = self.model.embedding.forward(ctx.tokens)
        stream = Residual(x)
        if taps is not None:
            taps["embed"] = x.clone()
        views = self.cache.views
        ahead = self._ahead if self._prefetching else None
        for i, e in enumerate(self.model.schedule):
            if ahead is not None and i + 1 < len(self.model.schedule):
                ahead.issue(self._layer_weights[i + 1])
            self.model.layers[e.layer].forward(stream, ctx, views[i])
            if taps is not None:
                taps[f"layer{i}"] = stream.flush().clone()
        if ahead is not None:
            ahead.join()
        h = self.model.final_norm.apply(stream, rows=want_rows, lazy=want_rows is None and taps is None)
        if taps is not None:
            taps["final_norm"] = h.float()
        return self.model.head.forward(h)

    # ---------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry], taps: Optional[dict] = None) -> torch.Tensor:
        """Run the tokens of `entries` and return fp32 logits [n_want, vocab]
        (device), in the order of the entries and of their `want`.

        `taps`, when a dictionary is given, is filled with fp32 copies (device) of the step's intermediate
        results, the debugging taps of the reference (mynah-slm src/arch_qwen3.h:15-18, 46-49: on_embed,
        on_layer, on_final): "embed" [T, hidden], "layer<i>" [T, hidden] for run i of the schedule (the residual
        stream behind it), "final_norm" [wanted rows, hidden] (each wanted row once, ascending). Such a step
        runs kernel by kernel, not from a captured graph, and needs at least one wanted place."""
        self._validate(entries)
        if taps is not None and not any(len(e.want) for e in entries):
            raise EngineError("a step with taps needs at least one wanted place")
        pages = self.cache.pages
        for e in entries:
            pages.reserve(e.slot, len(e.tokens))
        is_decode = all(len(e.tokens) == 1 for e in entries)
        if taps is not None:
            out = self._eager_step(entries, is_decode, taps)
        elif is_decode and self.use_graphs and self.graph_safe:
            logits = self._decode_graph_step(entries, "plain")
            rows = [b for b, e in enumerate(entries) for _ in e.want]
            if rows == list(range(len(entries))):
                out = logits[:len(entries)].clone()          # the graph's output buffer is reused by the next step
            else:
                out = logits[torch.tensor(rows, dtype=torch.int64, device=self.device)]
        else:
            out = None
            if not is_decode and self.use_graphs and self.graph_safe and self.dtype == torch.bfloat16:
                out = self._prompt_graph_step(entries)
            if out is None:
                out = self._eager_step(entries, is_decode)
        for e in entries:
            pages.commit(e.slot, len(e.tokens))
        return out

    # --------------------------------------------------------- prompt graphs
    def _prompt_graph_step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """A prompt step replayed from a captured graph, or None when this shape has no graph (yet). Rows,
        sequences, wanted rows and page lists are padded to the graph's capacities; padding rows belong to no
        sequence (tok_seq -1), padding sequences have no rows."""
        wants = [(b, int(w)) for b, e in enumerate(entries) for w in e.want]
        if not wants:
            return None
        B = len(entries)
        T = sum(len(e.tokens) for e in entries)
        if T > PROMPT_GRAPH_MAX_ROWS:
            return None
        need_ids = [sum(self.cache.pages.n_held(e.slot, g) for e in entries) for g in range(self.n_groups)]
        key = (_prompt_rows_bucket(T), self._bucket(B), self._bucket(len(wants)),
               tuple(max(4, self._bucket(n)) for n in need_ids))
        g = self._prompt_graphs.get(key)
        if g is None:
            seen = self._prompt_seen.get(key, 0)
            if len(self._prompt_seen) >= 1024:                # a book of shapes seen once: never larger than this
                self._prompt_seen.clear()
            self._prompt_seen[key] = seen + 1
            if seen == 0:
                return None                                   # once: run as it is; twice: worth a graph
            layout = StepLayout(T=key[0], B=key[1], W=key[2], ids_cap=list(key[3]))
            meta = torch.zeros((layout.size,), dtype=torch.int32, device=self.device)
            ctx = device_context(layout, meta, [self.n_pages] * self.n_groups, key[0], False, 1, self.runtime.status, self.dtype)
            g = _PromptGraph(layout, meta, ctx)
            if len(self._prompt_graphs) >= self.max_prompt_graphs:
                oldest = min(self._prompt_graphs, key=lambda k: self._prompt_graphs[k].last_use)
                del self._prompt_graphs[oldest]
            self._prompt_graphs[key] = g
        self._prompt_clock += 1
        g.last_use = self._prompt_clock
        layout = g.layout
        host, hi = self._staging.get(layout.size)
        _, n_want = self._fill(host.numpy(), layout, entries)
        want_view = layout.view(host.numpy(), "want")
        uniq, inverse = np.unique(want_view[:n_want], return_inverse=True)
        want_view[:len(uniq)] = uniq
        want_view[len(uniq):] = uniq[0]                       # padding: a row that is wanted anyway
        g.meta.copy_(host[:layout.size], non_blocking=True)
        self._staging.sent(hi)
        self._host_fields(g.ctx, entries)
        from ..ops import lib
        if g.graph is None:
            # run once for real (sizes scratch memory, warms the library), then record the same launches
            pdl_before = lib.set_pdl(True) if PDL_PROMPT else None
            try:
                n0 = lib.launch_count()
                out = self._forward(g.ctx, g.ctx.want)
                g.n_kernels = lib.launch_count() - n0
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    g.logits = self._forward(g.ctx, g.ctx.want)
            finally:
                if pdl_before is not None:
                    lib.set_pdl(pdl_before)
            lib.add_launches(-g.n_kernels)                    # recorded, not run
            g.graph = graph
            logits = out
        else:
            g.graph.replay()
            lib.add_launches(g.n_kernels)
            logits = g.logits
        if len(uniq) == n_want and np.array_equal(inverse, np.arange(n_want)):
            return logits[:n_want].clone()                    # the graph's output buffer is reused by the next replay
        return logits[torch.from_numpy(inverse.astype(np.int64)).to(self.device)]

    def _eager_step(self, entries: Sequence[StepEntry], is_decode: bool, taps: Optional[dict] = None) -> torch.Tensor:
        B = len(entries)
        T = sum(len(e.tokens) for e in entries)
        wants = [(b, int(w)) for b, e in enumerate(entries) for w in e.want]
        ids_cap = [sum(len(self.cache.pages.held(e.slot, g)[0]) for e in entries) for g in range(self.n_groups)]
        # wanted rows are normalised once each; duplicates are expanded afterwards
        layout = StepLayout(T=T, B=B, W=max(len(wants), 1), ids_cap=ids_cap)
        host, hi = self._staging.get(layout.size)
        max_q, n_want = self._fill(host.numpy(), layout, entries)
        want_np = layout.view(host.numpy(), "want")[:n_want]
        uniq, inverse = np.unique(want_np, return_inverse=True)
        layout.view(host.numpy(), "want")[:len(uniq)] = uniq
        dev = torch.empty((layout.size,), dtype=torch.int32, device=self.device)
        dev.copy_(host[:layout.size], non_blocking=True)
        self._staging.sent(hi)
        max_kv = max(self.cache.pages.length[e.slot] + len(e.tokens) for e in entries)
        splits = self._decode_pages(max_kv) if is_decode else 1
        ctx = device_context(layout, dev, [self.n_pages] * self.n_groups, max_q, is_decode, splits,
                             self.runtime.status, self.dtype)
        self._host_fields(ctx, entries)
        if n_want == 0:
            # nothing wanted: the cache is still filled; skip norm and head
            self._forward_layers_only(ctx)
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        rows = ctx.want[:len(uniq)]
        logits = self._forward(ctx, rows, taps)
        if len(uniq) != n_want or not np.array_equal(inverse, np.arange(n_want)):
            logits = logits[torch.from_numpy(inverse.astype(np.int64)).to(self.device)]
        return logits

    def _forward_layers_only(self, ctx: StepContext) -> None:
        x = self.model.embedding.forward(ctx.tokens)
        stream = Residual(x)
        for i, e in enumerate(self.model.schedule):
            self.model.layers[e.layer].forward(stream, ctx, self.cache.views[i])

    def _host_fields(self, ctx: StepContext, entries: Sequence[StepEntry]) -> None:
        ctx.host_q_lens = [len(e.tokens) for e in entries]
        ctx.host_past = [self.cache.pages.length[e.slot] for e in entries]
        ctx.host_slots = [e.slot for e in entries]

    # --------------------------------------------------------- decode graph
    @staticmethod
    def _bucket(B: int) -> int:
        b = 1
        while b < B:
            b *= 2
        return b

    @classmethod
    def _pages_bucket(cls, pages: int) -> int:
        """Page splits of a captured decode step: powers of two up to PAGE_BUCKET_STEP, multiples of it beyond
        (every split without a page is a CTA that starts only to leave)."""
        if PAGE_BUCKET_STEP <= 0 or pages <= PAGE_BUCKET_STEP:
            return cls._bucket(pages)
        return -(-pages // PAGE_BUCKET_STEP) * PAGE_BUCKET_STEP

    def _graph_for(self, B: int, max_kv: int) -> _DecodeGraph:
        """The captured step for this batch size and context: batch sizes and
        page counts are rounded up to powers of two, so a few graphs serve all."""
        bucket = self._bucket(B)
        max_pages_seq = -(-self.spec.max_positions // PAGE_TOKENS)
        splits = min(max(4, self._pages_bucket(self._decode_pages(max_kv))), max_pages_seq)
        g = self._graphs.get((bucket, splits))
        if g is not None:
            return g
        cap = min(bucket * max_pages_seq, self.n_pages + bucket)
        layout = StepLayout(T=bucket, B=bucket, W=1, ids_cap=[cap] * self.n_groups)
        meta = torch.zeros((layout.size,), dtype=torch.int32, device=self.device)
        ctx = device_context(layout, meta, [self.n_pages] * self.n_groups, 1, True, splits, self.runtime.status, self.dtype)
        g = _DecodeGraph(bucket, layout, meta, ctx, splits)
        self._graphs[(bucket, splits)] = g
        return g

    def _decode_graph_step(self, entries: Sequence[StepEntry], mode: str, replays: int = 1, grow: int = 1) -> torch.Tensor:
        B = len(entries)
        max_kv = max(self.cache.pages.length[e.slot] + grow for e in entries)
        g = self._graph_for(B, max_kv)
        host, hi = self._staging.get(g.layout.size)
        self._fill(host.numpy(), g.layout, entries, with_want=False)
        g.meta.copy_(host[:g.layout.size], non_blocking=True)
        self._staging.sent(hi)
        self._host_fields(g.ctx, entries)
        return self._run_graph(g, mode, replays)

    def _run_graph(self, g: _DecodeGraph, mode: str, replays: int = 1) -> torch.Tensor:
        """mode: "plain" (logits), "sample" (tokens), "loop" (tokens, and each
        sequence's token becomes its next input one position on)."""
        from ..ops import lib
        self.sampler.flush_resets()                   # the captured launches read the sampler's rows
        if mode not in g.graphs:
            # first use of this bucket: run once for real (this also sizes scratch
            # memory and warms the library), then record the same launches.
            # Steps of one or two sequences are recorded with programmatic dependent launch: their kernels are
            # so short that a product's start under the norm before it shows (batch 1: 1.014 -> 0.984 ms a
            # step); from batch 8 on it measured the same or slower.
            pdl_before = lib.set_pdl(True) if g.bucket <= PDL_MAX_ROWS else None
            try:
                n0 = lib.launch_count()
                out = self._decode_body(g, mode)
                n_kernels = lib.launch_count() - n0
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    res = self._decode_body(g, mode)
            finally:
                if pdl_before is not None:
                    lib.set_pdl(pdl_before)
            lib.add_launches(-n_kernels)              # recorded, not run
            res.copy_(out)                             # the eager run has produced this step's result
            g.graphs[mode] = (graph, res, n_kernels)
            replays -= 1
        graph, res, n_kernels = g.graphs[mode]
        for _ in range(replays):
            graph.replay()
        lib.add_launches(n_kernels * replays)
        return res

    def _decode_body(self, g: _DecodeGraph, mode: str) -> torch.Tensor:
        self._prefetching = g.bucket <= L2_PREFETCH_MAX_ROWS
        try:
            logits = self._forward(g.ctx, None)
        finally:
            self._prefetching = False
        if mode == "plain":
            return logits
        sampled = self.sampler.sample(logits, g.ctx.slots)
        if mode == "loop":
            kernels.decode_advance(g.ctx.tokens, sampled, g.ctx.tok_pos, g.ctx.kv_len, g.ctx.slots)
        return sampled

    # -------------------------------------------------- sampled decode steps
    def decode_sampled(self, slots: Sequence[int], tokens: Optional[Sequence[int]] = None,
                       feed: Optional[tuple[torch.Tensor, Sequence[int]]] = None) -> torch.Tensor:
        """One decode step for `slots` with `tokens` as their next inputs;
        samples on the device with the sampler's current parameters and returns
        the int32 tokens [bucket] (device; the first len(slots) rows count; the
        buffer is written again by a later step of the same size).
        With feed = (result of an earlier step, rows) sequence i's input is that
        result's row rows[i], taken on the device: the host need not have seen it."""
        pages = self.cache.pages
        if feed is not None:
            if not (self.use_graphs and self.graph_safe):
                raise EngineError("a step fed from the device needs CUDA graphs")
            if len(feed[1]) != len(slots):
                raise EngineError("feed: one row per sequence is needed")
            tokens = [0] * len(slots)
        elif tokens is None:
            raise EngineError("a step needs its input tokens")
        if self.use_graphs and self.graph_safe:
            # the common case: checks, pages and the step's description in one call of the native host runtime
            slots_a = np.asarray(slots, dtype=np.int32)
            toks_a = np.asarray(tokens, dtype=np.int32)
            if len(slots_a) == 0:
                raise EngineError("a step needs at least one sequence")
            try:
                max_kv = pages.max_length(slots_a.tolist()) + 1
            except KeyError as e:
                raise EngineError(f"slot {e.args[0]} is not open") from None
            g = self._graph_for(len(slots_a), max_kv)
            host, hi = self._staging.get(g.layout.size)
            from ..cache import CacheError
            try:
                pages.decode_prepare(host.numpy(), g.layout.offsets_array, g.layout.T, g.layout.B, g.layout.W,
                                     g.layout.ids_cap_array, slots_a, toks_a, self.spec.vocab_size, self.spec.max_positions)
            except CacheError as e:
                if "cache is full" in str(e):
                    raise
                raise EngineError(str(e)) from None
            g.meta.copy_(host[:g.layout.size], non_blocking=True)
            self._staging.sent(hi)
            if feed is not None:
                prev, rows = feed
                n = len(slots_a)
                if list(rows) == list(range(n)):
                    g.ctx.tokens[:n].copy_(prev[:n])
                else:
                    g.ctx.tokens[:n].copy_(prev[torch.tensor(list(rows), dtype=torch.int64, device=self.device)])
            out = self._run_graph(g, "sample", 1)
            pages.commit_many(slots_a, 1)
            return out
        entries = [StepEntry(s, (int(t),)) for s, t in zip(slots, tokens)]
        self._validate(entries)
        for e in entries:
            pages.reserve(e.slot, 1)
        logits = self._eager_step([StepEntry(e.slot, e.tokens, (0,)) for e in entries], True)
        slots_t = torch.tensor(list(slots), dtype=torch.int32, device=self.device)
        out = self.sampler.sample(logits, slots_t)
        for e in entries:
            pages.commit(e.slot, 1)
        return out

    def decode_loop(self, slots: Sequence[int], tokens: Sequence[int], n_steps: int) -> torch.Tensor:
        """`n_steps` sampled decode steps without the host in between: each
        sequence's sampled token is fed back on the device. Returns the tokens
        of the last step (device). Used where only throughput is wanted."""
        if not (self.use_graphs and self.graph_safe):
            raise EngineError("decode_loop needs CUDA graphs")
        entries = [StepEntry(s, (int(t),)) for s, t in zip(slots, tokens)]
        self._validate(entries)
        pages = self.cache.pages
        for e in entries:
            if pages.length[e.slot] + n_steps > self.spec.max_positions:
                raise EngineError(f"slot {e.slot} would outgrow the model's {self.spec.max_positions} positions")
            pages.reserve(e.slot, n_steps)
        out = self._decode_graph_step(entries, "loop", replays=n_steps, grow=n_steps)
        for e in entries:
            pages.commit(e.slot, n_steps)
        return out

    def check_status(self) -> None:
        """Raise if a kernel met an index it had to refuse. Synchronises."""
        from ..ops import gemm_bf16
        word = gemm_bf16.status_word(self.device)
        st = int((self.runtime.status | word).item())
        if st:
            self.runtime.status.zero_()
            word.zero_()
            if st & 16:
                from ..ops.lib import call, stream_ptr
                call("mynah_gemm_tcgen05_reset", stream_ptr())       # flags that a product which gave up may have left raised
            what = [name for bit, name in ((kernels.ST_PAGE_RANGE, "a position without a page"),
                                           (kernels.ST_POS_RANGE, "a position outside the rotation table"),
                                           (kernels.ST_TOKEN_RANGE, "a token id outside the vocabulary"),
                                           (kernels.ST_SPLIT_RANGE, "a decode launch too small for a sequence"),
                                           (16, "a bounded wait inside a kernel ran out")) if st & bit]
            raise EngineError("a kernel refused an index: " + ", ".join(what))
