"""The Python half of the C interface (`include/mynah_slm_b200.h`).

The C library forwards each of its calls to one function here. The functions
take and return plain numbers, strings and memory addresses of the caller's
arrays, and never raise: each returns (code, message, value), the code being
one of `enum mynah_status`. What they call is the engine's one step function,
its generation loop and its sampler; there is nothing of their own in them.
"""
from __future__ import annotations

import ctypes
import functools
import os
import time

import numpy as np

OK, ERR_ARGUMENT, ERR_CONFIG, ERR_WEIGHTS, ERR_CACHE_FULL, ERR_DEVICE, ERR_INTERNAL, STOPPED = range(8)
FINISH = {"stop": 0, "length": 1, "context": 2, "callback": 3}


def _code_of(e: BaseException) -> int:
    from ..cache.pages import CacheError
    from ..config.keys import ConfigError
    from ..csrc.build import BuildError
    from ..ops.lib import KernelError, KernelLibraryError
    from ..weights.loader import WeightError
    from .engine import EngineError
    from .generate import GenerationError
    if isinstance(e, WeightError):
        return ERR_WEIGHTS
    if isinstance(e, ConfigError):
        return ERR_CONFIG
    if isinstance(e, CacheError):
        return ERR_CACHE_FULL if "full" in str(e) or "no free slot" in str(e) else ERR_ARGUMENT
    if isinstance(e, (KernelLibraryError, BuildError)):
        return ERR_DEVICE
    if isinstance(e, EngineError):
        text = str(e)
        return ERR_DEVICE if ("CUDA device" in text or "a kernel refused" in text) else ERR_ARGUMENT
    if isinstance(e, (KernelError, GenerationError, ValueError, KeyError, FileNotFoundError, NotADirectoryError)):
        return ERR_ARGUMENT
    return ERR_INTERNAL


def _guarded(fn):
    @functools.wraps(fn)
    def call(*args):
        try:
            return OK, "", fn(*args)
        except BaseException as e:                 # noqa: BLE001 - nothing may cross into the C caller
            return _code_of(e), f"{e}" or type(e).__name__, None
    return call


def _ints(addr: int, n: int, ctype=ctypes.c_int32) -> np.ndarray:
    if n <= 0:
        return np.zeros((0,), dtype=np.int32)
    if not addr:
        raise ValueError("a NULL array was given where entries are needed")
    return np.ctypeslib.as_array(ctypes.cast(addr, ctypes.POINTER(ctype)), shape=(n,))


@_guarded
def create(folder: str, dtype: str, max_tokens: int, max_seqs: int):
    os.environ.setdefault("MYNAH_QUIET", "1")          # a first build must not write to the caller's stderr
    from .api import LLM
    if not os.path.isdir(folder):
        raise FileNotFoundError(f"{folder} is not a model folder")
    return LLM(folder, dtype=dtype, max_tokens=max_tokens, max_seqs=max_seqs if max_seqs > 0 else None)


@_guarded
def create_random(config_json: str, seed: int, dtype: str, max_tokens: int, max_seqs: int):
    os.environ.setdefault("MYNAH_QUIET", "1")
    from .api import LLM
    if not os.path.isfile(config_json):
        raise FileNotFoundError(f"{config_json} is not a file")
    return LLM.random(config_json, seed=seed, dtype=dtype, max_tokens=max_tokens, max_seqs=max_seqs if max_seqs > 0 else None)


@_guarded
def info(llm, what: str) -> int:
    eng = llm.engine
    if what == "vocab_size":
        return eng.spec.vocab_size
    if what == "max_positions":
        return eng.spec.max_positions
    if what == "hidden_size":
        return eng.spec.hidden_size
    if what == "n_layers":
        return len(eng.spec.layers)
    if what == "free_tokens":
        return eng.free_tokens()
    raise ValueError(f"unknown accessor {what!r}")


@_guarded
def eos_ids(llm, addr: int, capacity: int) -> int:
    ids = list(llm.engine.spec.eos_token_ids)
    out = _ints(addr, min(capacity, len(ids)))
    out[:] = ids[:len(out)]
    return len(ids)


@_guarded
def slot_open(llm) -> int:
    return llm.engine.open_sequence()


@_guarded
def slot_close(llm, slot: int) -> int:
    if slot not in llm.engine.cache.pages.length:
        raise ValueError(f"slot {slot} is not open")
    llm.engine.close_sequence(slot)
    return 0


@_guarded
def slot_length(llm, slot: int) -> int:
    return llm.engine.length(slot) if slot in llm.engine.cache.pages.length else -1


@_guarded
def step(llm, n: int, slots_addr: int, n_new_addr: int, tokens_addr: int, n_want_addr: int, want_addr: int, out_addr: int) -> int:
    from .engine import StepEntry
    if n < 1:
        raise ValueError("a step needs at least one sequence")
    slots, n_new, n_want = _ints(slots_addr, n, ctypes.c_int), _ints(n_new_addr, n, ctypes.c_int), _ints(n_want_addr, n, ctypes.c_int)
    if (n_new < 1).any() or (n_want < 0).any():
        raise ValueError("every sequence brings at least one token and a count of wanted places that is not negative")
    tokens, want = _ints(tokens_addr, int(n_new.sum())), _ints(want_addr, int(n_want.sum()), ctypes.c_int)
    entries, t, w = [], 0, 0
    for i in range(n):
        entries.append(StepEntry(int(slots[i]), tokens[t:t + n_new[i]].tolist(), want[w:w + n_want[i]].tolist()))
        t += int(n_new[i])
        w += int(n_want[i])
    eng = llm.engine
    logits = eng.step(entries)
    eng.check_status()
    rows = int(logits.shape[0])
    if rows:
        if not out_addr:
            raise ValueError("logits are wanted but logits_out is NULL")
        dst = np.ctypeslib.as_array(ctypes.cast(out_addr, ctypes.POINTER(ctypes.c_float)), shape=(rows, eng.spec.vocab_size))
        dst[:] = logits.cpu().numpy()
    return rows


def _params(p: tuple):
    from ..sampling.sampler import SamplingParams
    temp, top_k, top_p, min_p, repeat, freq, presence, window, seed = p
    return SamplingParams(temp=temp, top_k=top_k, top_p=top_p, min_p=min_p, repeat_penalty=repeat, freq_penalty=freq,
                          presence_penalty=presence, penalty_window=window, seed=seed)


@_guarded
def sample(llm, logits_addr: int, n_rows: int, p: tuple, rng_addr: int, out_addr: int) -> int:
    import torch
    from ..ops import kernels
    eng = llm.engine
    params = _params(p)
    params.validate()
    V = eng.spec.vocab_size
    if n_rows < 1 or not logits_addr or not out_addr:
        raise ValueError("sample needs rows of logits and a place for the tokens")
    src = np.ctypeslib.as_array(ctypes.cast(logits_addr, ctypes.POINTER(ctypes.c_float)), shape=(n_rows, V))
    logits = torch.from_numpy(np.array(src, dtype=np.float32)).to(eng.device)
    if params.temp <= 0.0:
        toks = kernels.argmax(logits)
    else:
        if not rng_addr:
            raise ValueError("a draw needs generator states (rng is NULL)")
        states = np.ctypeslib.as_array(ctypes.cast(rng_addr, ctypes.POINTER(ctypes.c_uint64)), shape=(n_rows,))
        rng = torch.from_numpy(states.view(np.int64).copy()).to(eng.device)
        dev_params = torch.tensor([params.temp, params.top_p, params.min_p, float(params.top_k), 1.0, 0.0, 0.0, 0.0],
                                  dtype=torch.float32, device=eng.device)
        toks = kernels.sample(logits, dev_params, rng, None)
        states[:] = rng.cpu().numpy().view(np.uint64)
    _ints(out_addr, n_rows)[:] = toks.cpu().numpy()
    return n_rows


@_guarded
def generate(llm, requests: list, p: tuple, stop, max_batch: int, cb_addr: int, ctx_addr: int, results: list):
    """requests: [(tokens address, n, max_new)]; results: [(tokens address, capacity)]. Returns
    (per request (n_tokens, produced, finish), timing tuple, stopped)."""
    params = _params(p)
    prompts = [_ints(a, n).tolist() for a, n, _ in requests]
    limits = [m for _, _, m in requests]
    if any(n < 1 for _, n, _ in requests):
        raise ValueError("empty prompt")
    cb = None
    stopped = [False]
    if cb_addr:
        fn = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int32)(cb_addr)

        def cb(index: int, token: int) -> int:
            r = fn(ctx_addr, index, token)
            if r:
                stopped[0] = True
            return r
    from ..sampling.sampler import SamplingParams  # noqa: F401
    from .api import EngineBackend
    from .generate import Request, Timing, generate as run
    eng = llm.engine
    stop_ids = tuple(eng.spec.eos_token_ids) if stop is None else tuple(stop)
    timing = Timing(load_s=llm.load_s)
    t0 = time.perf_counter()
    out = run(EngineBackend(eng, params), [Request(list(q), m) for q, m in zip(prompts, limits)], stop_ids=stop_ids,
              max_batch=max_batch, callback=cb, timing=timing)
    del t0
    llm.last_timing = timing
    summary = []
    for r, (addr, cap) in zip(out, results):
        n = min(len(r.tokens), cap)
        _ints(addr, n)[:] = r.tokens[:n]
        summary.append((n, int(r.produced), FINISH.get(r.finish_reason, 1)))
    return summary, (timing.load_s, timing.prefill_s, timing.decode_s, timing.ttft_s, timing.n_prompt, timing.n_gen), stopped[0]
