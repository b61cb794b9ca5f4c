"""Command line in the manner of the reference's `mynah-slm run`
(mynah-slm cli/main.c:22-46, :317-365).

    mynah-slm run (-m <model folder> | --random <config.json> [--weights-seed S]) --tokens 1,2,3
                  [-n 128] [--temp T] [--top-k K] [--top-p P] [--min-p M] [--seed S] [--repeat-penalty R]
                  [--no-stream] [--quiet] [--ctx N] [--dtype bfloat16|float32] [--batch B] [--ignore-eos]
                  [--logits-out <file.npy>]
    mynah-slm random -o <folder> --config <config.json> [--seed S] [--dtype bfloat16|float32]
    mynah-slm --version

The options the reference has keep their names, meanings and defaults: -m,
-n (128), --ctx, --temp (0.6), --top-k (20), --top-p (0.95), --min-p (0),
--seed (0), --repeat-penalty (1.0), --no-stream, --quiet. The model is a
folder (config.json + safetensors) instead of a GGUF file. The text options
(-p, --system, --think, --show-think, --raw) and -t/--threads have no
counterpart: prompts are token ids, given with --tokens (repeatable: several
prompts make a batch) or --tokens-file (one prompt per line). Generated ids
go to stdout, one line per prompt; the timing line goes to stderr
(src/timing.c:56-62), so stdout stays pipeable.

--random <config.json> runs a model whose weights are made on the device from
the configuration and a seed (--weights-seed, else --seed), without a folder.
--logits-out <file.npy> first runs every prompt whole, one after another, and
writes the fp32 logits of all their positions as one array [positions, vocab]
in the .npy format of the reference's parity tool (tests/test_parity.c:140-146,
tests/npy.c:17-48: version 1.0, '<f4').
"""
from __future__ import annotations

import json
import sys

from . import __version__

USAGE = __doc__


def _fail(msg: str) -> int:
    print(f"mynah-slm: {msg}", file=sys.stderr)
    return 2


def _parse_ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def _write_logits(llm, prompts: list[list[int]], path: str) -> None:
    """Every prompt whole in a step of its own; the logits of all positions, in the order of the prompts."""
    import numpy as np
    from .engine.engine import StepEntry
    rows = []
    for p in prompts:
        slot = llm.engine.open_sequence()
        rows.append(llm.engine.step([StepEntry(slot, p, range(len(p)))]).cpu().numpy())
        llm.engine.check_status()
        llm.engine.close_sequence(slot)
    with open(path, "wb") as f:
        np.lib.format.write_array(f, np.ascontiguousarray(np.concatenate(rows), dtype="<f4"), version=(1, 0))


def cmd_run(argv: list[str]) -> int:
    o = {"model": None, "max_new": 128, "ctx": 0, "temp": 0.6, "top_k": 20, "top_p": 0.95, "min_p": 0.0, "seed": 0,
         "repeat_penalty": 1.0, "stream": True, "quiet": False, "dtype": "bfloat16", "ignore_eos": False,
         "batch": 64, "device": "cuda:0", "random": None, "weights_seed": None, "logits_out": None}
    prompts: list[list[int]] = []
    i = 0
    valued = {"-m": ("model", str), "-n": ("max_new", int), "--ctx": ("ctx", int), "--temp": ("temp", float),
              "--top-k": ("top_k", int), "--top-p": ("top_p", float), "--min-p": ("min_p", float),
              "--seed": ("seed", int), "--repeat-penalty": ("repeat_penalty", float), "--dtype": ("dtype", str),
              "--batch": ("batch", int), "--device": ("device", str), "--random": ("random", str),
              "--weights-seed": ("weights_seed", int), "--logits-out": ("logits_out", str)}
    while i < len(argv):
        a = argv[i]
        if a in valued or a in ("--tokens", "--tokens-file"):
            if i + 1 >= len(argv):
                return _fail(f"{a} needs a value")
            v = argv[i + 1]
            i += 2
            try:
                if a == "--tokens":
                    prompts.append(_parse_ids(v))
                elif a == "--tokens-file":
                    with open(v) as f:
                        prompts += [_parse_ids(line) for line in f if line.strip()]
                else:
                    key, conv = valued[a]
                    o[key] = conv(v)
            except (ValueError, OSError) as e:
                return _fail(f"bad value for {a}: {e}")
        elif a == "--no-stream":
            o["stream"] = False
            i += 1
        elif a == "--quiet":
            o["quiet"] = True
            i += 1
        elif a == "--ignore-eos":
            o["ignore_eos"] = True
            i += 1
        else:
            return _fail(f"unknown option '{a}'")
    if bool(o["model"]) == bool(o["random"]) or not prompts:
        return _fail("run needs -m <model folder> or --random <config.json> (one of them), and --tokens <ids> "
                     "(or --tokens-file <file>)")
    if any(not p for p in prompts):
        return _fail("empty prompt")

    from .engine.api import LLM
    longest = max(len(p) for p in prompts)
    per_seq = o["ctx"] if o["ctx"] > 0 else longest + o["max_new"] + 8       # cli/main.c:264-265
    per_seq = -(-per_seq // 64) * 64
    try:
        max_tokens = per_seq * min(len(prompts), o["batch"])
        if o["random"]:
            wseed = o["seed"] if o["weights_seed"] is None else o["weights_seed"]
            llm = LLM.random(o["random"], seed=wseed, dtype=o["dtype"], max_tokens=max_tokens, device=o["device"])
        else:
            llm = LLM(o["model"], dtype=o["dtype"], max_tokens=max_tokens, device=o["device"])
        if o["logits_out"]:
            _write_logits(llm, prompts, o["logits_out"])
    except Exception as e:                                                    # noqa: BLE001 - report, as the reference does
        print(f"mynah-slm: {e}", file=sys.stderr)
        return 1
    streamed = len(prompts) == 1 and o["stream"]

    def cb(index: int, tok: int) -> int:
        if streamed:
            print(tok, end=" ", flush=True)
        return 0

    max_new = o["max_new"]
    if o["ctx"] > 0:
        max_new = max(0, min(max_new, per_seq - longest))
    try:
        results = llm.generate(prompts, max_new=max_new, temp=o["temp"], top_k=o["top_k"], top_p=o["top_p"],
                               min_p=o["min_p"], seed=o["seed"], repeat_penalty=o["repeat_penalty"],
                               ignore_eos=o["ignore_eos"], max_batch=o["batch"], callback=cb)
    except Exception as e:                                                    # noqa: BLE001
        print(f"mynah-slm: {e}", file=sys.stderr)
        return 1
    if streamed:
        print()
    else:
        for r in results:
            print(" ".join(str(t) for t in r.tokens))
    if not o["quiet"]:
        print(llm.last_timing.format(), file=sys.stderr)
    return 0


def cmd_random(argv: list[str]) -> int:
    import torch
    o = {"out": None, "config": None, "seed": 0, "dtype": "bfloat16"}
    i = 0
    names = {"-o": "out", "--config": "config", "--seed": "seed", "--dtype": "dtype"}
    while i < len(argv):
        if argv[i] not in names:
            return _fail(f"unknown option '{argv[i]}'")
        if i + 1 >= len(argv):
            return _fail(f"{argv[i]} needs a value")
        o[names[argv[i]]] = argv[i + 1]
        i += 2
    if not o["out"] or not o["config"]:
        return _fail("random needs -o <folder> and --config <config.json>")
    from .registry import parse_config
    from .weights.random_init import write_random_model
    try:
        with open(o["config"]) as f:
            typed = parse_config(json.load(f))
        dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[o["dtype"]]
        write_random_model(o["out"], typed, int(o["seed"]), dtype)
    except Exception as e:                                                    # noqa: BLE001
        print(f"mynah-slm: {e}", file=sys.stderr)
        return 1
    return 0


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        print(USAGE, file=sys.stderr)
        return 2
    if argv[0] in ("--version", "-v"):
        print(__version__)
        return 0
    if argv[0] in ("--help", "-h"):
        print(USAGE)
        return 0
    if argv[0] in ("run", "random") and any(a in ("--help", "-h") for a in argv[1:]):
        print(USAGE)
        return 0
    if argv[0] == "run":
        return cmd_run(argv[1:])
    if argv[0] == "random":
        return cmd_random(argv[1:])
    print(f"mynah-slm: unknown command '{argv[0]}'", file=sys.stderr)
    print(USAGE, file=sys.stderr)
    return 2


if __name__ == "__main__":
    raise SystemExit(main())
