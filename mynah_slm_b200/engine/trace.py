"""Trace replay over `Engine.step` (the program behind `bin/trace_run`).

The reference's ancestor is tests/test_parity.c (mynah-slm): token ids in,
one step at a time, logits of every position out, no judgement of its own
(:6-8, :140-146). This one takes batches, unequal lengths and explicit ends,
and holds nothing of its own: requests map to the engine's slots, tokens go
through the engine's step function, and the logits it writes are the step's.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids through the engine and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from .engine import Engine, StepEntry
    os.makedirs(args.out, exist_ok=True)
    engine = Engine.from_folder(args.model, dtype=args.dtype, max_tokens=args.max_tokens, device=args.device)
    slots: dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.open_sequence()
            entries.append(StepEntry(slots[rid], e["tokens"], tuple(e.get("want", ()))))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                arr = logits.cpu().numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            engine.check_status()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                engine.close_sequence(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0
