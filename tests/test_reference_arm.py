"""The reference arm of bench.py on a tiny model: the reference checkout is copied and compiled, a random-weights
GGUF is written for it, and its own forward pass runs the workload's shape (sequences one after another, prompts
token by token, greedy decode steps). Skipped where the checkout, gcc or the gguf package is absent."""
import os
import sys

import pytest

from helpers import TINY

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_runs_a_tiny_model():
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm
    try:
        r = reference_arm.run(dict(TINY["B"]), n_seqs=2, prompt_len=12, warmup=1, steps=3, budget_s=300.0)
    except reference_arm.Unavailable as e:
        pytest.skip(str(e))
    assert r["decode_tokens"] == 6 and r["prompt_tokens"] == 22 and r["decode_s"] > 0 and r["prompt_s"] > 0


def test_reference_arm_gives_up_when_the_run_would_not_fit():
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm
    try:
        reference_arm.build()
    except reference_arm.Unavailable as e:
        pytest.skip(str(e))
    with pytest.raises(reference_arm.Unavailable, match="cannot fit the time limit"):
        reference_arm.run(dict(TINY["A"]), n_seqs=8, prompt_len=200, warmup=1, steps=3, budget_s=1e-9)
