"""The step function's taps (embedding, the residual stream behind every layer, the final norm) against the
plain implementation's, stage by stage, as the reference gates its engine against its oracle
(mynah-slm tools/eval/compare.py:34-41, taps of src/arch_qwen3.h:15-18, 46-49): when a logit row is off, the first
stage that is off tells where to look. In 32-bit every stage is held to the tolerance of the logits. In bfloat16
every layer is fed the engine's own input of that layer and held to one unit in the last place."""
import numpy as np
import pytest
import torch

from helpers import BF16_LAYER_REL, FP32_REL, TINY, assert_close, make_folder, prompts_for
from plain.model import PlainQwen3, bf16_round, linear, rms_norm, rope_table

pytestmark = pytest.mark.gpu


def _engine(folder, dtype, max_tokens, **kw):
    from mynah_slm_b200.engine.engine import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def _entry(slot, tokens, want):
    from mynah_slm_b200.engine.engine import StepEntry
    return StepEntry(slot, tokens, want)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_every_stage_in_32_bit(tmp_path, name):
    folder = make_folder(tmp_path, name, torch.float32)
    plain = PlainQwen3.from_folder(folder)
    eng = _engine(folder, "float32", 512)
    L = TINY[name]["num_hidden_layers"]
    for n in (1, 70, 150):
        toks = prompts_for(name, [n], seed=n)[0]
        ref_taps, taps = {}, {}
        ref = plain.forward(toks, ref_taps)
        slot = eng.open_sequence()
        got = eng.step([_entry(slot, toks, range(n))], taps=taps).cpu().numpy()
        eng.check_status()
        assert sorted(taps) == sorted(["embed", "final_norm"] + [f"layer{i}" for i in range(L)])
        assert np.array_equal(ref_taps["embed"], taps["embed"].cpu().numpy()), "the embedding is a table lookup"
        for stage in [f"layer{i}" for i in range(L)] + ["final_norm"]:
            assert_close(ref_taps[stage], taps[stage].cpu().numpy(), FP32_REL, f"{name} {n} tokens, stage {stage}")
        assert_close(ref, got, FP32_REL, f"{name} {n} tokens, logits")
        # the same rows from a step without taps (decode steps of one token replay a graph instead)
        eng.close_sequence(slot)
        slot = eng.open_sequence()
        again = eng.step([_entry(slot, toks, range(n))]).cpu().numpy()
        eng.close_sequence(slot)
        assert_close(got, again, 1e-6, f"{name} {n} tokens, with and without taps")


def test_taps_of_a_batch_and_of_a_decode_step(tmp_path):
    """Taps cover all rows of a step: a ragged batch of prompts, then a decode step of the same sequences."""
    folder = make_folder(tmp_path, "B", torch.float32)
    plain = PlainQwen3.from_folder(folder)
    eng = _engine(folder, "float32", 512)
    seqs = prompts_for("B", [40, 7, 65], seed=2)
    slots = [eng.open_sequence() for _ in seqs]
    taps = {}
    eng.step([_entry(s, q[:-1], (len(q) - 2,)) for s, q in zip(slots, seqs)], taps=taps)
    refs = []
    for q in seqs:
        t = {}
        plain.forward(q, t)
        refs.append(t)
    row = 0
    for q, t in zip(seqs, refs):
        n = len(q) - 1
        for stage in ("embed", "layer0", "layer2"):
            assert_close(t[stage][:n], taps[stage][row:row + n].cpu().numpy(), FP32_REL, f"prompt rows, {stage}")
        row += n
    assert_close(np.stack([t["final_norm"][len(q) - 2] for q, t in zip(seqs, refs)]), taps["final_norm"].cpu().numpy(),
                 FP32_REL, "final norm of the wanted rows")
    taps = {}
    eng.step([_entry(s, q[-1:], (0,)) for s, q in zip(slots, seqs)], taps=taps)
    for stage in ("layer0", "layer2", "final_norm"):
        assert_close(np.stack([t[stage][-1] for t in refs]), taps[stage].cpu().numpy(), FP32_REL, f"decode rows, {stage}")
    from mynah_slm_b200.engine.engine import EngineError
    with pytest.raises(EngineError, match="wanted place"):
        eng.step([_entry(slots[0], [1], ())], taps={})


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_every_layer_in_bfloat16_from_its_own_input(tmp_path, name):
    """Layer i of the engine, given what the engine's layer i-1 produced, against the plain implementation's
    bfloat16 mode given the same: one layer's worth of rounding, not a whole model's."""
    folder = make_folder(tmp_path, name, torch.bfloat16)
    mirror = PlainQwen3.from_folder(folder, bf16=True)
    eng = _engine(folder, "bfloat16", 1024)
    L = TINY[name]["num_hidden_layers"]
    for n in (1, 16, 70, 150, 300):
        if n > TINY[name]["max_position_embeddings"]:
            continue
        toks = prompts_for(name, [n], seed=100 + n)[0]
        slot = eng.open_sequence()
        taps = {}
        got = eng.step([_entry(slot, toks, range(n))], taps=taps).cpu().numpy()
        eng.check_status()
        eng.close_sequence(slot)
        t = {k: v.cpu().numpy() for k, v in taps.items()}
        assert np.array_equal(t["embed"], mirror.t["model.embed_tokens.weight"][np.asarray(toks)])
        cos, sin = rope_table(mirror.HD, np.arange(n), mirror.theta)
        x = t["embed"]
        for i in range(L):
            assert_close(mirror.block(i, x, cos, sin), t[f"layer{i}"], BF16_LAYER_REL, f"{name} {n} tokens, layer {i}")
            x = t[f"layer{i}"]
        assert_close(bf16_round(rms_norm(x, mirror.t["model.norm.weight"], mirror.eps)), t["final_norm"], BF16_LAYER_REL,
                     f"{name} {n} tokens, final norm")
        head = mirror.t["model.embed_tokens.weight"] if mirror.tied else mirror.t["lm_head.weight"]
        assert_close(linear(t["final_norm"], head), got, 1e-4, f"{name} {n} tokens, the head on the engine's own rows")
