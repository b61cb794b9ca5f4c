"""Randomly drawn configurations and randomly cut batches against the plain implementation: sizes and cuts that
nobody chose by hand (seeded, so a failure can be run again)."""
import numpy as np
import pytest
import torch

from helpers import BF16_REL, FP32_REL, TINY, make_folder, rel_err
from plain.model import PlainQwen3

pytestmark = pytest.mark.gpu
DTYPES = [("float32", torch.float32), ("bfloat16", torch.bfloat16)]


def _check(what, ref, got, tol):
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    e = rel_err(ref, got)
    if e > tol:
        rows = np.linalg.norm(ref - got, axis=-1) / np.maximum(np.linalg.norm(ref, axis=-1), 1e-30)
        raise AssertionError(f"{what}: rel error {e:.3e} > {tol:.0e}, first wrong row {int(np.argmax(rows > tol))}")


@pytest.mark.parametrize("seed", [1, 2])
def test_random_configurations(tmp_path, seed):
    """Head sizes in steps of 16, any number of heads and groups, widths and vocabularies that are no power of two,
    windows on some layers: a ragged prompt step and the last tokens one by one, in both precisions."""
    from mynah_slm_b200.engine.engine import Engine, StepEntry
    rng = np.random.default_rng(seed)
    for ci in range(10):
        HD, KV = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 192, 256])), int(rng.choice([1, 2, 3, 4]))
        G, D = int(rng.choice([1, 2, 3, 4, 5, 8])), int(rng.choice([40, 72, 88, 96, 104, 136, 200, 264]))
        F, V = int(rng.choice([56, 96, 136, 208, 264, 400])), int(rng.choice([97, 130, 257, 500, 777, 1001, 1537]))
        L = int(rng.integers(1, 4))
        win = bool(rng.random() < 0.5)
        cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=L, hidden_size=D,
                   num_attention_heads=KV * G, num_key_value_heads=KV, head_dim=HD, intermediate_size=F, vocab_size=V,
                   rope_theta=float(rng.choice([10000.0, 500000.0])), rms_norm_eps=float(rng.choice([1e-6, 1e-5, 1e-3])),
                   tie_word_embeddings=bool(rng.random() < 0.5), max_position_embeddings=512, hidden_act="silu",
                   attention_bias=False, rope_scaling=None, use_sliding_window=win,
                   sliding_window=int(rng.choice([17, 40, 64, 100])) if win else None,
                   max_window_layers=int(rng.integers(0, L + 1)), eos_token_id=1)
        lens = [int(x) for x in rng.integers(3, 300, size=3)]
        seqs = [rng.integers(0, V, size=n).tolist() for n in lens]
        for dtype, wdt in DTYPES:
            tag = f"seed {seed} configuration {ci} ({cfg}) {dtype}"
            folder = make_folder(tmp_path, f"c{ci}{dtype}", wdt, config=cfg, seed=ci)
            plain = PlainQwen3.from_folder(folder)
            eng = Engine.from_folder(folder, dtype=dtype, max_tokens=64 * 16)
            slots = [eng.open_sequence() for _ in seqs]
            heads = [max(1, n - 6) for n in lens]
            out = eng.step([StepEntry(sl, s[:h], range(h)) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
            got, row = [[] for _ in seqs], 0
            for i, h in enumerate(heads):
                got[i].append(out[row:row + h]); row += h
            done = list(heads)
            live = [i for i in range(3) if done[i] < lens[i]]
            while live:
                out = eng.step([StepEntry(slots[i], seqs[i][done[i]:done[i] + 1], (0,)) for i in live]).cpu().numpy()
                for r, i in enumerate(live):
                    got[i].append(out[r:r + 1]); done[i] += 1
                live = [i for i in live if done[i] < lens[i]]
            eng.check_status()
            for i, s in enumerate(seqs):
                _check(f"{tag}, sequence of {lens[i]}", plain.forward(s), np.concatenate(got[i]), FP32_REL if dtype == "float32" else BF16_REL)


@pytest.mark.parametrize("dtype,wdt", DTYPES)
@pytest.mark.parametrize("name", ["A", "C", "E"])
def test_random_cuts_of_random_batches(tmp_path, name, dtype, wdt):
    """Batches of one to five sequences whose prompts come in one to three pieces of random sizes (the pieces of a
    step run together), with random wanted places, then token by token; slots and pages are reused round after round."""
    from mynah_slm_b200.engine.engine import Engine, StepEntry
    folder = make_folder(tmp_path, name, wdt)
    plain = PlainQwen3.from_folder(folder)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=64 * 40)
    V, P = TINY[name]["vocab_size"], TINY[name]["max_position_embeddings"]
    tol = FP32_REL if dtype == "float32" else BF16_REL
    rng = np.random.default_rng(13)
    for rnd in range(8):
        B = int(rng.integers(1, 6))
        lens = [int(rng.integers(2, min(260, P) + 1)) for _ in range(B)]
        seqs = [rng.integers(0, V, size=n).tolist() for n in lens]
        slots = [eng.open_sequence() for _ in seqs]
        cuts = []
        for n in lens:
            p = int(rng.integers(1, n + 1))
            pts = sorted(set([0, p] + [int(x) for x in rng.integers(1, p + 1, size=int(rng.integers(0, 3)))]))
            cuts.append(list(zip(pts[:-1], pts[1:])))
        got, done = [dict() for _ in seqs], [0] * B
        while any(cuts):
            entries, meta = [], []
            for i in range(B):
                if cuts[i]:
                    lo, hi = cuts[i].pop(0)
                    want = sorted(set(int(x) for x in rng.integers(0, hi - lo, size=min(hi - lo, int(rng.integers(0, 6))))))
                    entries.append(StepEntry(slots[i], seqs[i][lo:hi], tuple(want)))
                    meta.append((i, lo, want))
                    done[i] = hi
            out = eng.step(entries).cpu().numpy()
            row = 0
            for i, lo, want in meta:
                for w in want:
                    got[i][lo + w] = out[row]; row += 1
        live = []
        for i in range(B):
            if done[i] < lens[i]:
                live.append(i)
            else:
                eng.close_sequence(slots[i])
        while live:
            out = eng.step([StepEntry(slots[i], seqs[i][done[i]:done[i] + 1], (0,)) for i in live]).cpu().numpy()
            nxt = []
            for r, i in enumerate(live):
                got[i][done[i]] = out[r]
                done[i] += 1
                if done[i] < lens[i]:
                    nxt.append(i)
                else:
                    eng.close_sequence(slots[i])
            live = nxt
        eng.check_status()
        for i, s in enumerate(seqs):
            if got[i]:
                pos = sorted(got[i])
                _check(f"{name} {dtype} round {rnd} sequence {i} of {lens[i]}", plain.forward(s)[pos], np.stack([got[i][p] for p in pos]), tol)
