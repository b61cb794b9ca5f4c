"""Steps with many sequences, against the plain implementation.

A decode step of up to 16 rows runs this package's own small-batch products
and, while it has few pages, the one-launch attention; from 17 rows on the
products go another way (the library, or the wide-tile kernel), the attention
takes three launches and the sampler sees up to 64 rows, all inside captured
graphs of the buckets 32 and 64. These tests put 8, 17, 33 and 64 sequences
into one step: unequal prompts in one prompt step, then decode steps in which
the shorter requests end earlier, then a second batch in the slots and pages
the first gave back; in bfloat16 and in 32-bit, on the tiny configurations
whose head sizes the tensor-core kernels take, and on two layers with the
measured layer sizes. Every logit row is compared with the plain
implementation run on the whole sequence.
"""
import numpy as np
import pytest
import torch

from helpers import BF16_REL, FP32_REL, TINY, assert_close, make_folder
from plain.model import PlainQwen3

pytestmark = pytest.mark.gpu


def _engine(folder, dtype, max_tokens, **kw):
    from mynah_slm_b200.engine.engine import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def _entry(slot, tokens, want):
    from mynah_slm_b200.engine.engine import StepEntry
    return StepEntry(slot, tokens, want)


def run_batch(eng, seqs, prompt_lens, n_decode, want_prompt):
    """One batch through the step function: all prompts in one step, then one token each until every request has
    had its `n_decode[i]` decode steps; a request that is done closes at once. Returns per request the places
    whose logits were taken and the rows got."""
    slots = [eng.open_sequence() for _ in seqs]
    places = [list(want_prompt(p)) for p in prompt_lens]
    out = eng.step([_entry(s, q[:p], w) for s, q, p, w in zip(slots, seqs, prompt_lens, places)]).cpu().numpy()
    got = [[] for _ in seqs]
    row = 0
    for i, w in enumerate(places):
        got[i].append(out[row:row + len(w)])
        row += len(w)
    t = 0
    live = [i for i in range(len(seqs)) if n_decode[i] > 0]
    for i in range(len(seqs)):
        if n_decode[i] == 0:
            eng.close_sequence(slots[i])
    while live:
        out = eng.step([_entry(slots[i], [seqs[i][prompt_lens[i] + t]], (0,)) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
            places[i].append(prompt_lens[i] + t)
        t += 1
        for i in live:
            if t >= n_decode[i]:
                eng.close_sequence(slots[i])
        live = [i for i in live if t < n_decode[i]]
    eng.check_status()
    return slots, places, [np.concatenate(g) for g in got]


def shapes_of_a_batch(rng, n_seqs, max_prompt, min_decode, max_decode):
    prompt_lens = rng.integers(1, max_prompt + 1, size=n_seqs).tolist()
    prompt_lens[0] = 1                                   # a prompt of one token among the others
    prompt_lens[-1] = max_prompt
    n_decode = rng.integers(min_decode, max_decode + 1, size=n_seqs).tolist()
    n_decode[n_seqs // 2] = max_decode                   # someone stays to the end
    if n_seqs > 2:
        n_decode[1] = 1                                  # and someone leaves after the first decode step
    return prompt_lens, n_decode


@pytest.mark.parametrize("n_seqs", [8, 17, 33, 64])
@pytest.mark.parametrize("name,dtype", [("D", "bfloat16"), ("D", "float32"), ("E", "bfloat16"), ("E", "float32")])
def test_many_sequences_in_a_step(tmp_path, name, dtype, n_seqs):
    wdt = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_folder(tmp_path, name, wdt)
    plain = PlainQwen3.from_folder(folder)
    V = TINY[name]["vocab_size"]
    rng = np.random.default_rng(1000 + n_seqs)
    tol = FP32_REL if dtype == "float32" else BF16_REL
    batches = [shapes_of_a_batch(rng, n_seqs, 140, 2, 12), shapes_of_a_batch(rng, n_seqs // 2 + 1, 100, 8, 10)]
    need = max(sum(-(-(p + d) // 64) * 64 for p, d in zip(*b)) for b in batches)
    eng = _engine(folder, dtype, need, max_seqs=n_seqs)       # exactly the slots and the pages of the largest batch
    seen = []
    for bi, (prompt_lens, n_decode) in enumerate(batches):
        seqs = [rng.integers(0, V, size=p + d).tolist() for p, d in zip(prompt_lens, n_decode)]
        slots, places, got = run_batch(eng, seqs, prompt_lens, n_decode, lambda p: (0, p - 1) if p > 1 else (0,))
        seen.append(set(slots))
        for i, q in enumerate(seqs):
            ref = plain.forward(q)[places[i]]
            assert_close(ref, got[i], tol, f"{name} {dtype} {n_seqs} sequences, batch {bi}, request {i} "
                                           f"(prompt {prompt_lens[i]}, decoded {n_decode[i]})")
    assert seen[1] <= seen[0], "the second batch did not run in slots of the first"
    assert eng.free_tokens() == eng.n_pages * 64, "pages were lost"
    if eng.use_graphs:
        buckets = {k[0] for k in eng._graphs}
        assert max(buckets) >= n_seqs, f"no captured step of {n_seqs} rows was used: {sorted(buckets)}"


def test_64_sequences_of_the_measured_layer_sizes(tmp_path):
    """Two layers of the measured shape (width 1,024, 16 query heads over 8 kv heads of 128, feed-forward 3,072),
    64 sequences in a step, three of them with prompts beyond 2,048 positions: the decode steps run from the
    graph of 64 rows and 48 pages, every product of a layer and the head take the route of 17 rows and more, the
    attention takes three launches. Short sequences sit beside long ones, a prompt of one token among them; some
    end after the first decode step."""
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=1024,
               num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=4099,
               rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096,
               hidden_act="silu", attention_bias=False, rope_scaling=None, use_sliding_window=False, sliding_window=None,
               max_window_layers=2, eos_token_id=1)
    folder = make_folder(tmp_path, "shape", torch.bfloat16, config=cfg, seed=6)
    plain = PlainQwen3.from_folder(folder)
    rng = np.random.default_rng(64)
    n_seqs = 64
    prompt_lens = rng.integers(1, 130, size=n_seqs).tolist()
    prompt_lens[0], prompt_lens[20], prompt_lens[41], prompt_lens[63] = 1, 2110, 2049, 2100
    n_decode = rng.integers(1, 9, size=n_seqs).tolist()
    n_decode[20] = n_decode[63] = 8
    n_decode[41] = 3
    seqs = [rng.integers(0, cfg["vocab_size"], size=p + d).tolist() for p, d in zip(prompt_lens, n_decode)]
    need = sum(-(-(p + d) // 64) * 64 for p, d in zip(prompt_lens, n_decode))
    eng = _engine(folder, "bfloat16", need, max_seqs=n_seqs)
    _, places, got = run_batch(eng, seqs, prompt_lens, n_decode, lambda p: (p - 1,))
    assert (64, 48) in eng._graphs, sorted(eng._graphs)
    for i, q in enumerate(seqs):
        ref = plain.forward(q)[places[i]]
        assert_close(ref, got[i], BF16_REL, f"request {i} (prompt {prompt_lens[i]}, decoded {n_decode[i]})")
    assert eng.free_tokens() == eng.n_pages * 64, "pages were lost"


@pytest.mark.parametrize("name", ["D", "E", "B"])
def test_a_further_piece_of_a_prompt_from_a_replayed_graph(tmp_path, name):
    """Prompts that go on where an earlier step stopped (positions > 0 in the cache), in steps whose padded shape
    comes five times: the first runs as it is, the second is captured, the others are replayed from the graph
    with other tokens, other lengths and other starting positions, in other slots and pages."""
    folder = make_folder(tmp_path, name, torch.bfloat16)
    plain = PlainQwen3.from_folder(folder)
    V = TINY[name]["vocab_size"]
    eng = _engine(folder, "bfloat16", 64 * 16)
    rng = np.random.default_rng(17)
    for rnd in range(5):
        # three pieces of 33 to 42 tokens behind 65 to 85 positions: always 128 padded rows, 4 sequences, 8 pages
        firsts = rng.integers(65, 86, size=3).tolist()
        seconds = rng.integers(33, 43, size=3).tolist()
        if rnd % 2 == 0:
            firsts[int(rng.integers(0, 3))] = 0                     # beside them, one that starts at position 0
        seqs = [rng.integers(0, V, size=a + b).tolist() for a, b in zip(firsts, seconds)]
        slots = [eng.open_sequence() for _ in seqs]
        started = [(s, q[:a]) for s, q, a in zip(slots, seqs, firsts) if a > 0]
        eng.step([_entry(s, t, ()) for s, t in started])
        n_before = sum(1 for g in eng._prompt_graphs.values() if g.graph is not None)
        got = eng.step([_entry(s, q[a:a + b], range(b)) for s, q, a, b in zip(slots, seqs, firsts, seconds)]).cpu().numpy()
        eng.check_status()
        row = 0
        for q, a, b in zip(seqs, firsts, seconds):
            assert_close(plain.forward(q[:a + b])[a:a + b], got[row:row + b], BF16_REL,
                         f"{name} round {rnd}: piece of {b} behind {a}")
            row += b
        for s in slots:
            eng.close_sequence(s)
        assert n_before == (1 if rnd >= 2 else 0), f"round {rnd}: {n_before} captured prompt steps before it"
    assert len(eng._prompt_graphs) == 1, "the five steps did not share one padded shape"


def test_layers_of_the_8b_shape(tmp_path):
    """Two layers with the layer sizes of the largest workload (width 4,096, 32 query heads over 8 kv heads of
    128, feed-forward 12,288, a head of its own): prompts of unequal lengths in one step, then decode steps, against
    the plain implementation."""
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=4096,
               num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=2056,
               rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096,
               hidden_act="silu", attention_bias=False, rope_scaling=None, use_sliding_window=False, sliding_window=None,
               max_window_layers=2, eos_token_id=1)
    folder = make_folder(tmp_path, "shape8b", torch.bfloat16, config=cfg, seed=8)
    plain = PlainQwen3.from_folder(folder)
    rng = np.random.default_rng(8)
    prompt_lens, n_decode = [300, 1, 150, 70, 129], [4, 4, 2, 4, 1]
    seqs = [rng.integers(0, cfg["vocab_size"], size=p + d).tolist() for p, d in zip(prompt_lens, n_decode)]
    need = sum(-(-(p + d) // 64) * 64 for p, d in zip(prompt_lens, n_decode))
    eng = _engine(folder, "bfloat16", need)
    _, places, got = run_batch(eng, seqs, prompt_lens, n_decode, lambda p: sorted({0, p // 2, p - 1}))
    for i, q in enumerate(seqs):
        assert_close(plain.forward(q)[places[i]], got[i], BF16_REL, f"request {i} (prompt {prompt_lens[i]}, decoded {n_decode[i]})")
    assert eng.free_tokens() == eng.n_pages * 64, "pages were lost"
