"""The engine against the plain implementation: whole prompts, the last tokens
one by one, unequal batches one after another, long decoding, the first
tokens; in 32-bit and in bfloat16, on three tiny configurations that differ in
every size and option."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import BF16_REL, FP32_REL, TINY, assert_close, make_folder, prompts_for
from plain.model import PlainQwen3
from plain.sampler import PlainSampler, plain_generate

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CASES = [("A", "float32", torch.float32), ("A", "bfloat16", torch.bfloat16),
         ("B", "float32", torch.float32), ("B", "bfloat16", torch.bfloat16),
         ("C", "float32", torch.float32), ("C", "bfloat16", torch.bfloat16)]
IDS = [f"{n}-{d}" for n, d, _ in CASES]


def tol(dtype: str) -> float:
    return FP32_REL if dtype == "float32" else BF16_REL


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name, _, wdt in CASES:
        if (name, wdt) not in out:
            out[(name, wdt)] = make_folder(root, name, wdt)
    return out


@pytest.fixture(scope="module")
def plain_models(folders):
    return {key: PlainQwen3.from_folder(path) for key, path in folders.items()}


def _engine(folder, dtype, max_tokens, **kw):
    from mynah_slm_b200.engine.engine import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def _entry(slot, tokens, want):
    from mynah_slm_b200.engine.engine import StepEntry
    return StepEntry(slot, tokens, want)


@pytest.mark.parametrize("name,dtype,wdt", CASES, ids=IDS)
def test_whole_prompts_alone(folders, plain_models, name, dtype, wdt):
    eng = _engine(folders[(name, wdt)], dtype, 256)
    plain = plain_models[(name, wdt)]
    for toks in prompts_for(name, [1, 2, 17, 64, 65, 150]):
        slot = eng.open_sequence()
        got = eng.step([_entry(slot, toks, range(len(toks)))]).cpu().numpy()
        eng.check_status()
        eng.close_sequence(slot)
        assert_close(plain.forward(toks), got, tol(dtype), f"{name} {dtype} whole prompt of {len(toks)}")


@pytest.mark.parametrize("name,dtype,wdt", CASES, ids=IDS)
def test_last_32_tokens_one_by_one(folders, plain_models, name, dtype, wdt):
    eng = _engine(folders[(name, wdt)], dtype, 192)
    plain = plain_models[(name, wdt)]
    for n in (33, 100, 130):
        toks = prompts_for(name, [n], seed=n)[0]
        ref = plain.forward(toks)
        slot = eng.open_sequence()
        head = n - 32
        rows = [eng.step([_entry(slot, toks[:head], range(head))]).cpu().numpy()]
        for t in range(head, n):
            rows.append(eng.step([_entry(slot, toks[t:t + 1], (0,))]).cpu().numpy())
        eng.check_status()
        eng.close_sequence(slot)
        assert_close(ref, np.concatenate(rows), tol(dtype), f"{name} {dtype} {n} tokens, last 32 one by one")


@pytest.mark.parametrize("graphs", [True, False], ids=["graphs", "eager"])
@pytest.mark.parametrize("name,dtype,wdt", CASES, ids=IDS)
def test_unequal_batches_one_after_another(folders, plain_models, name, dtype, wdt, graphs):
    """Batches of unequal prompts; every request decodes a different number of
    tokens, so the shorter ones end earlier; the next batch starts in the slots
    and pages the first gave back. The cache is exactly as large as the
    largest batch needs."""
    plain = plain_models[(name, wdt)]
    rng = np.random.default_rng(5)
    V = TINY[name]["vocab_size"]
    batches = [[(7, 8), (1, 3), (12, 20)], [(1, 16), (5, 2), (33, 9), (64, 5)], [(70, 1), (3, 40)]]
    need = max(sum(-(-(p + d) // 64) * 64 for p, d in b) for b in batches)
    eng = _engine(folders[(name, wdt)], dtype, need, use_graphs=graphs)
    seen_slots = []
    for bi, batch in enumerate(batches):
        seqs = [rng.integers(0, V, size=p + d).tolist() for p, d in batch]
        slots = [eng.open_sequence() for _ in batch]
        seen_slots.append(set(slots))
        got = [[] for _ in batch]
        out = eng.step([_entry(s, q[:p], range(p)) for s, q, (p, d) in zip(slots, seqs, batch)]).cpu().numpy()
        row = 0
        for i, (p, d) in enumerate(batch):
            got[i].append(out[row:row + p]); row += p
        live = list(range(len(batch)))
        t = 0
        while live:
            live = [i for i in live if t < batch[i][1]]
            if not live:
                break
            out = eng.step([_entry(slots[i], [seqs[i][batch[i][0] + t]], (0,)) for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
            t += 1
            for i in list(live):
                if t >= batch[i][1]:
                    eng.close_sequence(slots[i])                    # ends earlier than the others
        eng.check_status()
        for i, q in enumerate(seqs):
            assert_close(plain.forward(q), np.concatenate(got[i]), tol(dtype),
                         f"{name} {dtype} batch {bi} request {i} (prompt {batch[i][0]}, decoded {batch[i][1]})")
    assert seen_slots[1] & seen_slots[0], "the second batch did not reuse a slot"
    assert eng.free_tokens() == eng.n_pages * 64, "pages were lost"


@pytest.mark.parametrize("name,dtype,wdt", [c for c in CASES if c[0] in ("A", "C")], ids=[i for i in IDS if i[0] in "AC"])
def test_long_decoding(folders, plain_models, name, dtype, wdt):
    """A short prompt and then hundreds of single steps: across page ends and,
    on C, far past the window of 40."""
    plain = plain_models[(name, wdt)]
    n = 240 if name == "A" else 330
    toks = prompts_for(name, [n], seed=77)[0]
    eng = _engine(folders[(name, wdt)], dtype, -(-n // 64) * 64)
    slot = eng.open_sequence()
    rows = [eng.step([_entry(slot, toks[:3], (0, 1, 2))]).cpu().numpy()]
    for t in range(3, n):
        rows.append(eng.step([_entry(slot, toks[t:t + 1], (0,))]).cpu().numpy())
    eng.check_status()
    assert_close(plain.forward(toks), np.concatenate(rows), tol(dtype), f"{name} {dtype} long decoding")
    if name == "C":
        # the windowed group has given back what left the window; the full group has not
        assert len(eng.cache.pages.held(slot, 0)[0]) == -(-n // 64)
        assert len(eng.cache.pages.held(slot, 1)[0]) <= 2


@pytest.mark.parametrize("name,dtype,wdt", CASES, ids=IDS)
def test_first_tokens_and_chunked_prompt(folders, plain_models, name, dtype, wdt):
    plain = plain_models[(name, wdt)]
    eng = _engine(folders[(name, wdt)], dtype, 256)
    toks = prompts_for(name, [90], seed=3)[0]
    ref = plain.forward(toks)
    # one token at a time from the very first
    slot = eng.open_sequence()
    rows = [eng.step([_entry(slot, toks[t:t + 1], (0,))]).cpu().numpy() for t in range(5)]
    assert_close(ref[:5], np.concatenate(rows), tol(dtype), f"{name} {dtype} first tokens")
    eng.close_sequence(slot)
    # a prompt cut into pieces of unequal size, beside a whole one in the same steps
    a, b = eng.open_sequence(), eng.open_sequence()
    cuts = [(0, 1), (1, 40), (40, 64), (64, 90)]
    got_a = []
    for i, (lo, hi) in enumerate(cuts):
        entries = [_entry(a, toks[lo:hi], range(hi - lo))]
        if i == 1:
            entries.append(_entry(b, toks, (len(toks) - 1,)))
        out = eng.step(entries).cpu().numpy()
        got_a.append(out[:hi - lo])
        if i == 1:
            assert_close(ref[-1:], out[hi - lo:], tol(dtype), f"{name} {dtype} whole prompt beside a piece")
    eng.check_status()
    assert_close(ref, np.concatenate(got_a), tol(dtype), f"{name} {dtype} prompt in pieces")
    # nothing wanted: the step still fills the cache
    eng.close_sequence(a)
    eng.close_sequence(b)
    c = eng.open_sequence()
    assert eng.step([_entry(c, toks[:50], ())]).shape == (0, TINY[name]["vocab_size"])
    out = eng.step([_entry(c, toks[50:51], (0,))]).cpu().numpy()
    assert_close(ref[50:51], out, tol(dtype), f"{name} {dtype} after a step that wanted nothing")


@pytest.mark.parametrize("name,dtype,wdt", [CASES[0], CASES[3], CASES[4]], ids=[IDS[0], IDS[3], IDS[4]])
def test_trace_run_program(folders, plain_models, tmp_path, name, dtype, wdt):
    """bin/trace_run as a user runs it: a process, JSON lines in, .f32 files out."""
    plain = plain_models[(name, wdt)]
    V = TINY[name]["vocab_size"]
    a, b = prompts_for(name, [70, 9], seed=21)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[60:61], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": []}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[61:62], "want": [0]}], "end": []},
        {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["a", "c"]},
    ]
    out = tmp_path / "out"
    env = dict(os.environ, HOME=str(tmp_path / "home"))
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[(name, wdt)], "--dtype", dtype,
                        "--out", str(out), "--max-tokens", "192"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    ra, rb = plain.forward(a), plain.forward(b)
    load = lambda i: np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
    assert_close(np.stack([ra[0], ra[59], rb[7]]), load(0), tol(dtype), "trace step 0")
    assert_close(ra[60:61], load(1), tol(dtype), "trace step 1")
    assert_close(ra[61:62], load(2), tol(dtype), "trace step 2")
    assert_close(rb[8:9], load(3), tol(dtype), "trace step 3")


@pytest.mark.parametrize("name", ["B", "C", "D", "E"])
def test_prompt_steps_replayed_from_graphs(tmp_path, name):
    """A prompt step's shape is captured the second time it comes and replayed from then on, with rows,
    sequences and wanted rows padded to the graph's capacities. Batches of different prompts and lengths that
    share a padded shape go through the same graph; every logit row is compared with the plain implementation,
    and slots and pages are used again in between."""
    folder = make_folder(tmp_path, name, torch.bfloat16)       # D and E take the tensor-core attention kernels
    eng = _engine(folder, "bfloat16", 1024)
    plain = PlainQwen3.from_folder(folder)
    assert eng.use_graphs and eng.graph_safe
    for rnd, lens in enumerate([[40, 7, 70], [33, 20, 75], [1, 64, 37], [60, 60, 8], [150], [129], [140]]):
        prompts = prompts_for(name, lens, seed=40 + rnd)
        slots = [eng.open_sequence() for _ in prompts]
        wants = [(0, n - 1) if n > 1 else (0,) for n in lens]
        got = eng.step([_entry(s, p, w) for s, p, w in zip(slots, prompts, wants)]).cpu().numpy()
        eng.check_status()
        row = 0
        for p, w in zip(prompts, wants):
            ref = plain.forward(p)
            for j in w:
                assert_close(ref[j:j + 1], got[row:row + 1], BF16_REL, f"round {rnd}, prompt of {len(p)}, place {j}")
                row += 1
        # one decoded token each on top of what the replayed step wrote into the cache
        nxt = [int(np.argmax(plain.forward(p)[-1])) for p in prompts]
        got = eng.step([_entry(s, [t], (0,)) for s, t in zip(slots, nxt)]).cpu().numpy()
        for b, (p, t) in enumerate(zip(prompts, nxt)):
            assert_close(plain.forward(p + [t])[-1:], got[b:b + 1], BF16_REL, f"round {rnd}, decode after prompt {b}")
        for s in slots:
            eng.close_sequence(s)
    captured = [g for g in eng._prompt_graphs.values() if g.graph is not None]
    assert len(captured) >= 2, "the repeated shapes were not captured"


@pytest.mark.parametrize("name,window", [("D", None), ("E", 700)])
def test_a_long_context(tmp_path, name, window):
    """2,300 positions: a prompt step of 18 key tiles (in one piece, and a second sequence in two pieces), then
    decode steps over 36 and more pages, with a window whose edge lies far back; against the plain
    implementation at the positions where a fault of a far tile or page would show."""
    cfg = dict(TINY[name], max_position_embeddings=4096)
    if window is not None:
        cfg["sliding_window"] = window
    folder = make_folder(tmp_path, name, torch.bfloat16, config=cfg)
    plain = PlainQwen3.from_folder(folder)
    rng = np.random.default_rng(77)
    n = 2300
    toks = rng.integers(0, cfg["vocab_size"], size=n + 3).tolist()
    ref = plain.forward(toks)                                          # [n + 3, V], whole sequence, no cache
    eng = _engine(folder, "bfloat16", 3 * 2560)
    a, b = eng.open_sequence(), eng.open_sequence()
    places = (0, 63, 64, 127, 128, 1000, 2047, 2048, n - 1)
    got = eng.step([_entry(a, toks[:n], places)]).cpu().numpy()
    eng.check_status()
    for i, j in enumerate(places):
        assert_close(ref[j:j + 1], got[i:i + 1], BF16_REL, f"whole prompt, place {j}")
    eng.step([_entry(b, toks[:1111], ())])                             # the same prompt in two pieces
    got_b = eng.step([_entry(b, toks[1111:n], (n - 1111 - 1,))]).cpu().numpy()
    assert_close(ref[n - 1:n], got_b, BF16_REL, "prompt in two pieces")
    for t in range(3):                                                 # both sequences decode together
        got = eng.step([_entry(a, [toks[n + t]], (0,)), _entry(b, [toks[n + t]], (0,))]).cpu().numpy()
        eng.check_status()
        assert_close(ref[n + t:n + t + 1], got[0:1], BF16_REL, f"decode step {t}")
        assert_close(ref[n + t:n + t + 1], got[1:2], BF16_REL, f"decode step {t}, the sequence that came in pieces")


def test_layers_of_the_benchmark_shape(tmp_path):
    """Two layers with the layer sizes of the measured configuration (width 1,024, 16 query heads over 8 kv heads
    of 128, feed-forward 3,072; a small odd vocabulary keeps the plain implementation quick): the prompt-step
    products run as pairs of CTAs, with K in two halves and with the fused activation, the prompt attention has 17
    key tiles, decode steps read 33 pages. A prompt of 2,100 tokens alone, a ragged batch of two more, then all
    three token by token, against the plain implementation."""
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=1024,
               num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=4099,
               rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096,
               hidden_act="silu", attention_bias=False, rope_scaling=None, use_sliding_window=False, sliding_window=None,
               max_window_layers=2, eos_token_id=1)
    folder = make_folder(tmp_path, "shape", torch.bfloat16, config=cfg, seed=5)
    plain = PlainQwen3.from_folder(folder)
    eng = _engine(folder, "bfloat16", 64 * 80)
    rng = np.random.default_rng(123)
    lens = [2100, 700, 1300]
    seqs = [rng.integers(0, cfg["vocab_size"], size=n + 3).tolist() for n in lens]
    refs = [plain.forward(s) for s in seqs]
    slots = [eng.open_sequence() for _ in seqs]
    places = (0, 127, 128, 1000, 2047, 2048, lens[0] - 1)
    got = eng.step([_entry(slots[0], seqs[0][:lens[0]], places)]).cpu().numpy()
    eng.check_status()
    for i, j in enumerate(places):
        assert_close(refs[0][j:j + 1], got[i:i + 1], BF16_REL, f"prompt of {lens[0]}, place {j}")
    got = eng.step([_entry(slots[1], seqs[1][:lens[1]], (0, 255, lens[1] - 1)),
                    _entry(slots[2], seqs[2][:lens[2]], (63, 64, lens[2] - 1))]).cpu().numpy()
    eng.check_status()
    for r, (i, j) in enumerate([(1, 0), (1, 255), (1, lens[1] - 1), (2, 63), (2, 64), (2, lens[2] - 1)]):
        assert_close(refs[i][j:j + 1], got[r:r + 1], BF16_REL, f"ragged batch, sequence {i}, place {j}")
    for t in range(3):
        got = eng.step([_entry(s, [q[n + t]], (0,)) for s, q, n in zip(slots, seqs, lens)]).cpu().numpy()
        eng.check_status()
        for i, n in enumerate(lens):
            assert_close(refs[i][n + t:n + t + 1], got[i:i + 1], BF16_REL, f"decode step {t}, sequence {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "E"])
def test_a_prompt_piece_far_behind_a_short_window(tmp_path, name, dtype):
    """Windows of 40 positions and pages of 64: when a prompt goes on in pieces, the windowed layers have given
    back whole pages before the piece's first key tile ends, so a tile's first page may not exist any more. Pieces
    that start at many offsets of a page and of a key tile, against the plain implementation."""
    wdt = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_folder(tmp_path, name, wdt)
    plain = PlainQwen3.from_folder(folder)
    eng = _engine(folder, dtype, 64 * 16)
    rng = np.random.default_rng(91)
    for cuts in ([0, 150, 230], [0, 104, 105, 300], [0, 64, 128, 192, 256, 320], [0, 200, 201, 264, 330], [0, 127, 171, 340]):
        n = cuts[-1]
        toks = rng.integers(0, TINY[name]["vocab_size"], size=n).tolist()
        ref = plain.forward(toks)
        slot = eng.open_sequence()
        got = [eng.step([_entry(slot, toks[lo:hi], range(hi - lo))]).cpu().numpy() for lo, hi in zip(cuts[:-1], cuts[1:])]
        eng.check_status()
        eng.close_sequence(slot)
        assert_close(ref, np.concatenate(got), tol(dtype), f"{name} {dtype} pieces at {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_padding_and_company_change_nothing(folders, dtype):
    """A decode step's logits for one sequence have the same bits whether its
    rows are padding or other sequences and whichever row it takes. In 32-bit
    this holds across batch sizes too (every sum has a fixed order); in
    bfloat16 the library's matrix product may pick another kernel for another
    batch size, so across sizes the comparison is to rounding."""
    eng = _engine(folders[("B", torch.bfloat16)], dtype, 1024)
    p = prompts_for("B", [20, 31, 5, 9, 14], seed=8)

    def run(which):
        slots = {i: eng.open_sequence() for i in which}
        eng.step([_entry(slots[i], p[i], ()) for i in which])
        out = eng.step([_entry(slots[i], [p[i][0]], (0,)) for i in which]).cpu().numpy()
        for s in slots.values():
            eng.close_sequence(s)
        return {i: out[r] for r, i in enumerate(which)}
    three = run([0, 1, 2])                    # a bucket of 4 with one padding row
    four = run([3, 2, 1, 0])                  # the same bucket, full, other rows
    assert np.array_equal(three[1], four[1]) and np.array_equal(three[2], four[2]) and np.array_equal(three[0], four[0])
    alone, five = run([1]), run([4, 3, 2, 1, 0])
    if dtype == "float32":
        assert np.array_equal(alone[1], three[1]) and np.array_equal(alone[1], five[1])
    else:
        assert_close(alone[1][None], three[1][None], 1e-2, "alone against a batch of three")
        assert_close(alone[1][None], five[1][None], 1e-2, "alone against a batch of five")


def test_step_refuses_bad_input(folders):
    from mynah_slm_b200.cache.pages import CacheError
    from mynah_slm_b200.engine.engine import EngineError
    eng = _engine(folders[("A", torch.float32)], "float32", 128)
    s = eng.open_sequence()
    with pytest.raises(EngineError, match="outside the vocabulary"):
        eng.step([_entry(s, [512], (0,))])
    with pytest.raises(EngineError, match="wanted place"):
        eng.step([_entry(s, [1, 2], (2,))])
    with pytest.raises(EngineError, match="not open"):
        eng.step([_entry(99, [1], (0,))])
    with pytest.raises(EngineError, match="twice"):
        eng.step([_entry(s, [1], ()), _entry(s, [2], ())])
    with pytest.raises(EngineError, match="the model allows 256"):
        eng.step([_entry(s, [1] * 257, ())])
    with pytest.raises(CacheError, match="full"):
        eng.step([_entry(s, [1] * 129, ())])
    assert eng.length(s) == 0                                    # nothing was taken by the refused steps
    eng.step([_entry(s, [1] * 128, ())])


@pytest.mark.parametrize("name,dtype,wdt", [CASES[0], CASES[2], CASES[5]], ids=[IDS[0], IDS[2], IDS[5]])
def test_greedy_generation_through_the_entry_point(folders, plain_models, name, dtype, wdt):
    from mynah_slm_b200 import LLM
    plain = plain_models[(name, wdt)]
    llm = LLM(folders[(name, wdt)], dtype=dtype, max_tokens=64 * 8)
    prompts = prompts_for(name, [7, 1, 12, 30, 3], seed=31)
    n_new = [8, 5, 12, 3, 9]
    res = []
    for batch in (2, 8):                                         # two batches after one another, and one
        # each distinct limit is its own call
        outs = {}
        for m in sorted(set(n_new)):
            idx = [i for i, k in enumerate(n_new) if k == m]
            r = llm.generate([prompts[i] for i in idx], max_new=m, temp=0.0, ignore_eos=True, max_batch=batch)
            for i, x in zip(idx, r):
                outs[i] = x
        res.append([outs[i].tokens for i in range(len(prompts))])
    assert res[0] == res[1]
    if dtype == "float32":
        for i, p in enumerate(prompts):
            want, _ = plain_generate(plain, p, n_new[i], PlainSampler(temp=0))
            assert res[0][i] == want, f"request {i}"
    # the model's own stop set ends a sequence before the stop token is emitted
    p0 = prompts[2]
    free = llm.generate([p0], max_new=12, temp=0.0, ignore_eos=True)[0].tokens
    stop_at = next((j for j in range(1, len(free)) if free[j] not in free[:j]), 0)
    r = llm.generate([p0], max_new=12, temp=0.0, stop_ids=[free[stop_at]])[0]
    assert r.tokens == free[:stop_at] and r.produced == stop_at + 1 and r.finish_reason == "stop"
    assert llm.last_timing.n_gen == stop_at + 1 and "decode" in llm.last_timing.format()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_without_the_host_in_between(folders, dtype):
    """`decode_loop` (K sampled steps with the token fed back on the device, what the measurement times) against
    the same K steps through the host: the same tokens, and the same cache afterwards."""
    from mynah_slm_b200.sampling.sampler import SamplingParams
    prompts = prompts_for("B", [40, 3, 65], seed=9)
    K = 9
    lasts, afters = [], []
    for through_host in (False, True):
        eng = _engine(folders[("B", torch.bfloat16)], dtype, 64 * 8)
        eng.sampler.set_params(SamplingParams(temp=0.0))
        slots = [eng.open_sequence() for _ in prompts]
        logits = eng.step([_entry(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)])
        toks = logits.argmax(dim=-1).cpu().tolist()
        if through_host:
            for _ in range(K):
                toks = eng.decode_sampled(slots, toks)[:len(slots)].cpu().tolist()
        else:
            toks = eng.decode_loop(slots, toks, K)[:len(slots)].cpu().tolist()
        eng.check_status()
        lasts.append(toks)
        afters.append(eng.step([_entry(s, [t], (0,)) for s, t in zip(slots, toks)]).cpu())
    assert lasts[0] == lasts[1]
    assert torch.equal(afters[0], afters[1])


def test_temperature_generation_matches_plain_in_32_bit(folders, plain_models):
    """Temperature 0.8, seed 1, on B in 32-bit: token for token what the plain
    sampler draws from the plain model, whatever the batch."""
    from mynah_slm_b200 import LLM
    from mynah_slm_b200.sampling.sampler import stream_state
    key = ("B", torch.bfloat16)
    llm = LLM(folders[key], dtype="float32", max_tokens=64 * 8)
    prompts = prompts_for("B", [1, 5, 33, 64], seed=41)
    kw = dict(max_new=16, temp=0.8, top_k=0, top_p=1.0, seed=1, ignore_eos=True)
    together = [r.tokens for r in llm.generate(prompts, **kw)]
    apart = [r.tokens for r in llm.generate(prompts, max_batch=1, **kw)]
    assert together == apart                                       # a sequence's draws do not depend on its batch
    for i, p in enumerate(prompts):
        s = PlainSampler(temp=0.8, top_k=0, top_p=1.0, rng_state=stream_state(1, i))
        want, _ = plain_generate(plain_models[key], p, 16, s)
        assert together[i] == want, f"request {i}"
    # the reference's defaults (top-k 20, top-p 0.95) and the penalties
    kw = dict(max_new=10, temp=0.6, top_k=20, top_p=0.95, seed=7, repeat_penalty=1.2, ignore_eos=True)
    got = llm.generate(prompts[:2], **kw)
    for i, p in enumerate(prompts[:2]):
        s = PlainSampler(temp=0.6, top_k=20, top_p=0.95, repeat_penalty=1.2, rng_state=stream_state(7, i))
        want, _ = plain_generate(plain_models[key], p, 10, s)
        assert got[i].tokens == want, f"request {i} with filters and penalty"


def test_command_line(folders, tmp_path):
    folder = folders[("A", torch.float32)]
    cli = [sys.executable, os.path.join(ROOT, "bin", "mynah-slm")]
    p = subprocess.run(cli + ["run", "-m", folder, "--tokens", "5,17,3", "--tokens", "9", "-n", "6", "--temp", "0",
                              "--dtype", "float32", "--ignore-eos"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l.split() for l in p.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(l) == 6 for l in lines)
    assert "prefill" in p.stderr and "decode" in p.stderr and "TTFT" in p.stderr
    q = subprocess.run(cli + ["run", "-m", folder, "--tokens", "5,17,3", "-n", "6", "--temp", "0", "--dtype", "float32",
                              "--ignore-eos", "--quiet"], capture_output=True, text=True, timeout=600)
    assert q.returncode == 0 and q.stdout.split() == lines[0] and "prefill" not in q.stderr
    # a model made from a configuration and a seed, with no folder; and the prompts' logits written beside
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY["A"]))
    npy = tmp_path / "logits.npy"
    r = subprocess.run(cli + ["run", "--random", str(cfg_path), "--weights-seed", "0", "--tokens", "5,17,3", "--tokens", "9",
                              "-n", "6", "--temp", "0", "--dtype", "float32", "--ignore-eos", "--quiet",
                              "--logits-out", str(npy)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l.split() for l in r.stdout.strip().splitlines()] == lines      # the folder was written from seed 0 too
    from plain.model import PlainQwen3
    plain = PlainQwen3.from_folder(folder)
    assert_close(np.concatenate([plain.forward([5, 17, 3]), plain.forward([9])]), np.load(npy), FP32_REL, "--logits-out")
    both = subprocess.run(cli + ["run", "-m", folder, "--random", str(cfg_path), "--tokens", "1"], capture_output=True, text=True)
    assert both.returncode == 2 and "one of them" in both.stderr
    bad = subprocess.run(cli + ["run", "-m", folder, "--bogus"], capture_output=True, text=True)
    assert bad.returncode == 2 and "unknown option '--bogus'" in bad.stderr
    assert subprocess.run(cli + ["--version"], capture_output=True, text=True).stdout.strip()


def test_a_reused_slot_starts_with_an_empty_ring(folders):
    """Penalties look at the ring of a slot's recent tokens. A sequence that opens in a slot another sequence
    has just left must not see that sequence's tokens: driven through the engine alone (no generation loop), the
    second user of a slot samples what the first user of a fresh engine's slot samples."""
    from mynah_slm_b200.sampling.sampler import SamplingParams
    params = SamplingParams(temp=0.0, repeat_penalty=5.0, presence_penalty=2.0, freq_penalty=1.0)
    other, mine = prompts_for("A", [9, 6], seed=12)

    def decode(eng, slot, prompt, n):
        tok = int(eng.step([_entry(slot, prompt, (len(prompt) - 1,))]).argmax(dim=-1).item())
        out = []
        for _ in range(n):
            tok = int(eng.decode_sampled([slot], [tok])[:1].cpu().item())
            out.append(tok)
        eng.check_status()
        return out

    fresh = _engine(folders[("A", torch.float32)], "float32", 128)
    fresh.sampler.set_params(params)
    want = decode(fresh, fresh.open_sequence(), mine, 12)
    plain_greedy = _engine(folders[("A", torch.float32)], "float32", 128)
    s0 = plain_greedy.open_sequence()
    assert decode(plain_greedy, s0, mine, 12) != want, "the penalties change nothing here: the test shows nothing"
    eng = _engine(folders[("A", torch.float32)], "float32", 128)
    eng.sampler.set_params(params)
    first = eng.open_sequence()
    decode(eng, first, other, 20)                       # fills the slot's ring
    eng.close_sequence(first)
    again = eng.open_sequence()
    assert again == first
    assert decode(eng, again, mine, 12) == want


def test_a_wait_that_runs_out_is_reported_and_the_engine_goes_on(folders, plain_models):
    """Status bit 16: a bounded wait inside a kernel ran out. The wait here is a probe kernel's (a word of global
    memory that nothing sets, a limit of 50 microseconds): it sets the bit in the product kernel's status word and
    returns; `check_status` raises with the reason, clears the word, resets the product kernel's flags, and the next
    steps give the right logits."""
    from mynah_slm_b200.engine.engine import EngineError
    from mynah_slm_b200.ops import gemm_bf16
    from mynah_slm_b200.ops.lib import call, ptr, stream_ptr
    key = ("B", torch.bfloat16)
    eng = _engine(folders[key], "bfloat16", 256)
    toks = prompts_for("B", [40], seed=2)[0]
    slot = eng.open_sequence()
    eng.step([_entry(slot, toks[:30], ())])
    eng.check_status()                                            # nothing to report
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    call("mynah_wait_probe", ptr(flag), ptr(gemm_bf16.status_word(eng.device)), 50_000, stream_ptr())
    with pytest.raises(EngineError, match="a bounded wait inside a kernel ran out"):
        eng.check_status()
    eng.check_status()                                            # cleared
    got = eng.step([_entry(slot, toks[30:], range(10))]).cpu().numpy()
    eng.check_status()
    assert_close(plain_models[key].forward(toks)[30:], got, BF16_REL, "steps after a reported timeout")
    # a flag that is set ends the wait without a report
    flag.fill_(1)
    call("mynah_wait_probe", ptr(flag), ptr(gemm_bf16.status_word(eng.device)), 50_000, stream_ptr())
    eng.check_status()
