"""The plain implementation itself (no GPU): against the reference's own numpy
model code (golden outputs under tests/golden/), and the properties the
reference tests its kernels for (mynah-slm tests/test_kernels.c:42-264)."""
import os
import sys

import numpy as np
import pytest

from helpers import rel_err
from plain.model import (PlainQwen3, gqa_attention, rms_norm, rope_apply, rope_table, softmax_rows, stable_sigmoid,
                         swiglu)
from plain.sampler import PlainSampler, SplitMix64, plain_generate

GOLD = os.path.join(os.path.dirname(__file__), "golden")
sys.path.insert(0, GOLD)
from golden_common import CONFIGS, build  # noqa: E402


@pytest.mark.parametrize("name", ["A", "B"])
def test_matches_reference_oracle(name):
    gold = np.load(os.path.join(GOLD, "oracle_logits.npz"))
    c, tensors, tokens = build(name)
    assert np.array_equal(tokens, gold[f"{name}_tokens"])
    model = PlainQwen3(dict(c), tensors)
    taps = {}
    logits = model.forward(tokens, taps)
    # the oracle computes in float32 throughout; the plain implementation keeps double sums
    assert rel_err(gold[f"{name}_layer0"], taps["layer0"]) < 2e-6
    assert rel_err(gold[f"{name}_logits"], logits) < 5e-6
    assert np.array_equal(gold[f"{name}_logits"].argmax(-1), logits.argmax(-1))


def test_gate_rejects_wrong_models():
    """The comparison must be able to fail: interleaved rotation, no per-head
    norm and a derived head_dim all have to show (tools/eval/test_gate.py:96-110)."""
    import plain.model as pm
    gold = np.load(os.path.join(GOLD, "oracle_logits.npz"))
    c, tensors, tokens = build("A")
    ref = gold["A_logits"]

    ones = {k: (np.ones_like(v) if k.endswith(("q_norm.weight", "k_norm.weight")) else v) for k, v in tensors.items()}
    assert rel_err(ref, PlainQwen3(dict(c), ones).forward(tokens)) > 1e-3

    orig = pm.rope_apply

    def interleaved(x, cos, sin):
        a, b = x[..., 0::2], x[..., 1::2]
        c_, s_ = cos[:, None, :], sin[:, None, :]
        out = np.empty_like(x)
        out[..., 0::2] = a * c_ - b * s_
        out[..., 1::2] = b * c_ + a * s_
        return out
    pm.rope_apply = interleaved
    try:
        assert rel_err(ref, PlainQwen3(dict(c), tensors).forward(tokens)) > 1e-3
    finally:
        pm.rope_apply = orig

    # a residual stream kept in 16 bits (tools/eval/test_gate.py:106-109)
    real = pm.rms_norm
    pm.rms_norm = lambda x, w, eps: real(x.astype(np.float16).astype(np.float32), w, eps)
    try:
        assert rel_err(ref, PlainQwen3(dict(c), tensors).forward(tokens)) > 1e-4
    finally:
        pm.rms_norm = real

    # head_dim derived as hidden / heads instead of read from its own key (tests/test_model.c:99-113: "128, not
    # d_model/n_heads"): on B, whose heads are 32 wide while hidden / heads is 16, such a model cannot even be
    # put together, or gives other logits
    cb, tb, tokb = build("B")
    derived = dict(cb, head_dim=cb["hidden_size"] // cb["num_attention_heads"])
    assert derived["head_dim"] != cb["head_dim"]
    try:
        wrong = PlainQwen3(derived, tb).forward(tokb)
        shows = wrong.shape != gold["B_logits"].shape or rel_err(gold["B_logits"], wrong) > 1e-3
    except (ValueError, IndexError):
        shows = True
    assert shows


def test_rms_norm_properties():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 64)).astype(np.float32) * 7
    w = np.ones(64, dtype=np.float32)
    y = rms_norm(x, w, 1e-6)
    assert np.allclose(np.sqrt((y.astype(np.float64) ** 2).mean(-1)), 1.0, atol=1e-5)        # unit RMS
    assert np.allclose(rms_norm(x * 1000, w, 1e-12), rms_norm(x, w, 1e-12), rtol=1e-5, atol=1e-6)  # scale-invariant
    g = rng.standard_normal(64).astype(np.float32)
    assert np.allclose(rms_norm(x, g, 1e-6), y * g, rtol=1e-6, atol=1e-7)                    # a plain gain, not 1+w
    assert np.allclose(rms_norm(x, np.zeros(64, np.float32), 1e-6), 0.0)
    # per head: each head is normalised on its own
    q = rng.standard_normal((3, 4, 16)).astype(np.float32)
    q2 = q.copy(); q2[:, 1] *= 50
    n1, n2 = rms_norm(q, np.ones(16, np.float32), 1e-6), rms_norm(q2, np.ones(16, np.float32), 1e-6)
    assert np.allclose(n1[:, 0], n2[:, 0]) and np.allclose(n1[:, 1], n2[:, 1], atol=1e-5)


def test_rope_properties():
    hd = 16
    pos = np.arange(9)
    cos, sin = rope_table(hd, pos, 10000.0)
    x = np.zeros((9, 1, hd), dtype=np.float32); x[:, 0, 0] = 1.0
    y = rope_apply(x, cos, sin)
    assert np.allclose(y[0], x[0])                                      # position 0 is the identity
    nz = np.nonzero(np.abs(y[3, 0]) > 1e-9)[0].tolist()
    assert nz == [0, hd // 2]                                           # split-half: 0 pairs with 8, not with 1
    rng = np.random.default_rng(1)
    q = rng.standard_normal((9, 2, hd)).astype(np.float32)
    assert np.allclose(np.linalg.norm(rope_apply(q, cos, sin), axis=-1), np.linalg.norm(q, axis=-1), rtol=1e-5)
    # relative distance: <R(p)q, R(p+d)k> depends on d only
    a, b = rng.standard_normal(hd).astype(np.float32), rng.standard_normal(hd).astype(np.float32)
    def dot_at(p, d):
        c2, s2 = rope_table(hd, np.array([p, p + d]), 10000.0)
        r = rope_apply(np.stack([a, b])[:, None, :], c2, s2)
        return float(r[0, 0] @ r[1, 0])
    assert abs(dot_at(0, 3) - dot_at(40, 3)) < 1e-4


def test_activations_are_stable():
    x = np.array([-1e5, -100.0, -1.0, 0.0, 1.0, 100.0, 1e5], dtype=np.float32)
    s = stable_sigmoid(x)
    assert np.all(np.isfinite(s)) and s[0] == 0.0 and s[-1] == 1.0 and s[3] == 0.5
    assert np.all(np.isfinite(swiglu(x, x)))
    p = softmax_rows(np.array([[1000.0, 1000.0, 999.0]], dtype=np.float32))
    assert np.isfinite(p).all() and abs(p.sum() - 1) < 1e-6 and p[0, 0] == p[0, 1]


def test_attention_properties():
    rng = np.random.default_rng(2)
    T, H, KV, HD = 6, 4, 2, 8
    q = rng.standard_normal((T, H, HD)).astype(np.float32)
    k = rng.standard_normal((T, KV, HD)).astype(np.float32)
    v = rng.standard_normal((T, KV, HD)).astype(np.float32)
    out = gqa_attention(q, k, v)
    assert np.allclose(out[0, 0], v[0, 0], atol=1e-6) and np.allclose(out[0, 3], v[0, 1], atol=1e-6)   # one key: v itself
    q2 = q.copy(); q2[:, 1] = q2[:, 0]
    o2 = gqa_attention(q2, k, v)
    assert np.allclose(o2[:, 0], o2[:, 1])                              # grouped heads share K and V
    k3, v3 = k.copy(), v.copy(); k3[4:] = 1e9; v3[4:] = 1e30
    assert np.allclose(gqa_attention(q, k3, v3)[:4], out[:4])           # earlier positions ignore later tokens
    lo, hi = v[:3, 0].min(0), v[:3, 0].max(0)
    assert np.all(out[2, 0] >= lo - 1e-6) and np.all(out[2, 0] <= hi + 1e-6)   # a convex combination
    w = gqa_attention(q, k, v, window=2)
    assert np.allclose(w[:2], out[:2]) and not np.allclose(w[4], out[4])
    assert np.allclose(w[5, 0], gqa_attention(q[5:6], k[4:6], v[4:6], q_pos=[5], k_pos=[4, 5])[0, 0], atol=1e-6)


def test_splitmix_and_sampler():
    r = SplitMix64(0x853C49E6748FEA9B)
    u = [r.next_uniform() for _ in range(1000)]
    assert all(0.0 <= x < 1.0 for x in u) and 0.45 < sum(u) / len(u) < 0.55
    logits = np.array([0.1, 2.0, 2.0, -1.0, 0.5], dtype=np.float32)
    assert PlainSampler(temp=0).sample(logits.copy()) == 1              # first maximum wins
    # top_k=1 is greedy whatever the draw
    assert PlainSampler(temp=1.0, top_k=1, top_p=1.0).sample(logits.copy()) == 1
    # top-p below the best token's own probability still keeps that token
    assert PlainSampler(temp=0.05, top_k=0, top_p=0.01, seed=3).sample(np.array([5.0, 1.0, 0.0], np.float32)) == 0
    # min-p removes everything far below the best
    s = PlainSampler(temp=1.0, top_k=0, top_p=1.0, min_p=0.5, seed=5)
    draws = {s.sample(np.array([3.0, 2.9, 0.0, -2.0], np.float32)) for _ in range(200)}
    assert draws == {0, 1}
    # the draw follows the distribution
    s = PlainSampler(temp=1.0, top_k=0, top_p=1.0, seed=7)
    lg = np.log(np.array([0.7, 0.2, 0.1], dtype=np.float32))
    counts = np.bincount([s.sample(lg.copy()) for _ in range(4000)], minlength=3) / 4000
    assert np.allclose(counts, [0.7, 0.2, 0.1], atol=0.03)


def test_penalties():
    s = PlainSampler(temp=0, repeat_penalty=2.0, freq_penalty=0.5, presence_penalty=0.25, penalty_window=4)
    for t in (1, 2, 1):
        s.accept(t)
    lg = np.array([0.0, 4.0, -2.0, 1.0], dtype=np.float32)
    s.apply_penalties(lg)
    # token 1 sits twice in the ring and is penalised once per entry, each time with count 2
    t1 = (4.0 / 2 - 0.5 * 2 - 0.25); t1 = (t1 / 2 - 0.5 * 2 - 0.25)
    assert lg[1] == pytest.approx(t1) and lg[2] == pytest.approx(-2.0 * 2 - 0.5 - 0.25) and lg[3] == 1.0
    for t in (3, 3, 3, 3):
        s.accept(t)                                                      # the ring holds only the window
    assert s.n_recent == 4 and sorted(s.recent) == [3, 3, 3, 3]


def test_plain_generate_stops_before_emitting():
    c, tensors, tokens = build("A")
    model = PlainQwen3(dict(c), tensors)
    out, produced = plain_generate(model, tokens[:5].tolist(), 6, PlainSampler(temp=0))
    assert len(out) == 6 and produced == 6
    j = next((i for i in range(len(out)) if out[i] not in out[:i] and i > 0), 0)
    out2, produced2 = plain_generate(model, tokens[:5].tolist(), 6, PlainSampler(temp=0), eos={out[j]})
    assert out2 == out[:j] and produced2 == j + 1
