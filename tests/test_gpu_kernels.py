"""Each kernel alone against its plain reference, at sizes other than the
engine's tiny models (widths and vocabularies that are no power of two, head
sizes in steps of 16, odd numbers of heads and groups)."""
import numpy as np
import pytest
import torch

from helpers import rel_err
from plain.model import gqa_attention, rms_norm, rope_apply, rope_table, swiglu as plain_swiglu
from plain.sampler import PlainSampler

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"f32": torch.float32, "bf16": torch.bfloat16}


def _k():
    from mynah_slm_b200.ops import kernels
    return kernels


def _tol(dt):
    return 2e-6 if dt == "f32" else 8e-3


def _round(a: np.ndarray, dt: str) -> np.ndarray:
    """What the values are after being stored in the run's type."""
    if dt == "f32":
        return a.astype(np.float32)
    return torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16).float().numpy()


def test_library_is_ours_and_loaded():
    from mynah_slm_b200.ops import lib
    handle = lib.load()
    assert handle.mynah_device_arch() == 100
    maps = open("/proc/self/maps").read()
    assert "libmynah_slm_b200.so" in maps


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("V,D,T", [(777, 100, 13), (1000, 1024, 3)])
def test_embed_gather(dt, V, D, T):
    k = _k()
    rng = np.random.default_rng(0)
    table = torch.from_numpy(rng.standard_normal((V, D)).astype(np.float32)).to(DT[dt]).to(DEV)
    toks = torch.from_numpy(rng.integers(0, V, size=T).astype(np.int32)).to(DEV)
    x = k.embed_gather(table, toks)
    assert x.dtype == torch.float32
    assert torch.equal(x, table.float()[toks.long()])          # a lookup: exact, no scaling


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("T,D,eps", [(7, 100, 1e-5), (3, 1000, 1e-6), (5, 4096, 1e-6), (2, 24, 1e-3)])
def test_rmsnorm_with_residual_and_rows(dt, T, D, eps):
    k = _k()
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((T, D)) * 30).astype(np.float32)
    delta = _round(rng.standard_normal((T, D)), dt)
    gain = _round(1 + 0.1 * rng.standard_normal(D), dt)
    xd = torch.from_numpy(x.copy()).to(DEV)
    out = k.rmsnorm(xd, torch.from_numpy(gain).to(DT[dt]).to(DEV), eps, DT[dt],
                    delta=torch.from_numpy(delta).to(DT[dt]).to(DEV))
    assert np.array_equal(xd.cpu().numpy(), (x + delta).astype(np.float32))           # the add is exact fp32
    ref = rms_norm(x + delta, gain, eps)
    assert rel_err(ref, out.float().cpu().numpy()) < _tol(dt)
    # a selection of rows, no add
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    out2 = k.rmsnorm(xd, torch.from_numpy(gain).to(DT[dt]).to(DEV), eps, DT[dt], rows=rows)
    assert torch.equal(out2, out[[T - 1, 0]])
    # a selection that names a row many times, with the add: every copy is the same, and x is only read
    # (CTAs that each added delta to the same row in place would add it several times)
    xe = torch.from_numpy(x.copy()).to(DEV)
    many = torch.tensor([0] * 40 + [T - 1] + [0] * 23, dtype=torch.int32, device=DEV)
    out4 = k.rmsnorm(xe, torch.from_numpy(gain).to(DT[dt]).to(DEV), eps, DT[dt],
                     delta=torch.from_numpy(delta).to(DT[dt]).to(DEV), rows=many)
    assert torch.equal(out4, out[many.long()]) and np.array_equal(xe.cpu().numpy(), x)
    # a gain stored in 32-bit stays 32-bit in a bf16 run
    g32 = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    out3 = k.rmsnorm(xd, torch.from_numpy(g32).to(DEV), eps, DT[dt])
    assert rel_err(rms_norm(x + delta, g32, eps), out3.float().cpu().numpy()) < _tol(dt)


@pytest.mark.parametrize("D", [1024, 4096, 5000])
def test_rmsnorm_of_rows_with_massive_channels(D):
    """The reference sums the squares in double because the residual stream of the real model has a few channels
    near 1e4 among values near 1 (mynah-slm src/kernels.c:116-123). Rows of that kind, in 32-bit, against a
    float64 norm: the small channels must not be lost in the sum."""
    k = _k()
    rng = np.random.default_rng(D)
    x = rng.standard_normal((6, D)).astype(np.float32)
    x[:, 7] = 8.0e3
    x[1::2, D - 3] = -1.2e4
    x[4] = rng.standard_normal(D).astype(np.float32) * 1e-3            # and a row of small values only
    gain = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    for eps in (1e-6, 1e-5):
        out = k.rmsnorm(torch.from_numpy(x.copy()).to(DEV), torch.from_numpy(gain).to(DEV), eps, torch.float32).cpu().numpy()
        x64 = x.astype(np.float64)
        ref = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + np.float64(np.float32(eps))) * gain.astype(np.float64)
        assert rel_err(ref.astype(np.float32), out) < 1e-6, (D, eps)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_swiglu_and_residual_add(dt):
    k = _k()
    rng = np.random.default_rng(2)
    T, F = 5, 333
    gu = _round(rng.standard_normal((T, 2 * F)) * 4, dt)
    gu[0, :4] = [-1e4, 1e4, -90.0, 90.0]                                             # the sigmoid must stay finite
    out = k.swiglu(torch.from_numpy(gu).to(DT[dt]).to(DEV)).float().cpu().numpy()
    assert np.isfinite(out).all()
    assert rel_err(plain_swiglu(gu[:, :F], gu[:, F:]), out) < _tol(dt)
    x = rng.standard_normal((T, F)).astype(np.float32)
    d = _round(rng.standard_normal((T, F)), dt)
    xd = torch.from_numpy(x.copy()).to(DEV)
    k.residual_add(xd, torch.from_numpy(d).to(DT[dt]).to(DEV))
    assert np.array_equal(xd.cpu().numpy(), x + d)


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 100), (65, 64, 17), (130, 777, 96), (2, 1000, 1024)])
def test_gemm_f32_is_true_fp32_and_cut_invariant(M, N, K):
    k = _k()
    rng = np.random.default_rng(3)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32)
    ad, wd = torch.from_numpy(a).to(DEV), torch.from_numpy(w).to(DEV)
    c = k.linear(ad, wd).cpu().numpy()
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    assert rel_err(ref, c) < 1e-6 * max(1.0, np.sqrt(K) / 8)        # fp32 accumulation, not tf32 (which gives ~1e-3)
    # a row's result does not depend on the rows computed with it
    one = k.linear(ad[M - 1:M].contiguous(), wd).cpu().numpy()
    assert np.array_equal(one[0], c[M - 1])


def _paged(kv: np.ndarray, page_ids, n_pages, dt, poison=None):
    """Scatter [T, KV, HD] into pages [n_pages, KV, 64, HD]."""
    T, KV, HD = kv.shape
    pages = np.full((n_pages, KV, 64, HD), 0.0 if poison is None else poison, dtype=np.float32)
    for t in range(T):
        pages[page_ids[t // 64], :, t % 64, :] = kv[t]
    return torch.from_numpy(pages).to(DT[dt]).to(DEV)


def _page_table(lists, bases=None):
    from mynah_slm_b200.ops.kernels import PageTableView
    indptr = np.cumsum([0] + [len(l) for l in lists]).astype(np.int32)
    ids = np.array([p for l in lists for p in l] or [0], dtype=np.int32)
    base = np.array(bases if bases is not None else [0] * len(lists), dtype=np.int32)
    return lambda n_pages: PageTableView(torch.from_numpy(indptr).to(DEV), torch.from_numpy(ids).to(DEV),
                                         torch.from_numpy(base).to(DEV), n_pages)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("H,KV,HD,rot", [(4, 2, 16, 16), (6, 3, 48, 48), (5, 5, 128, 128), (8, 2, 64, 32), (3, 1, 256, 256)])
def test_qk_norm_rope_store(dt, H, KV, HD, rot):
    k = _k()
    rng = np.random.default_rng(4)
    lens, past = [5, 1, 70], [0, 130, 60]                                        # three sequences; positions continue
    T = sum(lens)
    W = (H + 2 * KV) * HD
    qkv = _round(rng.standard_normal((T, W)) * 2, dt)
    qg, kg = _round(1 + 0.1 * rng.standard_normal(HD), dt), _round(1 + 0.1 * rng.standard_normal(HD), dt)
    eps, theta = 1e-5, 12345.0
    tok_seq = np.concatenate([[b] * n for b, n in enumerate(lens)]).astype(np.int32)
    tok_pos = np.concatenate([np.arange(p, p + n) for p, n in zip(past, lens)]).astype(np.int32)
    n_pages = 9
    lists = [[7], [0, 3, 5], [2, 8, 4]]                                          # scattered pages
    pt = _page_table(lists)(n_pages)
    kc = torch.full((n_pages, KV, 64, HD), 99.0, dtype=DT[dt], device=DEV)
    vc = torch.full((n_pages, KV, 64, HD), 99.0, dtype=DT[dt], device=DEV)
    cos, sin = k.rope_table(256, rot, theta, DEV)
    cr, sr = rope_table(rot, np.arange(256), theta)
    assert np.array_equal(cos.cpu().numpy(), cr) and np.array_equal(sin.cpu().numpy(), sr)   # built in double, as the reference
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    qd = torch.from_numpy(qkv).to(DT[dt]).to(DEV)
    k.qk_norm_rope_store(qd, H, KV, HD, torch.from_numpy(qg).to(DT[dt]).to(DEV), torch.from_numpy(kg).to(DT[dt]).to(DEV),
                         eps, cos, sin, rot, torch.from_numpy(tok_seq).to(DEV), torch.from_numpy(tok_pos).to(DEV), pt, kc, vc, status)
    assert status.item() == 0
    q = qkv[:, :H * HD].reshape(T, H, HD)
    kk = qkv[:, H * HD:(H + KV) * HD].reshape(T, KV, HD)
    vv = qkv[:, (H + KV) * HD:].reshape(T, KV, HD)

    def ref(x, g):
        n = rms_norm(x, g, eps)
        r = rope_apply(n[..., :rot], cr[tok_pos], sr[tok_pos])
        return np.concatenate([r, n[..., rot:]], axis=-1)
    got_q = qd.float().cpu().numpy()[:, :H * HD].reshape(T, H, HD)
    assert rel_err(ref(q, qg).reshape(T, -1), got_q.reshape(T, -1)) < _tol(dt)
    kc_np, vc_np = kc.float().cpu().numpy(), vc.float().cpu().numpy()
    rk = ref(kk, kg)
    written = np.zeros((n_pages, 64), dtype=bool)
    for t in range(T):
        pg, off = lists[tok_seq[t]][tok_pos[t] // 64], tok_pos[t] % 64
        written[pg, off] = True
        assert rel_err(rk[t].reshape(1, -1), kc_np[pg, :, off].reshape(1, -1)) < _tol(dt)
        assert np.array_equal(vc_np[pg, :, off], vv[t])                         # V is neither normed nor rotated
    untouched = ~written
    assert np.all(kc_np.transpose(0, 2, 1, 3)[untouched] == 99.0) and np.all(vc_np.transpose(0, 2, 1, 3)[untouched] == 99.0)
    # a position with no page is refused, not written somewhere
    bad_pos = torch.from_numpy(tok_pos + 64 * 3).to(DEV)
    k.qk_norm_rope_store(qd, H, KV, HD, None, None, eps, None, None, 0, torch.from_numpy(tok_seq).to(DEV), bad_pos, pt, kc, vc, status)
    assert status.item() & 1
    status.zero_()


def _attn_case(rng, lens_q, past, H, KV, HD, dt, scale_key=None):
    """Random q for the new tokens and K/V for whole sequences; returns the plain outputs."""
    seqs = []
    for nq, p in zip(lens_q, past):
        n = p + nq
        q = _round(rng.standard_normal((nq, H, HD)), dt)
        kk = _round(rng.standard_normal((n, KV, HD)), dt)
        vv = _round(rng.standard_normal((n, KV, HD)), dt)
        seqs.append((q, kk, vv))
    return seqs


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("H,KV,HD,window", [(4, 2, 16, 0), (6, 2, 32, 0), (6, 3, 48, 40), (5, 1, 80, 0), (2, 2, 128, 70), (3, 3, 256, 0)])
def test_attn_prefill_generic(dt, H, KV, HD, window):
    k = _k()
    rng = np.random.default_rng(5)
    lens_q, past = [7, 1, 33, 70], [0, 0, 100, 64]
    seqs = _attn_case(rng, lens_q, past, H, KV, HD, dt)
    n_pages, free = 16, list(np.random.default_rng(9).permutation(16))
    lists, kcs = [], None
    kc = torch.zeros((n_pages, KV, 64, HD), dtype=DT[dt], device=DEV)
    vc = torch.zeros_like(kc)
    for q, kk, vv in seqs:
        need = -(-kk.shape[0] // 64)
        pages = [int(free.pop()) for _ in range(need)]
        lists.append(pages)
        kc_s, vc_s = _paged(kk, pages, n_pages, dt, poison=1e4), _paged(vv, pages, n_pages, dt, poison=1e4)
        for pg in pages:
            kc[pg], vc[pg] = kc_s[pg], vc_s[pg]                                   # the tail of a page holds poison
    pt = _page_table(lists)(n_pages)
    T = sum(lens_q)
    qkv = torch.from_numpy(np.concatenate([s[0].reshape(s[0].shape[0], -1) for s in seqs])).to(DT[dt]).to(DEV)
    out = torch.zeros((T, H * HD), dtype=DT[dt], device=DEV)
    cu = torch.tensor(np.cumsum([0] + lens_q), dtype=torch.int32, device=DEV)
    kvl = torch.tensor([p + n for p, n in zip(past, lens_q)], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    k.attn_prefill_generic(qkv, out, len(seqs), max(lens_q), H, KV, HD, kc, vc, cu, kvl, pt, window, status)
    assert status.item() == 0
    got = out.float().cpu().numpy()
    row = 0
    for (q, kk, vv), nq, p in zip(seqs, lens_q, past):
        ref = gqa_attention(q, kk, vv, window=window or None, q_pos=np.arange(p, p + nq), k_pos=np.arange(p + nq))
        assert rel_err(ref.reshape(nq, -1), got[row:row + nq]) < (3e-6 if dt == "f32" else 1e-2), (nq, p)
        row += nq


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("H,KV,HD,window,splits", [(4, 2, 16, 0, 9), (6, 2, 32, 0, 16), (6, 3, 48, 40, 2), (5, 1, 80, 0, 9),
                                                   (16, 8, 128, 0, 12), (8, 1, 64, 100, 3), (3, 3, 256, 0, 9)])
def test_attn_decode(dt, H, KV, HD, window, splits):
    k = _k()
    rng = np.random.default_rng(6)
    lens = [1, 64, 65, 300, 0, 517]                                               # a padding sequence among them
    B = len(lens)
    n_pages = 24
    free = list(np.random.default_rng(10).permutation(n_pages))
    kc = torch.zeros((n_pages, KV, 64, HD), dtype=DT[dt], device=DEV)
    vc = torch.zeros_like(kc)
    lists, seqs = [], []
    for n in lens:
        kk, vv = _round(rng.standard_normal((n, KV, HD)), dt), _round(rng.standard_normal((n, KV, HD)), dt)
        pages = [int(free.pop()) for _ in range(-(-n // 64))]
        lists.append(pages)
        seqs.append((kk, vv))
        if n:
            kc_s, vc_s = _paged(kk, pages, n_pages, dt, poison=1e4), _paged(vv, pages, n_pages, dt, poison=1e4)
            for pg in pages:
                kc[pg], vc[pg] = kc_s[pg], vc_s[pg]
    q = _round(rng.standard_normal((B, H, HD)), dt)
    qd = torch.from_numpy(q.reshape(B, -1)).to(DT[dt]).to(DEV)
    out = torch.full((B, H * HD), 7.0, dtype=DT[dt], device=DEV)
    kvl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scratch = torch.empty(k.attn_decode_scratch_floats(B, H, HD, splits), dtype=torch.float32, device=DEV)
    k.attn_decode(qd, out, B, H, KV, HD, kc, vc, kvl, _page_table(lists)(n_pages), window, splits, scratch, status)
    assert status.item() == 0
    got = out.float().cpu().numpy()
    for b, n in enumerate(lens):
        if n == 0:
            assert np.all(got[b] == 0)
            continue
        kk, vv = seqs[b]
        ref = gqa_attention(q[b:b + 1], kk, vv, window=window or None, q_pos=[n - 1], k_pos=np.arange(n))
        assert rel_err(ref.reshape(1, -1), got[b:b + 1]) < (3e-6 if dt == "f32" else 1e-2), (b, n)
    # a larger launch gives the same bits; one that is too small says so instead of dropping keys
    out2 = torch.zeros_like(out)
    scratch2 = torch.empty(k.attn_decode_scratch_floats(B, H, HD, splits + 5), dtype=torch.float32, device=DEV)
    k.attn_decode(qd, out2, B, H, KV, HD, kc, vc, kvl, _page_table(lists)(n_pages), window, splits + 5, scratch2, status)
    assert torch.equal(out, out2) and status.item() == 0
    k.attn_decode(qd, out2, B, H, KV, HD, kc, vc, kvl, _page_table(lists)(n_pages), window, 1, scratch2, status)
    assert status.item() == 8
    status.zero_()


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("kind", ["prefill", "decode"])
def test_one_far_key_and_the_window_edge(dt, kind):
    """Random values hide a missed key among hundreds. Here one key's score
    stands out, so the output is that key's value or is not: at a far
    position, at the first position of a page, and on both sides of the
    window's edge. Two sequences with interleaved pages share the launch."""
    k = _k()
    H, KV, HD, n = 2, 1, 64, 400
    rng = np.random.default_rng(7)
    for window, target, visible in [(0, 3, True), (0, 64, True), (0, 399, True), (120, 280, True), (120, 279, False)]:
        # query at position n-1 sees keys > n-1-window
        kk = _round(rng.standard_normal((n, KV, HD)) * 0.1, dt)
        vv = _round(rng.standard_normal((n, KV, HD)), dt)
        q = _round(rng.standard_normal((1, H, HD)) * 0.1, dt)
        kk[target, 0] = q[0, 0] / np.linalg.norm(q[0, 0]) * 60.0            # score far above the others for head 0
        q[0, 0] *= 20
        other_k = _round(rng.standard_normal((n, KV, HD)) * 0.1, dt)
        other_v = _round(rng.standard_normal((n, KV, HD)), dt)
        lists = [[0, 2, 4, 6, 8, 10, 12], [1, 3, 5, 7, 9, 11, 13]]
        n_pages = 14
        kc = _paged(kk, lists[0], n_pages, dt) + _paged(other_k, lists[1], n_pages, dt)
        vc = _paged(vv, lists[0], n_pages, dt) + _paged(other_v, lists[1], n_pages, dt)
        pt = _page_table(lists)(n_pages)
        qd = torch.from_numpy(np.concatenate([q, q]).reshape(2, -1)).to(DT[dt]).to(DEV)
        out = torch.zeros((2, H * HD), dtype=DT[dt], device=DEV)
        kvl = torch.tensor([n, n], dtype=torch.int32, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        if kind == "decode":
            scratch = torch.empty(k.attn_decode_scratch_floats(2, H, HD, 7), dtype=torch.float32, device=DEV)
            k.attn_decode(qd, out, 2, H, KV, HD, kc, vc, kvl, pt, window, 7, scratch, status)
        else:
            cu = torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV)
            k.attn_prefill_generic(qd, out, 2, 1, H, KV, HD, kc, vc, cu, kvl, pt, window, status)
        got = out.float().cpu().numpy()[0, :HD]
        hit = np.abs(got - vv[target, 0]).max() < 0.05
        assert hit == visible, (window, target, visible)
        ref = gqa_attention(q, kk, vv, window=window or None, q_pos=[n - 1], k_pos=np.arange(n))
        assert rel_err(ref.reshape(1, -1), out.float().cpu().numpy()[0:1]) < (1e-5 if dt == "f32" else 2e-2)


@pytest.mark.parametrize("V", [777, 151936, 1000])
def test_argmax_first_maximum(V):
    k = _k()
    rng = np.random.default_rng(8)
    lg = rng.standard_normal((5, V)).astype(np.float32)
    lg[1, [V - 1, 17, 300]] = 9.0                                                  # ties: the lowest id wins
    lg[2, :] = 0.0
    got = k.argmax(torch.from_numpy(lg).to(DEV)).cpu().numpy()
    assert got.tolist() == [int(np.argmax(r)) for r in lg]
    assert got[1] == 17 and got[2] == 0


def _sampler_state(B, seeds):
    st = torch.tensor([s - (1 << 64) if s >= (1 << 63) else s for s in seeds], dtype=torch.int64, device=DEV)
    return st


@pytest.mark.parametrize("V", [777, 32000, 40003])      # one CTA a row; with the two-step maximum; a cluster a row
@pytest.mark.parametrize("temp,top_k,top_p,min_p", [(0.8, 0, 1.0, 0.0), (0.6, 20, 0.95, 0.0), (1.0, 5, 1.0, 0.0),
                                                    (1.3, 0, 0.7, 0.0), (1.0, 0, 1.0, 0.05), (0.7, 50, 0.9, 0.02),
                                                    (1.0, 1, 1.0, 0.0), (0.0, 20, 0.95, 0.0), (2.0, 0, 0.999, 0.0),
                                                    (1.0, 256, 0.98, 0.0), (0.9, 300, 0.9, 0.0), (1.0, 5, 0.5, 0.3),
                                                    (1.5, 7, 1.0, 0.0)])
def test_sample_matches_plain_sampler(V, temp, top_k, top_p, min_p):
    """Same logits, same generator state -> same token, draw after draw."""
    k = _k()
    rng = np.random.default_rng(11)
    B, rounds = 6, 12
    seeds = [int(rng.integers(1, 2 ** 62)) for _ in range(B)]
    plain = [PlainSampler(temp=temp, top_k=top_k, top_p=top_p, min_p=min_p, rng_state=s) for s in seeds]
    state = _sampler_state(B, seeds)
    params = torch.tensor([temp, top_p, min_p, float(top_k), 1.0, 0.0, 0.0, 0.0], dtype=torch.float32, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    for r in range(rounds):
        lg = (rng.standard_normal((B, V)) * (1.0 + r % 3)).astype(np.float32)
        lg[0, :8] = lg[0, 0]                                                       # equal probabilities: ids break ties
        lg[1, 100:110] = lg[1].max() + 0.5                                         # ten equal largest: a small top-k ends among them
        want = [p.sample(lg[b].copy()) for b, p in enumerate(plain)]
        got = k.sample(torch.from_numpy(lg.copy()).to(DEV), params, state, slots).cpu().tolist()
        assert got == want, (r, got, want)
    # the states advanced exactly as the plain generators did (greedy draws nothing)
    want_state = [p.rng.state for p in plain]
    got_state = [(int(s) + (1 << 64)) % (1 << 64) for s in state.cpu().tolist()]
    assert got_state == want_state


def test_sample_padding_rows_and_slot_mapping():
    k = _k()
    rng = np.random.default_rng(12)
    V = 500
    lg = rng.standard_normal((3, V)).astype(np.float32)
    state = _sampler_state(4, [11, 22, 33, 44])
    params = torch.tensor([1.0, 1.0, 0.0, 0.0, 1.0, 0.0, 0.0, 0.0], dtype=torch.float32, device=DEV)
    slots = torch.tensor([3, -1, 1], dtype=torch.int32, device=DEV)
    got = k.sample(torch.from_numpy(lg.copy()).to(DEV), params, state, slots).cpu().tolist()
    assert got[0] == PlainSampler(temp=1.0, top_k=0, top_p=1.0, rng_state=44).sample(lg[0].copy())
    assert got[2] == PlainSampler(temp=1.0, top_k=0, top_p=1.0, rng_state=22).sample(lg[2].copy())
    st = state.cpu().tolist()
    assert st[0] == 11 and st[2] == 33                                              # untouched slots keep their state


def test_penalties_and_ring_match_plain():
    k = _k()
    rng = np.random.default_rng(13)
    V, W, stride, B = 300, 5, 8, 3
    plain = [PlainSampler(temp=0, repeat_penalty=1.3, freq_penalty=0.2, presence_penalty=0.1, penalty_window=W) for _ in range(B)]
    ring = torch.zeros((B, stride), dtype=torch.int32, device=DEV)
    ring_n = torch.zeros(B, dtype=torch.int32, device=DEV)
    ring_head = torch.zeros(B, dtype=torch.int32, device=DEV)
    params = torch.tensor([0.0, 1.0, 0.0, 0.0, 1.3, 0.2, 0.1, float(W)], dtype=torch.float32, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    for step in range(12):
        toks = rng.integers(0, 6, size=B).astype(np.int32)                           # few ids: repeats inside the window
        for b in range(B):
            plain[b].accept(int(toks[b]))
        k.sampler_accept(torch.from_numpy(toks).to(DEV), ring, ring_n, ring_head, slots, params)
        lg = rng.standard_normal((B, V)).astype(np.float32)
        ref = lg.copy()
        for b in range(B):
            plain[b].apply_penalties(ref[b])
        d = torch.from_numpy(lg.copy()).to(DEV)
        k.apply_penalties(d, ring, ring_n, slots, params)
        assert np.allclose(d.cpu().numpy(), ref, rtol=1e-6, atol=1e-6), step
    assert ring_n.cpu().tolist() == [W] * B


def test_refusals_are_errors_not_wrong_results():
    from mynah_slm_b200.ops.lib import KernelError
    k = _k()
    q = torch.zeros((1, 4 * 264), dtype=torch.float32, device=DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    pt = _page_table([[0]])(1)
    kc = torch.zeros((1, 1, 64, 264), dtype=torch.float32, device=DEV)
    with pytest.raises(KernelError, match="head_dim 264"):
        k.attn_decode(q, q.clone(), 1, 4, 1, 264, kc, kc, torch.ones(1, dtype=torch.int32, device=DEV), pt, 0, 1,
                      torch.zeros(10000, device=DEV), st)
    with pytest.raises(KernelError, match="head_dim 264 exceeds"):
        k.attn_prefill_generic(q, q.clone(), 1, 1, 4, 1, 264, kc, kc, torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                               torch.ones(1, dtype=torch.int32, device=DEV), pt, 0, st)
    with pytest.raises(KernelError, match="not contiguous"):
        k.swiglu(torch.zeros((4, 8), device=DEV)[:, ::2])
    with pytest.raises(KernelError, match="unsupported dtype"):
        k.swiglu(torch.zeros((4, 8), device=DEV, dtype=torch.float16))


@pytest.mark.parametrize("H,KV,HD,window", [(16, 8, 128, 0), (8, 1, 64, 100), (32, 8, 128, 0), (16, 1, 128, 0), (6, 2, 64, 70)])
def test_attn_decode_tensor_cores(H, KV, HD, window):
    """The tensor-core decode kernel against the plain attention, with stale
    values (NaN bit patterns) in the unused tail of every page."""
    k = _k()
    assert k.attn_decode_tc_supported(torch.bfloat16, H, KV, HD)
    assert not k.attn_decode_tc_supported(torch.bfloat16, 6, 2, 48) and not k.attn_decode_tc_supported(torch.float32, H, KV, HD)
    rng = np.random.default_rng(14)
    lens = [1, 64, 65, 300, 0, 517, 128]
    B, n_pages = len(lens), 26
    free = list(np.random.default_rng(15).permutation(n_pages))
    kc = torch.full((n_pages, KV, 64, HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full((n_pages, KV, 64, HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    lists, seqs = [], []
    for n in lens:
        kk, vv = _round(rng.standard_normal((n, KV, HD)), "bf16"), _round(rng.standard_normal((n, KV, HD)), "bf16")
        pages = [int(free.pop()) for _ in range(-(-n // 64))]
        lists.append(pages)
        seqs.append((kk, vv))
        for t in range(n):
            kc[pages[t // 64], :, t % 64] = torch.from_numpy(kk[t]).to(torch.bfloat16).to(DEV)
            vc[pages[t // 64], :, t % 64] = torch.from_numpy(vv[t]).to(torch.bfloat16).to(DEV)
    q = _round(rng.standard_normal((B, H, HD)), "bf16")
    qd = torch.from_numpy(q.reshape(B, -1)).to(torch.bfloat16).to(DEV)
    kvl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    outs = []
    for splits in (9, 16):
        out = torch.full((B, H * HD), 7.0, dtype=torch.bfloat16, device=DEV)
        scratch = torch.full((k.attn_decode_scratch_floats(B, H, HD, splits),), float("nan"), dtype=torch.float32, device=DEV)
        k.attn_decode_tc(qd, out, B, H, KV, HD, kc, vc, kvl, _page_table(lists)(n_pages), window, splits, scratch, status)
        assert status.item() == 0
        outs.append(out)
    assert torch.equal(outs[0], outs[1])                       # the size of the launch does not change a bit
    # the pages' kernel merging by itself (the last CTA of a sequence's kv head): the same bits, counts left zero
    counters = torch.zeros(B * KV, dtype=torch.int32, device=DEV)
    for _ in range(2):
        out_m = torch.full((B, H * HD), 7.0, dtype=torch.bfloat16, device=DEV)
        scratch = torch.full((k.attn_decode_scratch_floats(B, H, HD, 9),), float("nan"), dtype=torch.float32, device=DEV)
        k.attn_decode_tc(qd, out_m, B, H, KV, HD, kc, vc, kvl, _page_table(lists)(n_pages), window, 9, scratch, status, counters)
        assert status.item() == 0 and torch.equal(out_m, outs[0]) and int(counters.abs().sum().item()) == 0
    got = outs[0].float().cpu().numpy()
    assert np.isfinite(got).all()
    for b, n in enumerate(lens):
        if n == 0:
            assert np.all(got[b] == 0)
            continue
        kk, vv = seqs[b]
        ref = gqa_attention(q[b:b + 1], kk, vv, window=window or None, q_pos=[n - 1], k_pos=np.arange(n))
        assert rel_err(ref.reshape(1, -1), got[b:b + 1]) < 1e-2, (b, n)
    # each sequence alone gives the same bits as in the batch
    b = 5
    out1 = torch.zeros((1, H * HD), dtype=torch.bfloat16, device=DEV)
    scratch = torch.empty(k.attn_decode_scratch_floats(1, H, HD, 9), dtype=torch.float32, device=DEV)
    k.attn_decode_tc(qd[b:b + 1].contiguous(), out1, 1, H, KV, HD, kc, vc, kvl[b:b + 1].contiguous(),
                     _page_table([lists[b]])(n_pages), window, 9, scratch, status)
    assert torch.equal(out1[0], outs[0][b])
    k.attn_decode_tc(qd, out, B, H, KV, HD, kc, vc, kvl, _page_table(lists)(n_pages), window, 2, scratch.new_empty(B * H * 2 * (HD + 2)), status)
    assert status.item() == 8
    status.zero_()


@pytest.mark.parametrize("H,KV,HD,window", [(16, 8, 128, 0), (8, 1, 64, 100), (32, 8, 128, 0), (16, 1, 128, 0), (6, 2, 64, 70),
                                             (4, 4, 128, 130), (64, 8, 64, 0)])
def test_attn_decode_streamed_pages_give_the_same_bits(H, KV, HD, window):
    """The pages of a step through persistent CTAs fed by TMA against the same pages one CTA each: the same bits in
    every output row and in every partial result, with NaN bit patterns in the unused tails of the pages (the
    stream copies whole tiles), empty sequences among the others, windows whose first page is cut, and more
    sequences than CTAs."""
    k = _k()
    rng = np.random.default_rng(41)
    lens = [1, 64, 65, 300, 0, 517, 128, 63, 2, 191] + rng.integers(1, 200, size=30).tolist()
    B = len(lens)
    n_pages = sum(-(-n // 64) for n in lens) + 3
    free = list(np.random.default_rng(42).permutation(n_pages))
    kc = torch.full((n_pages, KV, 64, HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full((n_pages, KV, 64, HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    lists, seqs = [], []
    for n in lens:
        kk, vv = _round(rng.standard_normal((n, KV, HD)), "bf16"), _round(rng.standard_normal((n, KV, HD)), "bf16")
        pages = [int(free.pop()) for _ in range(-(-n // 64))]
        lists.append(pages)
        seqs.append((kk, vv))
        for i, pg in enumerate(pages):
            m = min(64, n - i * 64)
            kc[pg, :, :m] = torch.from_numpy(kk[i * 64:i * 64 + m]).to(torch.bfloat16).to(DEV).transpose(0, 1)
            vc[pg, :, :m] = torch.from_numpy(vv[i * 64:i * 64 + m]).to(torch.bfloat16).to(DEV).transpose(0, 1)
    q = _round(rng.standard_normal((B, H, HD)), "bf16")
    qd = torch.from_numpy(q.reshape(B, -1)).to(torch.bfloat16).to(DEV)
    kvl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    splits = 12
    outs, parts = {}, {}
    before = k.attn_decode_stream_mode(0)
    try:
        for mode in (0, 2, 2):
            k.attn_decode_stream_mode(mode)
            out = torch.full((B, H * HD), 7.0, dtype=torch.bfloat16, device=DEV)
            scratch = torch.zeros((k.attn_decode_scratch_floats(B, H, HD, splits),), dtype=torch.float32, device=DEV)
            k.attn_decode_tc(qd, out, B, H, KV, HD, kc, vc, kvl, _page_table(lists)(n_pages), window, splits, scratch, status)
            assert status.item() == 0
            outs.setdefault(mode, []).append(out)
            parts.setdefault(mode, []).append(scratch)
    finally:
        k.attn_decode_stream_mode(before)
    assert torch.isfinite(outs[0][0].float()).all()
    for again in outs[2]:
        assert torch.equal(outs[0][0], again)
    # the partial results of every visible page too (what lies beyond a sequence's visible pages is never read)
    n_o = B * H * splits * HD
    for again in parts[2]:
        for b, n in enumerate(lens):
            lo = max(0, n - window) if window else 0
            n_vis = min(splits, (n - 1) // 64 + 1 - lo // 64) if n else 0
            for t, width, off in ((parts[0][0], HD, 0), (parts[0][0], 2, n_o)):
                one = t[off:off + B * H * splits * width].view(B, H, splits, width)[b, :, :n_vis]
                other = again[off:off + B * H * splits * width].view(B, H, splits, width)[b, :, :n_vis]
                assert torch.equal(one, other), (b, n, width)
    got = outs[2][0].float().cpu().numpy()
    for b, n in enumerate(lens):
        if n == 0:
            assert np.all(got[b] == 0)
            continue
        kk, vv = seqs[b]
        ref = gqa_attention(q[b:b + 1], kk, vv, window=window or None, q_pos=[n - 1], k_pos=np.arange(n))
        assert rel_err(ref.reshape(1, -1), got[b:b + 1]) < 1e-2, (b, n)


def test_attn_decode_tensor_cores_one_far_key():
    k = _k()
    H, KV, HD, n = 4, 2, 128, 400
    rng = np.random.default_rng(16)
    for window, target, visible in [(0, 3, True), (0, 64, True), (0, 399, True), (120, 280, True), (120, 279, False)]:
        kk = _round(rng.standard_normal((n, KV, HD)) * 0.1, "bf16")
        vv = _round(rng.standard_normal((n, KV, HD)), "bf16")
        q = _round(rng.standard_normal((1, H, HD)) * 0.1, "bf16")
        kk[target, 1] = _round(q[0, 3] / np.linalg.norm(q[0, 3]) * 60.0, "bf16")      # head 3 reads kv head 1
        q[0, 3] = _round(q[0, 3] * 16, "bf16")
        lists = [[5, 1, 6, 2, 0, 3, 4]]
        kc, vc = _paged(kk, lists[0], 7, "bf16"), _paged(vv, lists[0], 7, "bf16")
        out = torch.zeros((1, H * HD), dtype=torch.bfloat16, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        scratch = torch.empty(k.attn_decode_scratch_floats(1, H, HD, 7), dtype=torch.float32, device=DEV)
        k.attn_decode_tc(torch.from_numpy(q.reshape(1, -1)).to(torch.bfloat16).to(DEV), out, 1, H, KV, HD, kc, vc,
                         torch.tensor([n], dtype=torch.int32, device=DEV), _page_table(lists)(7), window, 7, scratch, status)
        got = out.float().cpu().numpy()[0, 3 * HD:4 * HD]
        assert (np.abs(got - vv[target, 1]).max() < 0.05) == visible, (window, target)
        ref = gqa_attention(q, kk, vv, window=window or None, q_pos=[n - 1], k_pos=np.arange(n))
        assert rel_err(ref.reshape(1, -1), out.float().cpu().numpy()) < 2e-2


@pytest.mark.parametrize("H,KV,HD,window,with_norm,with_rope", [(16, 8, 128, 0, True, True), (8, 1, 64, 100, True, True),
                                                                 (6, 2, 64, 70, False, True), (32, 8, 128, 0, True, False)])
def test_attn_decode_fused_is_norm_rope_store_and_attention(H, KV, HD, window, with_norm, with_rope):
    """One launch against the plain parts: per-head norm and rotation of q and of the new k, the write of the new
    position into the cache, attention over the pages, the merge. Lengths put the new position at a page's
    first and last row; the unused tail of every page holds NaN patterns."""
    k = _k()
    rng = np.random.default_rng(24)
    lens = [1, 64, 65, 300, 0, 517, 128]                       # lengths after this step (0: a padding row)
    B, n_pages, eps, theta = len(lens), 26, 1e-5, 5000.0
    free = list(np.random.default_rng(25).permutation(n_pages))
    kc = torch.full((n_pages, KV, 64, HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full((n_pages, KV, 64, HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    lists, seqs = [], []
    for n in lens:
        kk, vv = _round(rng.standard_normal((max(n - 1, 0), KV, HD)), "bf16"), _round(rng.standard_normal((max(n - 1, 0), KV, HD)), "bf16")
        pages = [int(free.pop()) for _ in range(-(-n // 64))]
        lists.append(pages)
        seqs.append((kk, vv))
        for t in range(n - 1):
            kc[pages[t // 64], :, t % 64] = torch.from_numpy(kk[t]).to(torch.bfloat16).to(DEV)
            vc[pages[t // 64], :, t % 64] = torch.from_numpy(vv[t]).to(torch.bfloat16).to(DEV)
    W = (H + 2 * KV) * HD
    qkv = _round(rng.standard_normal((B, W)) * 1.5, "bf16")
    qg = _round(1 + 0.1 * rng.standard_normal(HD), "bf16") if with_norm else None
    kg = _round(1 + 0.1 * rng.standard_normal(HD), "bf16") if with_norm else None
    dev = lambda a: None if a is None else torch.from_numpy(a).to(torch.bfloat16).to(DEV)
    cos, sin = k.rope_table(600, HD, theta, DEV) if with_rope else (None, None)
    cr, sr = rope_table(HD, np.arange(600), theta)
    pos = np.array([max(n - 1, 0) for n in lens], dtype=np.int32)
    kvl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tok_pos = torch.from_numpy(pos).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    counters = torch.zeros(B * KV, dtype=torch.int32, device=DEV)
    pt = _page_table(lists)(n_pages)
    qd = torch.from_numpy(qkv).to(torch.bfloat16).to(DEV)

    def run(splits, kc_, vc_, qd_=qd, kvl_=kvl, pos_=tok_pos, pt_=pt, rows=B):
        out = torch.full((rows, H * HD), 7.0, dtype=torch.bfloat16, device=DEV)
        scratch = torch.full((k.attn_decode_scratch_floats(rows, H, HD, splits),), float("nan"), dtype=torch.float32, device=DEV)
        k.attn_decode_fused(qd_, out, rows, H, KV, HD, dev(qg), dev(kg), eps, cos, sin, pos_, kc_, vc_, True, kvl_, pt_,
                            window, splits, scratch, counters, status)
        assert status.item() == 0 and int(counters.abs().sum()) == 0      # left zero for the next launch
        return out
    kc1, vc1 = kc.clone(), vc.clone()
    out_a = run(9, kc1, vc1)
    kc2, vc2 = kc.clone(), vc.clone()
    out_b = run(16, kc2, vc2)
    assert torch.equal(out_a, out_b) and torch.equal(kc1.nan_to_num(5.0), kc2.nan_to_num(5.0))
    # the cache rows and the rounded q are those of the separate pass, bit for bit
    kc3, vc3, q3 = kc.clone(), vc.clone(), qd.clone()
    seq_ids = torch.tensor([b if n > 0 else -1 for b, n in enumerate(lens)], dtype=torch.int32, device=DEV)
    k.qk_norm_rope_store(q3, H, KV, HD, dev(qg), dev(kg), eps, cos, sin, HD if with_rope else 0, seq_ids, tok_pos, pt, kc3, vc3, status)
    assert torch.equal(kc1.nan_to_num(5.0), kc3.nan_to_num(5.0)) and torch.equal(vc1.nan_to_num(5.0), vc3.nan_to_num(5.0))
    # ... and so is the result of the three separate launches, so a step may take either route
    out_sep = torch.zeros_like(out_a)
    k.attn_decode_tc(q3, out_sep, B, H, KV, HD, kc3, vc3, kvl, pt, window, 9,
                     torch.empty(k.attn_decode_scratch_floats(B, H, HD, 9), dtype=torch.float32, device=DEV), status)
    assert status.item() == 0 and torch.equal(out_sep, out_a)
    got = out_a.float().cpu().numpy()
    assert np.isfinite(got).all()

    def prep(x, g):
        y = rms_norm(x, g, eps) if with_norm else x
        return y
    for b, n in enumerate(lens):
        if n == 0:
            assert np.all(got[b] == 0)
            continue
        q = qkv[b, :H * HD].reshape(1, H, HD)
        kn = qkv[b, H * HD:(H + KV) * HD].reshape(1, KV, HD)
        vn = qkv[b, (H + KV) * HD:].reshape(1, KV, HD)
        q, kn = prep(q, qg), prep(kn, kg)
        if with_rope:
            q, kn = rope_apply(q, cr[[n - 1]], sr[[n - 1]]), rope_apply(kn, cr[[n - 1]], sr[[n - 1]])
        kk = np.concatenate([seqs[b][0], _round(kn, "bf16")]) if n > 1 else _round(kn, "bf16")
        vv = np.concatenate([seqs[b][1], vn]) if n > 1 else vn
        ref = gqa_attention(_round(q, "bf16"), kk, vv, window=window or None, q_pos=[n - 1], k_pos=np.arange(n))
        assert rel_err(ref.reshape(1, -1), got[b:b + 1]) < 1e-2, (b, n)
    # a sequence alone gives the same bits as in the batch
    b = 5
    kc4, vc4 = kc.clone(), vc.clone()
    out1 = run(9, kc4, vc4, qd[b:b + 1].contiguous(), kvl[b:b + 1].contiguous(), tok_pos[b:b + 1].contiguous(),
               _page_table([lists[b]])(n_pages), rows=1)
    assert torch.equal(out1[0], out_a[b])
    # a run that reads a cache another run wrote: only q is prepared, the cache is read whole
    out_c = torch.zeros_like(out_a)
    scratch = torch.empty(k.attn_decode_scratch_floats(B, H, HD, 9), dtype=torch.float32, device=DEV)
    k.attn_decode_fused(qd, out_c, B, H, KV, HD, dev(qg), dev(kg), eps, cos, sin, tok_pos, kc1, vc1, False, kvl, pt,
                        window, 9, scratch, counters, status)
    assert torch.equal(out_c, out_a)
    # too few splits for the pages, and a position beyond the table, are reported
    k.attn_decode_fused(qd, out_c, B, H, KV, HD, dev(qg), dev(kg), eps, cos, sin, tok_pos, kc1, vc1, False, kvl, pt,
                        window, 2, scratch, counters, status)
    assert status.item() & 8
    status.zero_()
    if with_rope:
        k.attn_decode_fused(qd, out_c, B, H, KV, HD, dev(qg), dev(kg), eps, cos, sin, tok_pos + 600, kc1, vc1, False, kvl, pt,
                            window, 9, scratch, counters, status)
        assert status.item() & 2
        status.zero_()
    assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("M,N,K", [(1, 1024, 1024), (3, 1000, 96), (8, 4096, 1024), (16, 1024, 3072), (5, 30000, 1024), (2, 20, 64),
                                   (8, 328, 2560), (2, 264, 9728), (7, 12, 32), (16, 2370, 4096), (1, 6, 12288), (9, 5000, 352)])
def test_gemv_decode_both_forms_give_the_same_bits(M, N, K):
    """The decode products with their weights through registers and through the ring of asynchronous copies: every
    output has the same bits (the same sums in the same order), for plain rows, fp32 rows and the SwiGLU epilogue;
    sizes that are no multiple of anything, one group of rows and many, rows too long to stage."""
    k = _k()
    rng = np.random.default_rng(N + K + M)
    w = _round(rng.standard_normal((N, K)) * 0.05, "bf16")
    x = _round(rng.standard_normal((M, K)), "bf16")
    wd = torch.from_numpy(w).to(torch.bfloat16).to(DEV)
    xd = torch.from_numpy(x).to(torch.bfloat16).to(DEV)
    ref = x.astype(np.float64) @ w.astype(np.float64).T
    outs = {}
    before = k.gemv_decode_mode(0)
    saved = k.GEMV_LIBRARY_FROM_ROWS
    k.GEMV_LIBRARY_FROM_ROWS = 0                     # every size through this kernel
    try:
        for mode in (0, 1):
            k.gemv_decode_mode(mode)
            outs[mode] = (k.linear(xd, wd), k.linear(xd, wd, out_dtype=torch.float32),
                          k.linear_swiglu(xd, wd) if N % 2 == 0 else None)
    finally:
        k.gemv_decode_mode(before)
        k.GEMV_LIBRARY_FROM_ROWS = saved
    for mode in (0, 1):
        assert rel_err(ref, outs[mode][1].cpu().numpy()) < 2e-5, mode
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    if N % 2 == 0:
        F = N // 2
        gu = _round(ref, "bf16")
        assert torch.equal(outs[0][2], outs[1][2])
        assert rel_err(plain_swiglu(gu[:, :F], gu[:, F:]), outs[1][2].float().cpu().numpy()) < 1.5e-2


@pytest.mark.parametrize("M,N,K", [(1, 1024, 1024), (3, 1000, 96), (8, 4096, 1024), (16, 1024, 3072), (5, 30000, 1024), (2, 20, 64),
                                   (8, 328, 2560), (2, 264, 9728)])      # rows of 41 KB: just under the opt-in limit; long rows
def test_gemv_decode_fused_kernels(M, N, K):
    """The decode products with their fusions: plain rows, fp32 rows, the norm
    prologue with the residual add, and the SwiGLU epilogue."""
    from mynah_slm_b200.parts.base import Residual
    k = _k()
    assert k.gemv_decode_supported(M, N, K) and not k.gemv_decode_supported(17, N, K) and not k.gemv_decode_supported(M, N, 80)
    rng = np.random.default_rng(17)
    w = _round(rng.standard_normal((N, K)) * 0.05, "bf16")
    x = _round(rng.standard_normal((M, K)), "bf16")
    wd = torch.from_numpy(w).to(torch.bfloat16).to(DEV)
    xd = torch.from_numpy(x).to(torch.bfloat16).to(DEV)
    ref = x.astype(np.float64) @ w.astype(np.float64).T
    got = k.linear(xd, wd)
    assert got.dtype == torch.bfloat16 and rel_err(ref, got.float().cpu().numpy()) < 6e-3
    got32 = k.linear(xd, wd, out_dtype=torch.float32)
    assert got32.dtype == torch.float32 and rel_err(ref, got32.cpu().numpy()) < 2e-5      # fp32 accumulation of bf16 products
    # a row's result does not depend on the other rows of the batch
    one = k.linear(xd[M - 1:M].contiguous(), wd, out_dtype=torch.float32)
    assert torch.equal(one[0], got32[M - 1])
    # norm prologue: residual + pending add -> norm -> product; the residual comes back updated
    res = (rng.standard_normal((M, K)) * 3).astype(np.float32)
    delta = _round(rng.standard_normal((M, K)), "bf16")
    gain = _round(1 + 0.1 * rng.standard_normal(K), "bf16")
    eps = 1e-5
    h_ref = _round(rms_norm(res + delta, gain, eps), "bf16")
    stream = Residual(torch.from_numpy(res.copy()).to(DEV))
    normed = k.NormedInput(stream, torch.from_numpy(delta).to(torch.bfloat16).to(DEV),
                           torch.from_numpy(gain).to(torch.bfloat16).to(DEV), eps, torch.bfloat16)
    old_x = stream.x
    saved_rows = k.FUSED_NORM_MAX_ROWS
    k.FUSED_NORM_MAX_ROWS = 16                     # the prologue for every row count the kernel takes (the engine's default is lower)
    try:
        got = k.linear(normed, wd, out_dtype=torch.float32).cpu().numpy()
    finally:
        k.FUSED_NORM_MAX_ROWS = saved_rows
    assert rel_err(h_ref.astype(np.float64) @ w.astype(np.float64).T, got) < 5e-3      # h may round the other way here and there
    assert np.array_equal(stream.x.cpu().numpy(), res + delta)
    # fused: the updated residual is a new buffer, the input rows are left alone
    assert np.array_equal(old_x.cpu().numpy(), res) or stream.x is old_x
    if k._norm_prologue_fits(M, K):
        assert stream.x is not old_x
    # the unfused route (norm kernel, then the product) through the same handle
    stream2 = Residual(torch.from_numpy(res.copy()).to(DEV))
    normed2 = k.NormedInput(stream2, torch.from_numpy(delta).to(torch.bfloat16).to(DEV),
                            torch.from_numpy(gain).to(torch.bfloat16).to(DEV), eps, torch.bfloat16)
    k.FUSED_NORM_MAX_ROWS = 0
    try:
        got2 = k.linear(normed2, wd, out_dtype=torch.float32).cpu().numpy()
    finally:
        k.FUSED_NORM_MAX_ROWS = saved_rows
    assert rel_err(got2, got) < 5e-3 and np.array_equal(stream2.x.cpu().numpy(), res + delta)
    # the same through the separate norm kernel gives the same rounding points
    h_dev = k.rmsnorm(torch.from_numpy(res.copy()).to(DEV), torch.from_numpy(gain).to(torch.bfloat16).to(DEV), eps,
                      torch.bfloat16, delta=torch.from_numpy(delta).to(torch.bfloat16).to(DEV))
    sep = k.linear(h_dev, wd, out_dtype=torch.float32).cpu().numpy()
    assert rel_err(sep, got) < 5e-3
    # SwiGLU epilogue: N gate rows then N up rows
    if N % 2 == 0 and N <= 4096:
        F = N // 2
        act = k.linear_swiglu(xd, wd).float().cpu().numpy()
        gu = _round(ref, "bf16")
        assert act.shape == (M, F) and rel_err(plain_swiglu(gu[:, :F], gu[:, F:]), act) < 1.5e-2


def test_fused_decode_path_equals_the_unfused_one(tmp_path):
    """A decode step through the fused kernels (a few rows) against the same
    step through the library product and the separate norm and activation
    kernels (forced by a batch of more than 16 rows is not needed: the fused
    path is switched off instead)."""
    from helpers import make_folder, prompts_for
    from mynah_slm_b200.engine.engine import Engine, StepEntry
    from mynah_slm_b200.ops import kernels
    folder = make_folder(tmp_path, "B", torch.bfloat16)
    p = prompts_for("B", [40, 7, 70], seed=19)
    outs = []
    for fused in (True, False):
        saved = kernels.gemv_decode_supported
        if not fused:
            kernels.gemv_decode_supported = lambda M, N, K: False
        try:
            eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=512, use_graphs=False)
            slots = [eng.open_sequence() for _ in p]
            eng.step([StepEntry(s, q, ()) for s, q in zip(slots, p)])
            rows = [eng.step([StepEntry(s, [q[t]], (0,)) for s, q in zip(slots, p)]).cpu().numpy() for t in range(3)]
            eng.check_status()
            outs.append(np.concatenate(rows))
        finally:
            kernels.gemv_decode_supported = saved
    assert rel_err(outs[1], outs[0]) < 1e-2


@pytest.mark.parametrize("which", ["mma_sync", "tcgen05", "tcgen05_one_stage"])
@pytest.mark.parametrize("H,KV,HD,window", [(16, 8, 128, 0), (4, 1, 64, 0), (6, 2, 128, 100), (8, 8, 64, 33), (2, 1, 128, 300)])
def test_attn_prefill_tensor_cores(H, KV, HD, window, which):
    """The two tensor-core prompt kernels against the plain attention: a ragged
    batch, prompts that continue earlier ones, a window, NaN in unused page tails. The tcgen05 kernel in both of
    its forms (two stages and a CTA an SM; one stage and two CTAs an SM), which give the same bits."""
    k = _k()
    k.attn_prefill_tcgen05_stages(1 if which == "tcgen05_one_stage" else 2)
    try:
        _attn_prefill_tensor_cores(k, H, KV, HD, window, which)
    finally:
        k.attn_prefill_tcgen05_stages(0)


def _attn_prefill_tensor_cores(k, H, KV, HD, window, which):
    assert k.attn_prefill_tc_supported(torch.bfloat16, H, KV, HD) and not k.attn_prefill_tc_supported(torch.bfloat16, 4, 2, 48)
    assert k.attn_prefill_tcgen05_supported(torch.bfloat16, H, KV, HD) and not k.attn_prefill_tcgen05_supported(torch.float32, H, KV, HD)
    kernel = k.attn_prefill_tc if which == "mma_sync" else k.attn_prefill_tcgen05
    rng = np.random.default_rng(18)
    lens_q, past = [7, 1, 130, 70, 64, 200, 515], [0, 0, 100, 64, 0, 313, 0]
    seqs = _attn_case(rng, lens_q, past, H, KV, HD, "bf16")
    n_pages = sum(-(-(p + n) // 64) for p, n in zip(past, lens_q)) + 3
    free = list(np.random.default_rng(20).permutation(n_pages))
    kc = torch.full((n_pages, KV, 64, HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full((n_pages, KV, 64, HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    lists = []
    for q, kk, vv in seqs:
        pages = [int(free.pop()) for _ in range(-(-kk.shape[0] // 64))]
        lists.append(pages)
        kt, vt = torch.from_numpy(kk).to(torch.bfloat16).to(DEV), torch.from_numpy(vv).to(torch.bfloat16).to(DEV)
        for i, pg in enumerate(pages):
            n = min(64, kk.shape[0] - 64 * i)
            kc[pg, :, :n] = kt[64 * i:64 * i + n].transpose(0, 1)
            vc[pg, :, :n] = vt[64 * i:64 * i + n].transpose(0, 1)
    pt = _page_table(lists)(n_pages)
    T = sum(lens_q)
    qkv = torch.from_numpy(np.concatenate([s[0].reshape(s[0].shape[0], -1) for s in seqs])).to(torch.bfloat16).to(DEV)
    out = torch.zeros((T, H * HD), dtype=torch.bfloat16, device=DEV)
    cu = torch.tensor(np.cumsum([0] + lens_q), dtype=torch.int32, device=DEV)
    kvl = torch.tensor([p + n for p, n in zip(past, lens_q)], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernel(qkv, out, len(seqs), max(lens_q), H, KV, HD, kc, vc, cu, kvl, pt, window, status)
    assert status.item() == 0
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    if which == "tcgen05_one_stage":                                             # the other form: the same bits
        k.attn_prefill_tcgen05_stages(2)
        out2 = torch.zeros_like(out)
        kernel(qkv, out2, len(seqs), max(lens_q), H, KV, HD, kc, vc, cu, kvl, pt, window, status)
        k.attn_prefill_tcgen05_stages(1)
        assert status.item() == 0 and torch.equal(out, out2)
    row = 0
    for (q, kk, vv), nq, p in zip(seqs, lens_q, past):
        ref = gqa_attention(q, kk, vv, window=window or None, q_pos=np.arange(p, p + nq), k_pos=np.arange(p + nq))
        assert rel_err(ref.reshape(nq, -1), got[row:row + nq]) < 1e-2, (nq, p)
        row += nq
    # one far key, at a page's first position and on both sides of the window's edge
    n, HDk = 400, HD
    for win, target, visible in [(0, 3, True), (0, 64, True), (120, 280, True), (120, 279, False)]:
        kk = _round(rng.standard_normal((n, KV, HDk)) * 0.1, "bf16")
        vv = _round(rng.standard_normal((n, KV, HDk)), "bf16")
        q = _round(rng.standard_normal((2, H, HDk)) * 0.1, "bf16")       # queries at positions n-2 and n-1
        kk[target, 0] = _round(q[1, 0] / np.linalg.norm(q[1, 0]) * 60.0, "bf16")
        q[1, 0] = _round(q[1, 0] * 16, "bf16")
        lst = [[6, 0, 5, 1, 4, 2, 3]]
        kc2, vc2 = _paged(kk, lst[0], 7, "bf16"), _paged(vv, lst[0], 7, "bf16")
        o2 = torch.zeros((2, H * HDk), dtype=torch.bfloat16, device=DEV)
        kernel(torch.from_numpy(q.reshape(2, -1)).to(torch.bfloat16).to(DEV), o2, 1, 2, H, KV, HDk, kc2, vc2,
               torch.tensor([0, 2], dtype=torch.int32, device=DEV), torch.tensor([n], dtype=torch.int32, device=DEV),
               _page_table(lst)(7), win, status)
        hit = np.abs(o2.float().cpu().numpy()[1, :HDk] - vv[target, 0]).max() < 0.05
        assert hit == visible, (win, target)


@pytest.mark.parametrize("M,N,K", [(2048, 4096, 1024), (2048, 1024, 2048), (130, 1000, 96), (17, 264, 64), (128, 128, 8),
                                   (300, 6144, 1024), (1000, 1024, 3072),
                                   (1500, 1096, 2112), (300, 520, 2048), (2048, 1024, 3072),   # few tiles: K in two halves
                                   (2048, 2560, 2048), (1900, 2600, 2120), (2304, 2304, 1024), # a last wave with idle SMs: k-blocks dealt out
                                   (4900, 2048, 64), (9000, 1096, 96)])    # enough tiles for pairs of CTAs; ragged edges
def test_gemm_tcgen05(M, N, K):
    """The tensor-memory product against float64, and against the library's product of the same operands."""
    from mynah_slm_b200.ops import gemm_bf16
    rng = np.random.default_rng(21)
    a = _round(rng.standard_normal((M, K)), "bf16")
    w = _round(rng.standard_normal((N, K)) * 0.05, "bf16")
    ad, wd = torch.from_numpy(a).to(torch.bfloat16).to(DEV), torch.from_numpy(w).to(torch.bfloat16).to(DEV)
    assert gemm_bf16.tcgen05_supported(M, N, K) and not gemm_bf16.tcgen05_supported(M, N, 100)
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    c32 = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
    gemm_bf16.gemm_tcgen05(ad, wd, N, 1, c32)
    assert gemm_bf16.status_word(torch.device(DEV)).item() == 0
    assert rel_err(ref, c32.cpu().numpy()) < 2e-5                         # bf16 products, fp32 sums
    c16 = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    gemm_bf16.gemm_tcgen05(ad, wd, N, 0, c16)
    if gemm_bf16.splits_k(M, N, K, torch.device(DEV)):
        # two halves of K summed at the end: fp32 sums in another order, rounded once
        assert rel_err(ref, c16.float().cpu().numpy()) < 2.5e-3           # (bf16 rounding: 2^-9 of the largest value)
        assert (c16 != c32.to(torch.bfloat16)).float().mean().item() < 0.05
    else:
        assert torch.equal(c16, c32.to(torch.bfloat16))                   # the same accumulator, rounded once
    lib32 = torch.mm(ad, wd.t(), out_dtype=torch.float32)
    assert rel_err(lib32.cpu().numpy(), c32.cpu().numpy()) < 2e-5
    # the same product again (workspace flags are left clear by every launch, and clearing them by hand is harmless)
    from mynah_slm_b200.ops import lib as klib
    klib.call("mynah_gemm_tcgen05_reset", klib.stream_ptr())
    again = torch.empty_like(c16)
    gemm_bf16.gemm_tcgen05(ad, wd, N, 0, again)
    assert torch.equal(again, c16) and gemm_bf16.status_word(torch.device(DEV)).item() == 0
    # through the dispatcher: more rows than one tile take this kernel, fewer the library's
    before = dict(gemm_bf16.counters)
    got = _k().linear(ad, wd)
    own = M >= gemm_bf16.TCGEN05_MIN_ROWS
    assert gemm_bf16.counters["own"] == before["own"] + (1 if own else 0)
    assert torch.equal(got, c16) if own else rel_err(c16.float().cpu().numpy(), got.float().cpu().numpy()) < 1e-2


@pytest.mark.parametrize("M,F,K", [(2048, 3072, 1024), (300, 200, 64), (129, 128, 96)])
def test_gemm_tcgen05_swiglu_epilogue(M, F, K):
    from mynah_slm_b200.ops import gemm_bf16
    rng = np.random.default_rng(22)
    a = _round(rng.standard_normal((M, K)), "bf16")
    w = _round(rng.standard_normal((2 * F, K)) * 0.1, "bf16")
    ad, wd = torch.from_numpy(a).to(torch.bfloat16).to(DEV), torch.from_numpy(w).to(torch.bfloat16).to(DEV)
    act = torch.empty((M, F), dtype=torch.bfloat16, device=DEV)
    gemm_bf16.gemm_tcgen05(ad, wd, F, 2, act)
    assert act.shape == (M, F) and gemm_bf16.status_word(torch.device(DEV)).item() == 0
    gu = _round(a.astype(np.float64) @ w.astype(np.float64).T, "bf16")
    assert rel_err(plain_swiglu(gu[:, :F], gu[:, F:]), act.float().cpu().numpy()) < 1.5e-2
    # against the unfused path of the library product and the separate activation kernel
    gemm_bf16.USE_TCGEN05 = False
    try:
        unfused = _k().linear_swiglu(ad, wd)
    finally:
        gemm_bf16.USE_TCGEN05 = True
    assert rel_err(unfused.float().cpu().numpy(), act.float().cpu().numpy()) < 1e-2


@pytest.mark.parametrize("H,KV,K,with_norm,with_rope,with_cache", [(16, 8, 1024, True, True, True), (3, 1, 96, True, True, True),
                                                                  (4, 2, 64, False, True, True), (5, 5, 128, True, False, False)])
def test_gemm_qkv_rope_epilogue(H, KV, K, with_norm, with_rope, with_cache):
    """The q/k/v projection whose epilogue norms, rotates and writes: against the plain parts, on a ragged
    batch with padding rows and scattered pages, and against the separate product and rope/store pass."""
    from mynah_slm_b200.ops import gemm_bf16
    k = _k()
    HD = 128
    rng = np.random.default_rng(31)
    lens, past = [150, 1, 70, 300], [0, 200, 64, 5]               # tokens this step, positions already in the cache
    T, pad = sum(lens), 23                                          # 23 padding rows at the end
    M = T + pad
    heads = H + 2 * KV if with_cache else H
    x = _round(rng.standard_normal((M, K)), "bf16")
    w = _round(rng.standard_normal((heads * HD, K)) * (1.0 / np.sqrt(K)), "bf16")
    qg = _round(1 + 0.1 * rng.standard_normal(HD), "bf16") if with_norm else None
    kg = _round(1 + 0.1 * rng.standard_normal(HD), "bf16") if with_norm else None
    dev = lambda a: None if a is None else torch.from_numpy(a).to(torch.bfloat16).to(DEV)
    eps, theta = 1e-6, 30000.0
    cos, sin = k.rope_table(700, HD, theta, DEV) if with_rope else (None, None)
    cr, sr = rope_table(HD, np.arange(700), theta)
    tok_seq = np.concatenate([[b] * n for b, n in enumerate(lens)] + [[-1] * pad]).astype(np.int32)
    tok_pos = np.concatenate([np.arange(p, p + n) for p, n in zip(past, lens)] + [np.zeros(pad)]).astype(np.int32)
    n_pages = 20
    free = list(np.random.default_rng(32).permutation(n_pages))
    lists = [[int(free.pop()) for _ in range(-(-(p + n) // 64))] for p, n in zip(past, lens)]
    pt = _page_table(lists)(n_pages)
    kc = torch.full((n_pages, KV, 64, HD), 99.0, dtype=torch.bfloat16, device=DEV)
    vc = torch.full((n_pages, KV, 64, HD), 99.0, dtype=torch.bfloat16, device=DEV)
    xd, wd = dev(x), dev(w)
    saved = gemm_bf16.USE_QKV_EPILOGUE
    gemm_bf16.USE_QKV_EPILOGUE = True
    try:
        assert gemm_bf16.qkv_rope_supported(xd, wd, H, KV, HD)
    finally:
        gemm_bf16.USE_QKV_EPILOGUE = saved
    q = gemm_bf16.gemm_qkv_rope(xd, wd, H, KV, HD, dev(qg), dev(kg), eps, cos, sin, torch.from_numpy(tok_seq).to(DEV),
                                torch.from_numpy(tok_pos).to(DEV), pt, kc if with_cache else None, vc if with_cache else None)
    assert gemm_bf16.status_word(torch.device(DEV)).item() == 0
    y = x.astype(np.float64) @ w.astype(np.float64).T             # [M, heads * HD]

    def prep(z, g):                                                # z [n, heads, HD] -> normed, rotated
        z = rms_norm(z, g, eps) if with_norm else z
        return rope_apply(z, cr[tok_pos[:T]], sr[tok_pos[:T]]) if with_rope else z
    got_q = q.float().cpu().numpy()[:T]
    ref_q = prep(y[:T, :H * HD].reshape(T, H, HD).astype(np.float32), qg).reshape(T, -1)
    assert rel_err(ref_q, got_q) < 6e-3
    if with_cache:
        ref_k = prep(y[:T, H * HD:(H + KV) * HD].reshape(T, KV, HD).astype(np.float32), kg)
        ref_v = y[:T, (H + KV) * HD:].reshape(T, KV, HD)
        kc_np, vc_np = kc.float().cpu().numpy(), vc.float().cpu().numpy()
        written = np.zeros((n_pages, 64), dtype=bool)
        for t in range(T):
            pg, off = lists[tok_seq[t]][tok_pos[t] // 64], tok_pos[t] % 64
            written[pg, off] = True
            assert rel_err(ref_k[t].reshape(1, -1), kc_np[pg, :, off].reshape(1, -1)) < 6e-3, t
            assert rel_err(ref_v[t].reshape(1, -1), vc_np[pg, :, off].reshape(1, -1)) < 6e-3, t
        assert np.all(kc_np.transpose(0, 2, 1, 3)[~written] == 99.0) and np.all(vc_np.transpose(0, 2, 1, 3)[~written] == 99.0)
        # the separate route: product, then the rope/store pass (it norms the bf16-rounded product: rounding apart)
        kc2, vc2 = torch.full_like(kc, 99.0), torch.full_like(vc, 99.0)
        qkv = k.linear(xd, wd)
        k.qk_norm_rope_store(qkv, H, KV, HD, dev(qg), dev(kg), eps, cos, sin, HD if with_rope else 0, torch.from_numpy(tok_seq).to(DEV),
                             torch.from_numpy(tok_pos).to(DEV), pt, kc2, vc2, torch.zeros(1, dtype=torch.int32, device=DEV))
        assert rel_err(qkv.float().cpu().numpy()[:T, :H * HD], got_q) < 1e-2
        assert rel_err(kc2.float().cpu().numpy().reshape(n_pages, -1), kc_np.reshape(n_pages, -1)) < 1e-2
        assert torch.equal(vc2, vc)                                # v is the rounded product either way
    # a position beyond the rotation table is reported, not used (into caches of its own: what is written there
    # is not looked at, only that nothing beyond the table was read and the status word says so)
    if with_rope:
        word = gemm_bf16.status_word(torch.device(DEV))
        assert word.item() == 0
        gemm_bf16.gemm_qkv_rope(xd, wd, H, KV, HD, dev(qg), dev(kg), eps, cos, sin, torch.from_numpy(tok_seq).to(DEV),
                                torch.from_numpy(tok_pos + 700).to(DEV), pt,
                                torch.zeros_like(kc) if with_cache else None, torch.zeros_like(vc) if with_cache else None)
        assert word.item() & 2, "a position outside the rotation table went unreported"
        word.zero_()
