"""The decode attention through `mynah_attn_decode_no_alloc`, the entry point
for callers that must not allocate device memory (a process that has given the
whole device to its own pool; a loop that cannot afford the stall of an
allocation). It is called here the way such a caller would call it: through
the exported C symbol, with pointers, and with no scratch buffer. Its output
must equal that of `mynah_attn_decode` with caller-provided scratch, on two
calls in a row (the built-in array keeps the first call's contents during the
second), and a problem too large for the built-in array must be refused.

This file sorts last so that a run that stops at the first failure has run
every other test before it.
"""
import ctypes
from ctypes import c_int, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
MAX_FLOATS = 4 * 1024 * 1024


def _symbol():
    from mynah_slm_b200.ops import lib
    handle = lib.load()
    fn = handle.mynah_attn_decode_no_alloc
    fn.restype = c_int
    P = c_void_p
    fn.argtypes = [P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P, P, P, P, P, c_int, c_int, c_int, P, P]
    return handle, fn


def _case(seed, B, H, KV, HD, lens, dtype):
    g = torch.Generator(device="cpu").manual_seed(seed)
    n_pages = sum(-(-n // 64) for n in lens) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    lists = []
    for n in lens:
        lists.append([perm.pop() for _ in range(-(-n // 64))])
    indptr = torch.tensor(np.cumsum([0] + [len(l) for l in lists]), dtype=torch.int32, device=DEV)
    ids = torch.tensor([p for l in lists for p in l], dtype=torch.int32, device=DEV)
    base = torch.zeros(B, dtype=torch.int32, device=DEV)
    kc = torch.randn((n_pages, KV, 64, HD), generator=g).to(dtype).to(DEV)
    vc = torch.randn((n_pages, KV, 64, HD), generator=g).to(dtype).to(DEV)
    q = torch.randn((B, H * HD), generator=g).to(dtype).to(DEV)
    kvl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    return q, kc, vc, kvl, indptr, ids, base, n_pages


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_no_alloc_entry_point_matches_the_allocating_one(dtype):
    from mynah_slm_b200.ops import kernels
    from mynah_slm_b200.ops.kernels import PageTableView
    handle, fn = _symbol()
    code = {torch.float32: 0, torch.bfloat16: 1}[dtype]
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # two calls in a row, of different shapes, the second smaller than the first:
    # what the first left in the built-in array must not leak into the second
    for seed, (B, H, KV, HD, lens, window) in enumerate([(5, 8, 2, 128, [300, 64, 1, 517, 130], 0),
                                                         (3, 6, 3, 48, [90, 200, 7], 40)]):
        q, kc, vc, kvl, indptr, ids, base, n_pages = _case(seed, B, H, KV, HD, lens, dtype)
        splits = max(-(-n // 64) for n in lens)
        want = torch.zeros((B, H * HD), dtype=dtype, device=DEV)
        scratch = torch.empty(kernels.attn_decode_scratch_floats(B, H, HD, splits), dtype=torch.float32, device=DEV)
        kernels.attn_decode(q, want, B, H, KV, HD, kc, vc, kvl, PageTableView(indptr, ids, base, n_pages), window,
                            splits, scratch, status)
        got = torch.full((B, H * HD), 3.0, dtype=dtype, device=DEV)
        rc = fn(q.data_ptr(), got.data_ptr(), code, B, H, KV, HD, H * HD, H * HD, kc.data_ptr(), vc.data_ptr(),
                kvl.data_ptr(), indptr.data_ptr(), ids.data_ptr(), base.data_ptr(), n_pages, window, splits,
                status.data_ptr(), stream)
        assert rc == 0, handle.mynah_last_error().decode()
        torch.cuda.synchronize()
        assert status.item() == 0
        tol = 3e-6 if dtype == torch.float32 else 1e-2
        err = (got.float() - want.float()).norm() / want.float().norm()
        assert err.item() <= tol, f"call {seed}: rel error {err.item():.3e}"
        assert torch.equal(got, want), f"call {seed}: same kernels, same order of sums, other bits"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    handle, fn = _symbol()
    B, H, HD, splits = 64, 32, 128, 64
    assert B * H * splits * (HD + 2) > MAX_FLOATS
    d = torch.zeros(16, dtype=torch.int32, device=DEV)
    rc = fn(d.data_ptr(), d.data_ptr(), 1, B, H, 8, HD, H * HD, H * HD, d.data_ptr(), d.data_ptr(), d.data_ptr(),
            d.data_ptr(), d.data_ptr(), d.data_ptr(), 1, 0, splits, d.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = handle.mynah_last_error().decode()
    assert "floats of scratch" in msg and str(MAX_FLOATS) in msg
