"""The plain sampler against the reference's own C sampler, compiled here from the reference checkout with gcc:
identical logits, parameters and seeds must give identical tokens, draw after draw, with the ring of accepted
tokens carried along. Skipped where the checkout or a C compiler is absent; the plain sampler then rests on the
reading of src/sampler.c that its functions cite."""
import ctypes
import os
import shutil
import subprocess

import numpy as np
import pytest

from plain.sampler import PlainSampler

SRC = os.environ.get("MYNAH_REFERENCE", "/root/reference") + "/src/sampler.c"


class Params(ctypes.Structure):
    # mynah-slm src/sampler.h:13-26
    _fields_ = [("temp", ctypes.c_float), ("top_k", ctypes.c_uint32), ("top_p", ctypes.c_float), ("min_p", ctypes.c_float),
                ("repeat_penalty", ctypes.c_float), ("freq_penalty", ctypes.c_float), ("presence_penalty", ctypes.c_float),
                ("penalty_window", ctypes.c_uint32), ("seed", ctypes.c_uint64)]


@pytest.fixture(scope="module")
def c_sampler(tmp_path_factory):
    cc = shutil.which("gcc") or shutil.which("cc")
    if not os.path.isfile(SRC) or cc is None:
        pytest.skip("the reference checkout or a C compiler is not here")
    out = str(tmp_path_factory.mktemp("ref_sampler") / "libref_sampler.so")
    r = subprocess.run([cc, "-std=c11", "-O2", "-shared", "-fPIC", "-D_DEFAULT_SOURCE", "-I", os.path.dirname(SRC), SRC, "-o", out, "-lm"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        pytest.skip(f"the reference's sampler does not compile here: {r.stderr[-300:]}")
    lib = ctypes.CDLL(out)
    lib.mynah_slm_sampler_new.restype = ctypes.c_void_p
    lib.mynah_slm_sampler_new.argtypes = [ctypes.POINTER(Params), ctypes.c_uint32]
    lib.mynah_slm_sampler_free.argtypes = [ctypes.c_void_p]
    lib.mynah_slm_sampler_accept.argtypes = [ctypes.c_void_p, ctypes.c_uint32]
    lib.mynah_slm_sample.restype = ctypes.c_uint32
    lib.mynah_slm_sample.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)]
    lib.mynah_slm_sampler_defaults.argtypes = [ctypes.POINTER(Params)]
    return lib


SETTINGS = [
    dict(temp=0.0),
    dict(temp=0.0, repeat_penalty=1.3, freq_penalty=0.2, presence_penalty=0.1, penalty_window=8),
    dict(temp=0.8, top_k=0, top_p=1.0, seed=1),
    dict(temp=0.6, top_k=20, top_p=0.95, seed=0),
    dict(temp=1.3, top_k=5, top_p=1.0, min_p=0.0, seed=7),
    dict(temp=1.0, top_k=0, top_p=0.5, seed=123456789),
    dict(temp=0.7, top_k=0, top_p=1.0, min_p=0.2, seed=3),
    dict(temp=0.9, top_k=50, top_p=0.9, min_p=0.05, repeat_penalty=1.2, freq_penalty=0.1, presence_penalty=0.3, penalty_window=16, seed=11),
    dict(temp=2.5, top_k=1, top_p=0.3, seed=5),
]


def test_defaults_are_the_reference_s(c_sampler):
    p = Params()
    c_sampler.mynah_slm_sampler_defaults(ctypes.byref(p))
    mine = PlainSampler()
    assert (round(p.temp, 6), p.top_k, round(p.top_p, 6), p.min_p, p.repeat_penalty, p.penalty_window) == \
        (round(mine.temp, 6), mine.top_k, round(mine.top_p, 6), mine.min_p, mine.repeat_penalty, mine.window)


@pytest.mark.parametrize("setting", SETTINGS, ids=[str(i) for i in range(len(SETTINGS))])
@pytest.mark.parametrize("vocab", [17, 512, 5000])
def test_plain_sampler_draws_what_the_reference_draws(c_sampler, setting, vocab):
    full = dict(temp=0.6, top_k=20, top_p=0.95, min_p=0.0, repeat_penalty=1.0, freq_penalty=0.0, presence_penalty=0.0,
                penalty_window=64, seed=0)
    full.update(setting)
    p = Params(**full)
    ref = c_sampler.mynah_slm_sampler_new(ctypes.byref(p), vocab)
    assert ref
    mine = PlainSampler(**full)
    rng = np.random.default_rng(vocab * 31 + len(str(setting)))
    try:
        for t in rng.integers(0, vocab, size=5):                 # a prompt goes into the ring first
            c_sampler.mynah_slm_sampler_accept(ref, int(t))
            mine.accept(int(t))
        for step in range(40):
            scale = [0.5, 3.0, 10.0][step % 3]
            logits = (rng.standard_normal(vocab) * scale).astype(np.float32)
            if step % 7 == 3:
                logits[rng.integers(0, vocab, size=3)] = logits.max()         # ties
            a, b = logits.copy(), logits.copy()
            want = int(c_sampler.mynah_slm_sample(ref, a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))))
            got = mine.sample(b)
            assert got == want, f"step {step}: plain {got}, reference {want}"
            c_sampler.mynah_slm_sampler_accept(ref, want)
            mine.accept(got)
    finally:
        c_sampler.mynah_slm_sampler_free(ref)
