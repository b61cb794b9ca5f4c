"""The random-weights mode: the host's fill against the plain function element by element, a folder that reads
back as written, and that the numbers are what they claim to be (normal, of the stated mean and deviation)."""
import numpy as np
import pytest
import torch

from helpers import TINY, make_folder
from plain import random_weights as plain_rw
from plain.model import read_folder


def _specs(name):
    from mynah_slm_b200.engine.model import Model
    from mynah_slm_b200.registry import parse_config
    from mynah_slm_b200.weights.random_init import _wanted
    return _wanted(Model(parse_config(dict(TINY[name])).model_spec()))


def _plain_tensor(ts, seed, bf16):
    mean = 1.0 if ts.init == "gain" else 0.0
    n = int(np.prod(ts.shape))
    return plain_rw.values(seed, ts.name, np.arange(n), mean, ts.std, bf16).reshape(ts.shape)


@pytest.mark.parametrize("name,seed", [("A", 0), ("B", 1), ("C", 12345678901234567)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_host_fill_equals_the_plain_function_bit_for_bit(name, seed, dtype):
    from mynah_slm_b200.weights.random_init import host_tensor
    for ts in _specs(name):
        got = host_tensor(ts, seed, dtype).to(torch.float32).numpy()
        want = _plain_tensor(ts, seed, dtype == torch.bfloat16)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), ts.name


def test_a_written_folder_reads_back_as_made(tmp_path):
    for name, dtype in (("A", torch.float32), ("B", torch.bfloat16)):
        folder = make_folder(tmp_path, name, dtype, seed=77)
        _, tensors = read_folder(folder)
        specs = _specs(name)
        assert sorted(tensors) == sorted(ts.name for ts in specs)
        for ts in specs:
            want = _plain_tensor(ts, 77, dtype == torch.bfloat16)
            assert np.array_equal(tensors[ts.name].view(np.uint32), want.view(np.uint32)), ts.name


def test_the_numbers_are_normal():
    z = plain_rw.normal(3, "some.tensor", np.arange(400000))
    assert abs(z.mean()) < 5e-3 and abs(z.std() - 1.0) < 5e-3
    assert abs(np.mean(z ** 3)) < 2e-2 and abs(np.mean(z ** 4) - 3.0) < 5e-2          # skewness, kurtosis
    assert 0.6815 < np.mean(np.abs(z) < 1.0) < 0.6840 and 4.3 < z.max() < 6.5 and -6.5 < z.min() < -4.3
    # neighbouring elements, other tensors and other seeds are unrelated
    assert abs(np.corrcoef(z[:-1], z[1:])[0, 1]) < 5e-3
    assert abs(np.corrcoef(z, plain_rw.normal(3, "some.tensor2", np.arange(400000)))[0, 1]) < 5e-3
    assert abs(np.corrcoef(z, plain_rw.normal(4, "some.tensor", np.arange(400000)))[0, 1]) < 5e-3
    # element by element: any subset gives the same numbers
    idx = np.array([5, 399999, 0, 123456])
    assert np.array_equal(plain_rw.normal(3, "some.tensor", idx), z[idx])
    # the cosine and the logarithm the numbers are built from, against the library's
    k = np.arange(0, 1 << 32, 99991, dtype=np.uint64)
    assert np.max(np.abs(plain_rw.cos_turn(k) - np.cos(2 * np.pi * k.astype(np.float64) / 4294967296.0))) < 1e-15
    u = (k.astype(np.float64) + 1.0) / 4294967296.0
    assert np.max(np.abs(plain_rw.log_of(u) - np.log(u))) < 1e-14
