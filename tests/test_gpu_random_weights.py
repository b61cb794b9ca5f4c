"""Random weights made on the device: the kernel against the plain function bit for bit, and an engine built
with no file against an engine that loads the folder the host wrote from the same configuration and seed."""
import numpy as np
import pytest
import torch

from helpers import TINY, make_folder, prompts_for
from plain import random_weights as plain_rw

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,seed", [("A", 0), ("B", 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_device_fill_equals_the_plain_function_bit_for_bit(name, seed, dtype):
    from mynah_slm_b200.engine.model import Model
    from mynah_slm_b200.registry import parse_config
    from mynah_slm_b200.weights.random_init import _wanted, device_tensor
    for ts in _wanted(Model(parse_config(dict(TINY[name])).model_spec())):
        got = device_tensor(ts, seed, dtype, "cuda:0").to(torch.float32).cpu().numpy()
        mean = 1.0 if ts.init == "gain" else 0.0
        want = plain_rw.values(seed, ts.name, np.arange(got.size), mean, ts.std, dtype == torch.bfloat16).reshape(ts.shape)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), ts.name


def test_device_fill_of_an_odd_large_tensor():
    """More elements than one pass of the grid covers, not a multiple of anything: every element is written once,
    and elements far into the tensor are those of the plain function."""
    from mynah_slm_b200.parts.base import TensorSpec
    from mynah_slm_b200.weights.random_init import device_tensor
    n = 148 * 16 * 256 * 3 + 12345
    ts = TensorSpec("big.odd", (n,), init="gain", std=0.1)
    got = device_tensor(ts, 9, torch.float32, "cuda:0").cpu().numpy()
    idx = np.concatenate([np.arange(5000), np.arange(n - 5000, n), np.random.default_rng(0).integers(0, n, 20000)])
    want = plain_rw.values(9, "big.odd", idx, 1.0, 0.1, False)
    assert np.array_equal(got[idx].view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("E", "bfloat16")])
def test_engine_with_random_weights_and_no_file(tmp_path, name, dtype):
    from mynah_slm_b200.engine.engine import Engine, StepEntry
    wdt = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_folder(tmp_path, name, wdt, seed=31)
    a = Engine.from_folder(folder, dtype=dtype, max_tokens=256)
    b = Engine.random(dict(TINY[name]), seed=31, dtype=dtype, max_tokens=256)
    toks = prompts_for(name, [70], seed=1)[0]
    outs = []
    for eng in (a, b):
        s = eng.open_sequence()
        outs.append(eng.step([StepEntry(s, toks, range(len(toks)))]).cpu())
        eng.check_status()
    assert torch.equal(outs[0], outs[1])
