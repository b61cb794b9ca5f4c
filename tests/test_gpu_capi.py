"""The C interface (include/mynah_slm_b200.h) driven by a C program that this test compiles: it loads a random
folder (or makes the weights from a configuration and a seed), steps Tiny-A and Tiny-B whole, token by token
and as an unequal batch whose shorter requests end earlier, generates through mynah_generate with a callback,
and meets every error with a code and a message. The logits are compared with the plain implementation; the
library itself must not write a byte to stdout or stderr."""
import json
import os
import shutil
import subprocess

import numpy as np
import pytest
import torch

from helpers import BF16_REL, FP32_REL, TINY, assert_close, make_folder, prompts_for
from plain.model import PlainQwen3
from plain.sampler import PlainSampler, plain_generate

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def program(tmp_path_factory):
    from mynah_slm_b200.csrc.build import capi_library_path
    lib = capi_library_path()
    cc = shutil.which("gcc") or shutil.which("cc")
    assert cc, "no C compiler"
    exe = str(tmp_path_factory.mktemp("capi") / "capi_program")
    r = subprocess.run([cc, "-std=c11", "-O1", "-Wall", "-I", os.path.join(ROOT, "mynah_slm_b200", "include"),
                        os.path.join(HERE, "capi", "capi_program.c"), "-o", exe, lib, f"-Wl,-rpath,{os.path.dirname(lib)}"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def _run(exe, args, tmp_path):
    env = dict(os.environ, MYNAH_SLM_B200_ROOT=ROOT, HOME=str(tmp_path))
    p = subprocess.run([exe, *args], capture_output=True, text=True, timeout=900, env=env)
    assert p.stderr == "", f"the library wrote to stderr: {p.stderr[-2000:]}"
    return p


def _script(steps):
    out = [len(steps)]
    for step_id, entries, end in steps:
        out += [step_id, len(entries)]
        for req, tokens, want in entries:
            out += [req, len(tokens), *tokens, len(want), *want]
        out += [len(end), *end]
    return np.asarray(out, dtype="<i4")


@pytest.mark.parametrize("name,dtype,model", [("A", "float32", "folder"), ("B", "bfloat16", "folder"), ("B", "float32", "random")])
def test_c_program_steps_whole_one_by_one_and_in_unequal_batches(program, tmp_path, name, dtype, model):
    wdt = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_folder(tmp_path, name, wdt, seed=21)
    plain = PlainQwen3.from_folder(folder)
    if model == "random":
        cfg = tmp_path / "cfg.json"
        cfg.write_text(json.dumps(TINY[name]))
        model_arg = f"random:{cfg}:21"
    else:
        model_arg = folder
    V = TINY[name]["vocab_size"]
    tol = FP32_REL if dtype == "float32" else BF16_REL
    a, b, c = prompts_for(name, [70, 9, 33], seed=5)
    steps, expect = [], {}
    sid = 0
    # each request alone and whole
    for r, q in enumerate((a, b, c)):
        steps.append((sid, [(r, q, list(range(len(q))))], [r]))
        expect[sid] = plain.forward(q)
        sid += 1
    # the last 32 tokens one by one
    steps.append((sid, [(0, a[:-32], [len(a) - 33])], []))
    expect[sid] = plain.forward(a)[len(a) - 33:len(a) - 32]
    sid += 1
    for t in range(len(a) - 32, len(a)):
        steps.append((sid, [(0, a[t:t + 1], [0])], [0] if t == len(a) - 1 else []))
        expect[sid] = plain.forward(a)[t:t + 1]
        sid += 1
    # an unequal batch; b ends after two decode steps, c after one; then a second batch in the freed slots
    ra, rb, rc = plain.forward(a), plain.forward(b), plain.forward(c)
    steps.append((sid, [(0, a[:60], [0, 59]), (1, b[:6], [5]), (2, c[:31], [30])], []))
    expect[sid] = np.stack([ra[0], ra[59], rb[5], rc[30]]); sid += 1
    steps.append((sid, [(0, a[60:61], [0]), (1, b[6:7], [0]), (2, c[31:32], [0])], [2]))
    expect[sid] = np.stack([ra[60], rb[6], rc[31]]); sid += 1
    steps.append((sid, [(0, a[61:62], [0]), (1, b[7:8], [])], [1]))
    expect[sid] = ra[61:62]; sid += 1
    steps.append((sid, [(0, a[62:63], [0])], [0]))
    expect[sid] = ra[62:63]; sid += 1
    steps.append((sid, [(3, c, [len(c) - 1]), (4, b, [0, len(b) - 1])], [3, 4]))
    expect[sid] = np.stack([rc[-1], rb[0], rb[-1]]); sid += 1
    script = tmp_path / "script.bin"
    _script(steps).tofile(script)
    out = tmp_path / "out"
    out.mkdir()
    p = _run(program, ["replay", model_arg, dtype, str(64 * 4), str(script), str(out)], tmp_path)
    assert p.returncode == 0, p.stdout[-3000:]
    lines = p.stdout.strip().splitlines()
    assert lines[0] == (f"vocab {V} layers {TINY[name]['num_hidden_layers']} hidden {TINY[name]['hidden_size']} "
                        f"positions {TINY[name]['max_position_embeddings']} page 64 free 256")
    assert lines[1:-1] == [f"done {i}" for i in range(sid)] and lines[-1] == "free 256"
    for i, ref in expect.items():
        got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
        assert_close(ref, got, tol, f"{name} {dtype} C step {i}")


def test_c_program_generates(program, tmp_path):
    folder = make_folder(tmp_path, "A", torch.float32, seed=22)
    plain = PlainQwen3.from_folder(folder)
    prompts = prompts_for("A", [7, 1, 12], seed=6)
    flat = [len(prompts)]
    for q in prompts:
        flat += [len(q), *q]
    path = tmp_path / "prompts.bin"
    np.asarray(flat, dtype="<i4").tofile(path)
    p = _run(program, ["generate", folder, "float32", str(64 * 4), str(path), "8", "0", "0", "-1"], tmp_path)
    assert p.returncode == 0, p.stdout[-3000:]
    lines = p.stdout.strip().splitlines()
    for i, q in enumerate(prompts):
        want, _ = plain_generate(plain, q, 8, PlainSampler(temp=0))
        assert lines[i] == f"request {i} finish 1 produced 8 tokens " + " ".join(str(t) for t in want)
    assert lines[3] == f"callback calls 24 emitted 24 prompt {sum(len(q) for q in prompts)} generated 24 decode_s_positive 1"
    assert lines[4] == "stopped rc 7 finish 3 n 3"
    # a stop token ends a request before it is emitted
    first = plain_generate(plain, prompts[0], 8, PlainSampler(temp=0))[0]
    stop_at = next((j for j in range(1, 8) if first[j] not in first[:j]), 0)
    p = _run(program, ["generate", folder, "float32", str(64 * 4), str(path), "8", "0", "0", str(first[stop_at])], tmp_path)
    line = p.stdout.strip().splitlines()[0]
    assert line == f"request 0 finish 0 produced {stop_at + 1} tokens" + "".join(f" {t}" for t in first[:stop_at])


def test_c_program_meets_errors_with_codes_and_messages(program, tmp_path):
    folder = make_folder(tmp_path, "A", torch.float32)
    p = _run(program, ["errors", folder], tmp_path)
    assert p.returncode == 0, p.stdout[-3000:]
    lines = p.stdout.strip().splitlines()
    assert lines[0].startswith("missing folder: rc 1 engine null message: ") and "/nonexistent/folder" in lines[0]
    assert lines[1].startswith("bad dtype: rc 1 message: ") and "float16" in lines[1]
    assert lines[2].startswith("token out of range: rc 1 message: ") and "outside the vocabulary" in lines[2]
    assert lines[3].startswith("unknown slot: rc 1 message: ") and "not open" in lines[3]
    assert lines[4].startswith("cache full: rc 4 message: ") and "full" in lines[4]
    assert lines[5] == "no buffer: rc 4 length 0"
    assert lines[6].startswith("close unknown: rc 1 message: ") and "not open" in lines[6]
