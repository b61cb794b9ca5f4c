"""The reference arm of bench.py: builds the unmodified reference (mynah-org/mynah-slm, a C engine for the CPU)
from a copy of its checkout under baseline/_ref, writes a random-weights GGUF of the benchmark's shape with the
`gguf` package, and times the reference's own load / state / forward calls on the benchmark's workload through a
small C harness (baseline/ref_harness.c).

The reference has no Python package (`pip install` of its checkout fails: no setup.py, no pyproject.toml), no
GPU path and no batch: it runs one sequence at a time, token by token, prompts included. Its `make` stops at an
OpenBLAS guard although no source uses BLAS, so the objects are compiled here by hand with the flags its Makefile
gives them. What this arm measures is therefore the same metric (decoded tokens a second for 8 requests with
2,048-token prompts) on the host's CPU cores; it says so with "device": "cpu".
"""
from __future__ import annotations

import glob
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SRC = os.path.join(REF, "src")
EXE = os.path.join(REF, "ref_harness")


class Unavailable(RuntimeError):
    pass


def _find_source() -> str:
    if os.path.isfile(os.path.join(SRC, "src", "arch_qwen3.c")):
        return SRC
    origin = os.environ.get("MYNAH_REFERENCE", "/root/reference")
    if not os.path.isfile(os.path.join(origin, "src", "arch_qwen3.c")):
        raise Unavailable(f"the reference checkout is neither under baseline/_ref/src nor at {origin}")
    os.makedirs(REF, exist_ok=True)
    shutil.copytree(origin, SRC)
    return SRC


def build() -> str:
    """The harness linked against the reference's own objects; built once, kept under baseline/_ref."""
    src = _find_source()
    stamp = os.path.join(REF, "harness_stamp")
    import hashlib
    with open(os.path.join(HERE, "ref_harness.c"), "rb") as f:
        want = hashlib.sha256(f.read()).hexdigest()
    if os.path.isfile(EXE) and os.path.isfile(stamp) and open(stamp).read() == want:
        return EXE
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        raise Unavailable("gcc is absent: the reference cannot be compiled")
    ingot = os.path.join(src, "third_party", "ingot")
    r = subprocess.run(["make", "lib", f"CC={cc}"], cwd=ingot, capture_output=True, text=True)
    if r.returncode != 0 or not os.path.isfile(os.path.join(ingot, "libingot.a")):
        raise Unavailable("the reference's container library (third_party/ingot) does not build here: " + r.stderr[-200:])
    sources = [f for f in sorted(glob.glob(os.path.join(src, "src", "*.c")))]
    cmd = [cc, "-std=c11", "-O2", "-D_DEFAULT_SOURCE", '-DMYNAH_SLM_BUILD="bench"', "-iquote", os.path.join(src, "src"),
           "-I", os.path.join(src, "include"), "-I", os.path.join(ingot, "include"), *sources, os.path.join(HERE, "ref_harness.c"),
           os.path.join(ingot, "libingot.a"), "-lpthread", "-lm", "-o", EXE]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise Unavailable("the reference's sources do not compile here: " + r.stderr[-300:])
    with open(stamp, "w") as f:
        f.write(want)
    return EXE


def write_gguf(path: str, cfg: dict, seed: int) -> None:
    """The benchmark's random model (this package's random weights, bfloat16 values) as a GGUF the reference
    loads: matrices as F16 (every bfloat16 value of this size is an F16 value), gains as F32, under the tensor
    names of the reference's loader (src/model.c:154-164, 193-198)."""
    try:
        import gguf
    except ImportError:
        raise Unavailable("the gguf package is absent: no checkpoint in the reference's format can be written") from None
    import numpy as np
    import torch

    sys.path.insert(0, os.path.dirname(HERE))
    from mynah_slm_b200 import parse_config
    from mynah_slm_b200.engine.model import Model
    from mynah_slm_b200.weights.random_init import _wanted, host_tensor

    typed = parse_config(cfg)
    w = gguf.GGUFWriter(path, "qwen3")
    w.add_block_count(cfg["num_hidden_layers"])
    w.add_embedding_length(cfg["hidden_size"])
    w.add_feed_forward_length(cfg["intermediate_size"])
    w.add_head_count(cfg["num_attention_heads"])
    w.add_head_count_kv(cfg["num_key_value_heads"])
    w.add_key_length(cfg["head_dim"])
    w.add_value_length(cfg["head_dim"])
    w.add_context_length(cfg["max_position_embeddings"])
    w.add_layer_norm_rms_eps(float(cfg["rms_norm_eps"]))
    w.add_rope_freq_base(float(cfg["rope_theta"]))
    eos = cfg.get("eos_token_id", 0)
    w.add_eos_token_id(int(eos[0] if isinstance(eos, (list, tuple)) else eos or 0))
    names = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight", "lm_head.weight": "output.weight"}
    per_layer = {"input_layernorm.weight": "attn_norm.weight", "self_attn.q_proj.weight": "attn_q.weight",
                 "self_attn.k_proj.weight": "attn_k.weight", "self_attn.v_proj.weight": "attn_v.weight",
                 "self_attn.o_proj.weight": "attn_output.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
                 "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight",
                 "self_attn.q_norm.weight": "attn_q_norm.weight", "self_attn.k_norm.weight": "attn_k_norm.weight"}
    for ts in _wanted(Model(typed.model_spec())):
        t = host_tensor(ts, seed, torch.bfloat16).to(torch.float32).numpy()
        if ts.name in names:
            name = names[ts.name]
        else:
            _, _, i, rest = ts.name.split(".", 3)
            name = f"blk.{i}.{per_layer[rest]}"
        w.add_tensor(name, t.astype(np.float32) if ts.role == "gain" else t.astype(np.float16))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def run(cfg: dict, n_seqs: int, prompt_len: int, warmup: int, steps: int, budget_s: float = 900.0) -> dict:
    """Returns {"decode_tokens", "decode_s", "prompt_tokens", "prompt_s", "threads"}; raises Unavailable with the reason."""
    exe = build()
    threads = os.cpu_count() or 1
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "random.gguf")
        t0 = time.time()
        write_gguf(path, cfg, seed=2)
        wrote_s = time.time() - t0
        r = subprocess.run([exe, path, str(n_seqs), str(prompt_len), str(warmup), str(steps), str(threads), "48", str(budget_s)],
                           capture_output=True, text=True, timeout=budget_s * 1.5 + 120)
    words = r.stdout.split()
    if r.returncode != 0 or not words:
        raise Unavailable("the reference's harness failed: " + (r.stdout + r.stderr)[-300:])
    if words[0] == "too_slow":
        raise Unavailable(f"the run cannot fit the time limit: the reference processes prompts token by token at {words[1]} tokens a "
                          f"second on this host's {threads} cores, so {n_seqs} prompts of {prompt_len} tokens and the decode steps would "
                          f"take about {words[2]} s (limit {budget_s:.0f} s)")
    if words[0] != "ok":
        raise Unavailable("the reference's harness said: " + r.stdout[-300:])
    return {"decode_tokens": int(words[1]), "decode_s": float(words[2]), "prompt_tokens": int(words[3]), "prompt_s": float(words[4]),
            "threads": threads, "gguf_written_s": round(wrote_s, 1)}


if __name__ == "__main__":
    print(build())
