"""Shared by the tests: tiny configurations, model folders in a temporary
place, and the measures that compare logits."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

# Tolerances, fixed before the first comparison was run. rel = ||a-b|| / ||a||
# per row of logits, the measure of the reference's own parity gate
# (mynah-slm tools/eval/compare.py:44-51).
FP32_REL = 1e-5      # true 32-bit engine against the plain float64-accumulating implementation
BF16_REL = 3e-2      # bfloat16 engine (bf16 activations, weights and cache; fp32 sums) against the same
# One layer of the bfloat16 engine, fed the engine's own input of that layer, against the plain implementation's
# bfloat16 mode (which rounds where the engine stores a value): the residual stream behind the layer may differ by
# one bfloat16 unit in the last place, in norm. Whole models cannot be held to this: a rounding that falls the
# other way in one layer changes the next layer's input by more than its own rounding decisions can stand, so from
# the second layer on the two are as far apart as two independently rounded runs.
BF16_LAYER_REL = 2.0 ** -8

TINY_A = dict(  # tied, small theta, group 2, head_dim 16, heads*head_dim == hidden
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=160, vocab_size=512,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256,
    hidden_act="silu", attention_bias=False, rope_scaling=None, use_sliding_window=False, sliding_window=None,
    eos_token_id=7)
TINY_B = dict(  # untied, large theta, group 3, head_dim 32, heads*head_dim != hidden
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
    num_attention_heads=6, num_key_value_heads=2, head_dim=32, intermediate_size=224, vocab_size=1000,
    rope_theta=1000000, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512,
    hidden_act="silu", attention_bias=False, rope_scaling=None, use_sliding_window=False, sliding_window=None,
    eos_token_id=[11, 13])
TINY_C = dict(  # a window on the upper layers, sizes that are no power of two, group 2 of 3 kv heads
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=4, hidden_size=80,
    num_attention_heads=6, num_key_value_heads=3, head_dim=48, intermediate_size=208, vocab_size=777,
    rope_theta=50000.0, rms_norm_eps=1e-4, tie_word_embeddings=False, max_position_embeddings=1024,
    hidden_act="silu", attention_bias=False, rope_scaling=None, use_sliding_window=True, sliding_window=40,
    max_window_layers=2, eos_token_id=5)
TINY_D = dict(  # head_dim 64, group 2: the sizes the tensor-core and fused decode kernels take
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=128,
    num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=192, vocab_size=640,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=512,
    hidden_act="silu", attention_bias=False, rope_scaling=None, use_sliding_window=False, sliding_window=None,
    eos_token_id=3)
TINY_E = dict(  # head_dim 128, one kv head for four query heads, a window from layer 1 on, untied head
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
    num_attention_heads=4, num_key_value_heads=1, head_dim=128, intermediate_size=160, vocab_size=500,
    rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512,
    hidden_act="silu", attention_bias=False, rope_scaling=None, use_sliding_window=True, sliding_window=40,
    max_window_layers=1, eos_token_id=9)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4}


def make_folder(tmp_path, name: str, dtype=torch.float32, seed=None, config=None) -> str:
    from mynah_slm_b200.registry import parse_config
    from mynah_slm_b200.weights.random_init import write_random_model
    cfg = dict(TINY[name]) if config is None else config
    typed = parse_config(cfg)
    folder = os.path.join(str(tmp_path), f"tiny_{name}_{'f32' if dtype == torch.float32 else 'bf16'}")
    write_random_model(folder, typed, SEEDS.get(name, 0) if seed is None else seed, dtype)
    return folder


def rel_err(ref: np.ndarray, got: np.ndarray) -> float:
    """Largest per-row ||ref-got|| / ||ref||."""
    ref = np.asarray(ref, dtype=np.float64).reshape(-1, ref.shape[-1])
    got = np.asarray(got, dtype=np.float64).reshape(-1, got.shape[-1])
    num = np.linalg.norm(ref - got, axis=-1)
    den = np.maximum(np.linalg.norm(ref, axis=-1), 1e-30)
    return float(np.max(num / den))


def assert_close(ref, got, tol, what=""):
    assert np.asarray(ref).shape == np.asarray(got).shape, f"{what}: shapes {np.asarray(ref).shape} vs {np.asarray(got).shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite logits"
    r = rel_err(ref, got)
    if r > tol:
        ref2 = np.asarray(ref).reshape(-1, np.asarray(ref).shape[-1])
        got2 = np.asarray(got).reshape(-1, np.asarray(got).shape[-1])
        rows = np.linalg.norm(ref2 - got2, axis=-1) / np.maximum(np.linalg.norm(ref2, axis=-1), 1e-30)
        first = int(np.argmax(rows > tol))
        raise AssertionError(f"{what}: rel error {r:.3e} > {tol:.0e}; first wrong row {first} of {len(rows)} "
                             f"(rel {rows[first]:.3e})")


def prompts_for(name: str, lengths, seed=123):
    rng = np.random.default_rng(seed)
    V = TINY[name]["vocab_size"]
    return [rng.integers(0, V, size=n).tolist() for n in lengths]
