"""Weights and tokens of the golden comparison, from numpy's seeded generator
(so the test can rebuild them without the file that made the outputs)."""
import numpy as np

CONFIGS = {
    "A": dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              intermediate_size=160, vocab_size=512, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, n_tokens=12, seed=0),
    "B": dict(num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
              intermediate_size=224, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-5,
              tie_word_embeddings=False, n_tokens=20, seed=1),
}


def build(name):
    c = CONFIGS[name]
    rng = np.random.default_rng(c["seed"])
    D, H, KV, HD, F, V = (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                          c["intermediate_size"], c["vocab_size"])
    mat = lambda *s: (rng.standard_normal(s) * 0.02).astype(np.float32)
    gain = lambda n: (1.0 + rng.standard_normal(n) * 0.1).astype(np.float32)
    t = {"model.embed_tokens.weight": mat(V, D), "model.norm.weight": gain(D)}
    if not c["tie_word_embeddings"]:
        t["lm_head.weight"] = mat(V, D)
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = gain(D)
        t[p + "self_attn.q_proj.weight"] = mat(H * HD, D)
        t[p + "self_attn.k_proj.weight"] = mat(KV * HD, D)
        t[p + "self_attn.v_proj.weight"] = mat(KV * HD, D)
        t[p + "self_attn.o_proj.weight"] = mat(D, H * HD)
        t[p + "self_attn.q_norm.weight"] = gain(HD)
        t[p + "self_attn.k_norm.weight"] = gain(HD)
        t[p + "post_attention_layernorm.weight"] = gain(D)
        t[p + "mlp.gate_proj.weight"] = mat(F, D)
        t[p + "mlp.up_proj.weight"] = mat(F, D)
        t[p + "mlp.down_proj.weight"] = mat(D, F)
    tokens = rng.integers(0, V, size=c["n_tokens"])
    return c, t, tokens
