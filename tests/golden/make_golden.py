"""Makes tests/golden/oracle_logits.npz: the logits of the REFERENCE's own
numpy model code (mynah-slm tools/oracle/model.py, imported from the reference
checkout, not copied) on two tiny random models. tests/test_plain.py compares
the plain implementation with them.

Run once, where the reference checkout is: python tests/golden/make_golden.py [path/to/mynah-slm]

The oracle reads GGUF files; here its `Qwen3Model` is given an object with the
same attributes (config, embed, out_norm, layers) built from the arrays of
golden_common.build, so no container is involved. The oracle's head is tied
only (tools/oracle/model.py:147); for the untied model the logits are its
dumped final norm times lm_head^T.
"""
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from golden_common import CONFIGS, build  # noqa: E402


def main():
    if len(sys.argv) < 2 and not os.environ.get("MYNAH_REFERENCE"):
        raise SystemExit("usage: make_golden.py <checkout of mynah-org/mynah-slm>   (or set MYNAH_REFERENCE)")
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ["MYNAH_REFERENCE"]
    sys.path.insert(0, os.path.join(ref, "tools"))
    from oracle.model import Qwen3Model
    out = {}
    for name in CONFIGS:
        c, t, tokens = build(name)
        cfg = types.SimpleNamespace(
            n_layers=c["num_hidden_layers"], d_model=c["hidden_size"], d_ff=c["intermediate_size"],
            n_heads=c["num_attention_heads"], n_kv_heads=c["num_key_value_heads"], head_dim=c["head_dim"],
            rms_eps=c["rms_norm_eps"], rope_theta=c["rope_theta"],
            q_dim=c["num_attention_heads"] * c["head_dim"], kv_dim=c["num_key_value_heads"] * c["head_dim"])
        layers = []
        for i in range(c["num_hidden_layers"]):
            p = f"model.layers.{i}."
            layers.append({"attn_norm": t[p + "input_layernorm.weight"], "wq": t[p + "self_attn.q_proj.weight"],
                           "wk": t[p + "self_attn.k_proj.weight"], "wv": t[p + "self_attn.v_proj.weight"],
                           "wo": t[p + "self_attn.o_proj.weight"], "q_norm": t[p + "self_attn.q_norm.weight"],
                           "k_norm": t[p + "self_attn.k_norm.weight"], "ffn_norm": t[p + "post_attention_layernorm.weight"],
                           "gate": t[p + "mlp.gate_proj.weight"], "up": t[p + "mlp.up_proj.weight"],
                           "down": t[p + "mlp.down_proj.weight"]})
        w = types.SimpleNamespace(config=cfg, embed=t["model.embed_tokens.weight"], out_norm=t["model.norm.weight"],
                                  layers=layers)
        dump = {"_layers": (0,)}
        logits = Qwen3Model(w).forward(tokens, dump)
        if not c["tie_word_embeddings"]:
            logits = dump["final_norm"] @ t["lm_head.weight"].T
        out[f"{name}_logits"] = logits.astype(np.float32)
        out[f"{name}_layer0"] = dump["layer0"].astype(np.float32)
        out[f"{name}_tokens"] = tokens.astype(np.int64)
        print(name, logits.shape, float(np.abs(logits).max()))
    np.savez_compressed(os.path.join(HERE, "oracle_logits.npz"), **out)


if __name__ == "__main__":
    main()
