"""Plain Qwen3-dense forward pass: whole sequences, no cache, numpy only.

One function per part. float32 values with float64 accumulators in the norms,
the dot products and the softmax sum, as the reference's scalar C code keeps
them. No code is shared with the product package.

Citations are paths inside mynah-org/mynah-slm.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

PAGE = 64  # only used to describe traces; the plain model has no cache


# ---------------------------------------------------------------- containers

def read_safetensors(path: str) -> dict[str, np.ndarray]:
    """Minimal reader: 8-byte little-endian header length, JSON table, payload.

    Layout per third_party/ingot/src/safetensors.c:357-403 (header) and
    :224-322 (one tensor object: dtype, shape, data_offsets). bf16 is widened
    exactly by a 16-bit shift (third_party/ingot/src/dtype.c:270-275).
    """
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    table = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, t in table.items():
        if name == "__metadata__":
            continue
        lo, hi = t["data_offsets"]
        buf = raw[base + lo:base + hi]
        dt = t["dtype"]
        if dt == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float32)
        elif dt == "BF16":
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            a = u.view(np.float32)
        elif dt == "F16":
            a = np.frombuffer(buf, dtype="<f2").astype(np.float32)
        elif dt == "I32":
            a = np.frombuffer(buf, dtype="<i4").copy()
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = a.reshape(t["shape"])
    return out


def read_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------- parts

def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> the nearest bfloat16 (ties to even) -> float32: what a value is after the bfloat16 engine has
    stored it (third_party/ingot/src/dtype.c:276-284 rounds the same way)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """out = x * (1/sqrt(mean(x^2)+eps)) * w over the last axis; the sum of
    squares is kept in double and the scale cast to float before use.
    src/kernels.c:118-128 (rms_scale, mynah_slm_rms_norm); plain gain, not 1+w
    (src/kernels.h:29-33)."""
    x = x.astype(np.float32)
    ss = np.sum(x.astype(np.float64) ** 2, axis=-1, keepdims=True)
    s = (1.0 / np.sqrt(ss / x.shape[-1] + np.float64(np.float32(eps)))).astype(np.float32)
    return (x * s * weight.astype(np.float32)).astype(np.float32)


def rope_table(head_dim: int, positions: np.ndarray, theta: float):
    """cos/sin[pos][i] = (float) cos/sin(pos * theta^(-2i/head_dim)), built in
    double. src/kernels.c:141-164 (mynah_slm_rope_init); theta is a float
    there (the function's parameter type), so it is rounded to float first."""
    half = head_dim // 2
    th = np.float64(np.float32(theta))
    inv = 1.0 / th ** (2.0 * np.arange(half, dtype=np.float64) / head_dim)
    ang = positions.astype(np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def rope_apply(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """NeoX split-half rotation: element i pairs with i + head_dim/2.
    x is [seq, heads, head_dim]; cos/sin are [seq, head_dim/2].
    src/kernels.c:173-189 (mynah_slm_rope_apply)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1).astype(np.float32)


def linear(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """y = W.x with W [out, in] row-major, no bias (src/arch_qwen3.c:52-83,
    project); products accumulated in double as the scalar dot does
    (src/kernels.c:72-74)."""
    return (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)


def stable_sigmoid(x: np.ndarray) -> np.ndarray:
    """x>=0: 1/(1+e^-x); else e^x/(1+e^x). src/kernels.c:193-197."""
    x = x.astype(np.float32)
    out = np.empty_like(x)
    pos = x >= 0
    out[pos] = 1.0 / (1.0 + np.exp(-x[pos]))
    e = np.exp(x[~pos])
    out[~pos] = e / (1.0 + e)
    return out


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """a_i = g_i * sigmoid(g_i) * u_i. src/kernels.c:203-205."""
    return (gate * stable_sigmoid(gate) * up).astype(np.float32)


def softmax_rows(s: np.ndarray) -> np.ndarray:
    """Max-subtracted, expf in float, sum in double, multiplied by
    (float)(1/sum). src/kernels.c:207-220. -inf entries give exactly 0."""
    m = np.max(s, axis=-1, keepdims=True)
    e = np.exp((s - m).astype(np.float32)).astype(np.float32)
    inv = (1.0 / np.sum(e.astype(np.float64), axis=-1, keepdims=True)).astype(np.float32)
    return (e * inv).astype(np.float32)


def gqa_attention(q, k, v, window: int | None = None, q_pos=None, k_pos=None, round_p=None):
    """Causal grouped-query attention over whole sequences.

    q [Tq, H, HD]; k, v [Tk, KV, HD]. Query head h reads kv head h // (H/KV);
    score = dot(q, k) * (1/sqrtf(HD)) with the scale applied after the dot;
    key t is visible to the query at position p when t <= p
    (src/kernels.c:228-250, n_kv = pos+1 at src/arch_qwen3.c:184; the mask form
    is tools/oracle/model.py:75-91).

    `window` (not in the reference, which has full attention only) restricts
    the visible keys further to p - window < t <= p.

    `round_p` (the bfloat16 mode): the function that rounds the unnormalised
    probabilities e^(s-max) for the second product, as a tensor-core kernel
    does; the sum that normalises stays the sum of the unrounded ones.
    """
    tq, n_heads, hd = q.shape
    tk, n_kv, _ = k.shape
    group = n_heads // n_kv
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    q_pos = np.arange(tq) if q_pos is None else np.asarray(q_pos)
    k_pos = np.arange(tk) if k_pos is None else np.asarray(k_pos)
    vis = k_pos[None, :] <= q_pos[:, None]
    if window is not None:
        vis &= k_pos[None, :] > q_pos[:, None] - window
    out = np.empty((tq, n_heads, hd), dtype=np.float32)
    for h in range(n_heads):
        g = h // group
        s = (q[:, h, :].astype(np.float64) @ k[:, g, :].astype(np.float64).T).astype(np.float32) * scale
        s = np.where(vis, s, -np.inf).astype(np.float32)
        if round_p is None:
            p = softmax_rows(s)
            out[:, h, :] = (p.astype(np.float64) @ v[:, g, :].astype(np.float64)).astype(np.float32)
        else:
            e = np.exp((s - np.max(s, axis=-1, keepdims=True)).astype(np.float32)).astype(np.float32)
            inv = (1.0 / np.sum(e.astype(np.float64), axis=-1, keepdims=True)).astype(np.float32)
            out[:, h, :] = (round_p(e).astype(np.float64) @ v[:, g, :].astype(np.float64)).astype(np.float32) * inv
    return out


# --------------------------------------------------------------------- model

class PlainQwen3:
    """Qwen3 dense decoder from a config.json dict and a name->array dict.

    Order of operations per docs/qwen3-arch.md:33-47 and src/arch_qwen3.c:178-252.

    With `bf16` the model rounds to bfloat16 wherever a bfloat16 engine stores a
    value: every norm's output, every product's output (the gate and up products
    are activated from their unrounded sums, then rounded once), queries, keys and
    values after the per-head norm and the rotation (the cache), the attention's
    output, and the probabilities for the second product when the head size is one
    a tensor-core kernel takes (64 or 128). Sums, softmax, norms, rotation and the
    residual stream stay as they are. The reference has no such mode; a test may
    hold a bfloat16 engine to it far more tightly than to the unrounded model.
    """

    def __init__(self, cfg: dict, tensors: dict[str, np.ndarray], bf16: bool = False):
        self.cfg = cfg
        self.bf16 = bool(bf16)
        self.r = bf16_round if bf16 else (lambda a: a)
        self.t = {k: np.asarray(v, dtype=np.float32) for k, v in tensors.items()}
        self.L = int(cfg["num_hidden_layers"])
        self.D = int(cfg["hidden_size"])
        self.H = int(cfg["num_attention_heads"])
        self.KV = int(cfg["num_key_value_heads"])
        self.HD = int(cfg["head_dim"])          # its own key, never D/H (src/model.h:33-36)
        self.eps = float(cfg["rms_norm_eps"])
        self.theta = float(cfg["rope_theta"])
        self.tied = bool(cfg["tie_word_embeddings"])
        self.V = int(cfg["vocab_size"])

    @classmethod
    def from_folder(cls, folder: str, bf16: bool = False) -> "PlainQwen3":
        cfg, tensors = read_folder(folder)
        return cls(cfg, tensors, bf16=bf16)

    def layer_window(self, i: int) -> int | None:
        """Window of layer i, from the config keys use_sliding_window,
        sliding_window and max_window_layers: layers with index >=
        max_window_layers are windowed when use_sliding_window is set. The
        reference reads none of these (its only checkpoint has
        use_sliding_window false, reference/qwen3-0.6b/config.json:21-28)."""
        c = self.cfg
        if c.get("use_sliding_window") and c.get("sliding_window") is not None:
            if i >= int(c.get("max_window_layers", 0)):
                return int(c["sliding_window"])
        return None

    def block(self, i: int, x: np.ndarray, cos, sin, taps=None) -> np.ndarray:
        t, p, r = self.t, f"model.layers.{i}.", self.r
        h = r(rms_norm(x, t[p + "input_layernorm.weight"], self.eps))         # arch_qwen3.c:201
        q = r(linear(h, t[p + "self_attn.q_proj.weight"])).reshape(-1, self.H, self.HD)   # :204
        k = r(linear(h, t[p + "self_attn.k_proj.weight"])).reshape(-1, self.KV, self.HD)  # :205
        v = r(linear(h, t[p + "self_attn.v_proj.weight"])).reshape(-1, self.KV, self.HD)  # :206
        q = rms_norm(q, t[p + "self_attn.q_norm.weight"], self.eps)           # :209-214, per head
        k = rms_norm(k, t[p + "self_attn.k_norm.weight"], self.eps)
        q = r(rope_apply(q, cos, sin))                                        # :217-218
        k = r(rope_apply(k, cos, sin))
        round_p = bf16_round if self.bf16 and self.HD in (64, 128) else None
        a = r(gqa_attention(q, k, v, window=self.layer_window(i), round_p=round_p))      # :220-221
        x = x + r(linear(a.reshape(-1, self.H * self.HD), t[p + "self_attn.o_proj.weight"]))  # :223-224
        h = r(rms_norm(x, t[p + "post_attention_layernorm.weight"], self.eps))  # :226
        g = linear(h, t[p + "mlp.gate_proj.weight"])                          # :229
        u = linear(h, t[p + "mlp.up_proj.weight"])                            # :230
        x = x + r(linear(r(swiglu(g, u)), t[p + "mlp.down_proj.weight"]))     # :231-234
        return x.astype(np.float32)

    def forward(self, tokens, taps: dict | None = None) -> np.ndarray:
        """Logits [seq, vocab] for one whole sequence starting at position 0."""
        tokens = np.asarray(tokens, dtype=np.int64)
        pos = np.arange(len(tokens))
        x = self.t["model.embed_tokens.weight"][tokens].astype(np.float32)    # no sqrt(D): :186
        if taps is not None:
            taps["embed"] = x.copy()
        cos, sin = rope_table(self.HD, pos, self.theta)
        for i in range(self.L):
            x = self.block(i, x, cos, sin)
            if taps is not None:
                taps[f"layer{i}"] = x.copy()
        h = self.r(rms_norm(x, self.t["model.norm.weight"], self.eps))        # :239
        if taps is not None:
            taps["final_norm"] = h.copy()
        head = self.t["model.embed_tokens.weight"] if self.tied else self.t["lm_head.weight"]  # :243-247
        return linear(h, head)
