"""Typed Qwen3 dense configuration, read from the architecture's config.json.

Field set follows the reference's `mynah_slm_config` (mynah-slm
src/model.h:26-50) with the keys of its vendored
reference/qwen3-0.6b/config.json:2-29. `head_dim` is its own key and is never
derived from hidden_size / heads (src/model.h:33-36). The stop set is the
union of config.json's and generation_config.json's `eos_token_id`
(docs/qwen3-arch.md:152-154: two terminators).

The reference runs full causal attention only. The window keys that
config.json carries (`use_sliding_window`, `sliding_window`,
`max_window_layers`) are honoured here: with `use_sliding_window` set, layers
with index >= `max_window_layers` see the last `sliding_window` positions
(the query's own included); the others see all of them.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Mapping, Optional

from .keys import (ConfigError, int_set, opt_bool, opt_int, req_bool, req_float,
                   req_int, req_str)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Qwen3ForCausalLM"


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    temperature: Optional[float] = None     # generation_config.json, when present
    top_k: Optional[int] = None
    top_p: Optional[float] = None

    # ------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "Qwen3Config":
        if d.get("model_type", "qwen3") != "qwen3":
            raise ConfigError(f"model_type is {d['model_type']!r}, expected 'qwen3'")
        if opt_bool(d, "attention_bias", False):
            raise ConfigError("attention_bias=true is not supported: the projections carry no bias")
        if d.get("rope_scaling") is not None:
            raise ConfigError(f"rope_scaling={d['rope_scaling']!r} is not supported (only null)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r} is not supported (only 'silu')")

        use_win = opt_bool(d, "use_sliding_window", False)
        window = opt_int(d, "sliding_window", None)
        if use_win and (window is None or window < 1):
            raise ConfigError("use_sliding_window is true but sliding_window is not a positive integer")
        gen = generation or {}
        eos = tuple(dict.fromkeys(int_set(d.get("eos_token_id"), "eos_token_id")
                                  + int_set(gen.get("eos_token_id"), "generation_config.eos_token_id")))
        cfg = cls(
            hidden_size=req_int(d, "hidden_size"),
            num_hidden_layers=req_int(d, "num_hidden_layers"),
            num_attention_heads=req_int(d, "num_attention_heads"),
            num_key_value_heads=req_int(d, "num_key_value_heads"),
            head_dim=req_int(d, "head_dim"),
            intermediate_size=req_int(d, "intermediate_size"),
            vocab_size=req_int(d, "vocab_size"),
            rms_norm_eps=req_float(d, "rms_norm_eps"),
            rope_theta=req_float(d, "rope_theta"),
            max_position_embeddings=req_int(d, "max_position_embeddings"),
            tie_word_embeddings=req_bool(d, "tie_word_embeddings"),
            hidden_act=act,
            use_sliding_window=use_win,
            sliding_window=window,
            max_window_layers=opt_int(d, "max_window_layers", 0) or 0,
            eos_token_ids=eos,
            bos_token_id=opt_int(d, "bos_token_id", None),
            torch_dtype=str(d.get("torch_dtype", "bfloat16")),
            temperature=float(gen["temperature"]) if "temperature" in gen else None,
            top_k=int(gen["top_k"]) if "top_k" in gen else None,
            top_p=float(gen["top_p"]) if "top_p" in gen else None,
        )
        cfg.check()
        return cfg

    def check(self) -> None:
        """Sanity rules of mynah-slm src/model.c:93-106, plus the sizes that the
        rotation needs (even head_dim, src/kernels.c:144)."""
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads}): GQA groups would not be whole")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for the split-half rotation")
        if not self.rms_norm_eps > 0.0:
            raise ConfigError(f"rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if not self.rope_theta > 0.0:
            raise ConfigError(f"rope_theta must be > 0, got {self.rope_theta}")
        for t in self.eos_token_ids:
            if not 0 <= t < self.vocab_size:
                raise ConfigError(f"eos_token_id {t} lies outside the vocabulary of {self.vocab_size}")

    # ------------------------------------------------------------- writing
    def to_dict(self) -> dict[str, Any]:
        """The config.json this configuration is read back from."""
        d = asdict(self)
        eos = d.pop("eos_token_ids")
        for k in ("temperature", "top_k", "top_p"):
            d.pop(k)
        d.update({
            "architectures": [ARCHITECTURE],
            "model_type": "qwen3",
            "attention_bias": False,
            "rope_scaling": None,
            "eos_token_id": (eos[0] if len(eos) == 1 else list(eos)) if eos else None,
        })
        return d

    # ---------------------------------------------------------------- spec
    def layer_window(self, i: int) -> Optional[int]:
        if self.use_sliding_window and self.sliding_window is not None and i >= self.max_window_layers:
            return self.sliding_window
        return None

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"eps": self.rms_norm_eps})
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "qk_norm": PartSpec("rmsnorm", {"eps": self.rms_norm_eps}),
                "position": PartSpec("rope_neox", {"theta": self.rope_theta, "rotary_dim": self.head_dim}),
                "window": self.layer_window(i),
                "prefix": p + "self_attn.",
            })
            ffn = PartSpec("swiglu_dense", {
                "hidden_size": self.hidden_size,
                "intermediate_size": self.intermediate_size,
                "activation": self.hidden_act,
                "prefix": p + "mlp.",
            })
            layers.append(LayerSpec(
                block=PartSpec("prenorm_residual", {}),
                mixer=mixer, ffn=ffn,
                norms={"mixer": PartSpec("rmsnorm", {"eps": self.rms_norm_eps, "dim": self.hidden_size,
                                                     "name": p + "input_layernorm.weight"}),
                       "ffn": PartSpec("rmsnorm", {"eps": self.rms_norm_eps, "dim": self.hidden_size,
                                                   "name": p + "post_attention_layernorm.weight"})},
                prefix=p))
        sampling = {k: v for k, v in (("temperature", self.temperature), ("top_k", self.top_k),
                                      ("top_p", self.top_p)) if v is not None}
        spec = ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            embedding=PartSpec("token_embedding", {"name": "model.embed_tokens.weight",
                                                   "vocab_size": self.vocab_size, "dim": self.hidden_size}),
            final_norm=PartSpec("rmsnorm", {"eps": self.rms_norm_eps, "dim": self.hidden_size,
                                            "name": "model.norm.weight"}),
            head=PartSpec("linear_head", {"tied": self.tie_word_embeddings, "name": "lm_head.weight",
                                          "vocab_size": self.vocab_size, "dim": self.hidden_size}),
            eos_token_ids=self.eos_token_ids,
            sampling_defaults=sampling,
        )
        spec.validate()
        return spec
