"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

from helpers import TINY_A, TINY_B, TINY_C
from mynah_slm_b200 import ConfigError, known_architectures, parse_config, register_architecture
from mynah_slm_b200.config.qwen3 import Qwen3Config


def test_official_config_reads():
    """The official Qwen3-0.6B config.json that the reference's checkout carries (reference/qwen3-0.6b/), when a
    checkout is at hand: $MYNAH_REFERENCE, or a folder `reference` beside this repository."""
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    root = os.environ.get("MYNAH_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(here)), "reference")
    path = os.path.join(root, "reference", "qwen3-0.6b", "config.json")
    try:
        cfg = json.load(open(path))
        gen = json.load(open(path.replace("config.json", "generation_config.json")))
    except OSError:
        pytest.skip("the reference checkout is not here")
    c = parse_config(cfg, gen)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (28, 1024, 16, 8)
    assert c.head_dim == 128 and c.head_dim != c.hidden_size // c.num_attention_heads   # never derived
    assert c.rope_theta == 1e6 and isinstance(c.rope_theta, float)                     # written as an int in the file
    assert c.rms_norm_eps == 1e-6
    assert c.eos_token_ids == (151645, 151643)                                          # both terminators
    assert c.tie_word_embeddings is True
    assert (c.temperature, c.top_k, c.top_p) == (0.6, 20, 0.95)


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                                 "head_dim", "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta",
                                 "max_position_embeddings", "tie_word_embeddings"])
def test_missing_key_is_named(key):
    cfg = copy.deepcopy(TINY_A)
    del cfg[key]
    with pytest.raises(ConfigError, match=f"missing config key: {key}"):
        parse_config(cfg)


def test_no_guessing_and_types():
    cfg = dict(TINY_A, head_dim=16.0)
    with pytest.raises(ConfigError, match="head_dim is not an integer"):
        parse_config(cfg)
    cfg = dict(TINY_A, rms_norm_eps="1e-6")
    with pytest.raises(ConfigError, match="rms_norm_eps is not a float"):
        parse_config(cfg)
    cfg = dict(TINY_A, tie_word_embeddings=1)
    with pytest.raises(ConfigError, match="tie_word_embeddings is not a boolean"):
        parse_config(cfg)


def test_sanity_rules():
    with pytest.raises(ConfigError, match="not a multiple"):
        parse_config(dict(TINY_A, num_attention_heads=5))
    with pytest.raises(ConfigError, match="must be even"):
        parse_config(dict(TINY_A, head_dim=15))
    with pytest.raises(ConfigError, match="attention_bias"):
        parse_config(dict(TINY_A, attention_bias=True))
    with pytest.raises(ConfigError, match="rope_scaling"):
        parse_config(dict(TINY_A, rope_scaling={"type": "yarn"}))
    with pytest.raises(ConfigError, match="hidden_act"):
        parse_config(dict(TINY_A, hidden_act="gelu"))
    with pytest.raises(ConfigError, match="sliding_window"):
        parse_config(dict(TINY_A, use_sliding_window=True, sliding_window=None))
    with pytest.raises(ConfigError, match="outside the vocabulary"):
        parse_config(dict(TINY_A, eos_token_id=99999))


def test_registry():
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="unknown architecture 'NopeForCausalLM'; known: .*Qwen3ForCausalLM"):
        parse_config(dict(TINY_A, architectures=["NopeForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        parse_config({k: v for k, v in TINY_A.items() if k != "architectures"})
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict)


def test_round_trip_and_spec():
    for cfg in (TINY_A, TINY_B, TINY_C):
        c = parse_config(cfg)
        c2 = parse_config(c.to_dict())
        assert c == c2
        spec = c.model_spec()
        assert len(spec.layers) == cfg["num_hidden_layers"] == len(spec.schedule)
        for i, ls in enumerate(spec.layers):
            assert ls.mixer["head_dim"] == cfg["head_dim"]
            assert ls.mixer["position"]["theta"] == float(cfg["rope_theta"])
            assert ls.norms["mixer"]["eps"] == cfg["rms_norm_eps"]
            want = cfg["sliding_window"] if cfg["use_sliding_window"] and i >= cfg.get("max_window_layers", 0) else None
            assert ls.mixer["window"] == want
        assert spec.head["tied"] == cfg["tie_word_embeddings"]


def test_window_layers_form_a_second_cache_group():
    from mynah_slm_b200.engine.model import Model
    plan = Model(parse_config(TINY_C).model_spec()).cache_plan()
    assert [(g.window, g.entries) for g in plan.groups] == [(None, [0, 1]), (40, [2, 3])]
    plan = Model(parse_config(TINY_A).model_spec()).cache_plan()
    assert [(g.window, g.entries) for g in plan.groups] == [(None, [0, 1])]


def test_schedule_validation():
    from dataclasses import replace
    from mynah_slm_b200.config.spec import ScheduleEntry
    spec = parse_config(TINY_A).model_spec()
    replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_from=1))).validate()
    with pytest.raises(ConfigError, match="names layer 5"):
        replace(spec, schedule=(ScheduleEntry(5),)).validate()
    with pytest.raises(ConfigError, match="does not run before"):
        replace(spec, schedule=(ScheduleEntry(0, cache_from=1), ScheduleEntry(1))).validate()
    with pytest.raises(ConfigError, match="keeps none of its own"):
        replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1, cache_from=0), ScheduleEntry(1, cache_from=1))).validate()
