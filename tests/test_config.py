"""Typed configuration, registry and memory estimates."""

from __future__ import annotations

import json

import pytest

from inference_engine_b200.architectures.llama import LlamaConfig
from inference_engine_b200.config import (
    ConfigError, build_model_spec, config_from_dict, get_architecture, load_config,
    load_stop_token_ids, register_architecture, supported_architectures,
)
from inference_engine_b200.config.spec import ModelSpec, PartSpec, ScheduleEntry
from tests.tiny_configs import TINY_A, TINY_B, TINY_C

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "bos_token_id": 128000, "eos_token_id": [128001, 128008, 128009],
    "head_dim": 64, "hidden_size": 2048, "intermediate_size": 8192, "max_position_embeddings": 131072,
    "model_type": "llama", "num_attention_heads": 32, "num_hidden_layers": 16, "num_key_value_heads": 8,
    "rms_norm_eps": 1e-05,
    "rope_scaling": {"factor": 32.0, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192, "rope_type": "llama3"},
    "rope_theta": 500000.0, "tie_word_embeddings": True, "torch_dtype": "bfloat16", "vocab_size": 128256,
}
LLAMA_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "intermediate_size": 14336,
    "max_position_embeddings": 131072, "num_attention_heads": 32, "num_hidden_layers": 32,
    "num_key_value_heads": 8, "rms_norm_eps": 1e-05,
    "rope_scaling": {"factor": 8.0, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192, "rope_type": "llama3"},
    "rope_theta": 500000.0, "tie_word_embeddings": False, "vocab_size": 128256,
}


def test_parses_the_1b_shape():
    cfg = config_from_dict(LLAMA_1B)
    assert isinstance(cfg, LlamaConfig)
    assert (cfg.head_dim, cfg.num_kv_groups, cfg.q_size, cfg.kv_size) == (64, 4, 2048, 512)
    assert cfg.tie_word_embeddings and cfg.rope_scaling.factor == 32.0
    assert cfg.eos_token_ids == (128001, 128008, 128009)


def test_defaults_as_the_reference():
    cfg = config_from_dict(LLAMA_8B)  # no head_dim, no eos, no dtype
    assert cfg.head_dim == 128 and cfg.eos_token_ids == () and cfg.torch_dtype == "bfloat16"
    minimal = {"architectures": ["LlamaForCausalLM"], "hidden_size": 32, "num_attention_heads": 2,
               "vocab_size": 10, "intermediate_size": 8, "num_hidden_layers": 1}
    cfg = config_from_dict(minimal)
    assert (cfg.num_key_value_heads, cfg.max_position_embeddings, cfg.rms_norm_eps, cfg.rope_theta) == (2, 2048, 1e-5, 10000.0)
    assert cfg.rope_scaling is None and not cfg.tie_word_embeddings
    assert config_from_dict({**minimal, "architectures": [], "model_type": "LlamaForCausalLM"}).hidden_size == 32


@pytest.mark.parametrize("raw,expected", [(LLAMA_1B, 1_235_814_400), (LLAMA_8B, 8_030_261_248)])
def test_param_count_matches_published_models(raw, expected):
    assert _footprint(raw).parameters == expected


def _footprint(raw):
    cfg = config_from_dict(raw)
    return get_architecture(cfg.architecture).footprint(cfg)


def test_memory_estimates():
    assert _footprint(LLAMA_1B).cache_bytes_per_token(2) == 32 * 1024
    assert _footprint(LLAMA_8B).cache_bytes_per_token(2) == 128 * 1024
    assert _footprint(LLAMA_8B).cache_tokens_that_fit(gpu_mem_gib=8) == 0
    assert _footprint(LLAMA_8B).cache_tokens_that_fit(gpu_mem_gib=180) > 1_000_000


def test_the_footprint_an_architecture_reports_is_that_of_the_built_model():
    """Counted from the parts' declared tensors and the cache groups (what `engine info` falls
    back to for an architecture that reports none)."""
    from inference_engine_b200.engine.model import Model

    for raw in (TINY_A, TINY_B, TINY_C):
        cfg = config_from_dict(raw)
        built = Model(build_model_spec(cfg), "bfloat16", max_positions=8).footprint()
        assert built == _footprint(raw)


def test_errors_name_what_is_wrong():
    with pytest.raises(ConfigError, match="unsupported architecture 'MixtralForCausalLM'.*LlamaForCausalLM"):
        config_from_dict({**TINY_A, "architectures": ["MixtralForCausalLM"]})
    with pytest.raises(ConfigError, match="rope_scaling type 'yarn'"):
        config_from_dict({**TINY_A, "rope_scaling": {"rope_type": "yarn", "factor": 4.0}})
    with pytest.raises(ConfigError, match="'hidden_size'"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "hidden_size"})
    with pytest.raises(ConfigError, match="not divisible"):
        config_from_dict({**TINY_A, "num_key_value_heads": 3})
    with pytest.raises(ConfigError, match="factor"):
        config_from_dict({**TINY_A, "rope_scaling": {"rope_type": "llama3"}})
    with pytest.raises(ConfigError, match="head_dim"):
        config_from_dict({**TINY_A, "head_dim": 15})
    assert issubclass(ConfigError, ValueError)


def test_legacy_rope_type_key_and_round_trip(tmp_path):
    cfg = config_from_dict(TINY_C)  # uses the legacy "type" key
    assert cfg.rope_scaling.rope_type == "llama3" and cfg.rope_scaling.low_freq_factor == 2.0
    for raw in (TINY_A, TINY_B, TINY_C, LLAMA_1B):
        cfg = config_from_dict(raw)
        assert config_from_dict(cfg.to_dict()) == cfg
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(tmp_path) == config_from_dict(TINY_B)
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path / "nowhere")


def test_stop_ids_merge_generation_config(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({**TINY_A, "eos_token_id": 128001}))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [128001, 128009]}))
    assert load_stop_token_ids(tmp_path) == (128001, 128009)


def test_the_description_is_data():
    spec = build_model_spec(config_from_dict(TINY_B))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    layer = spec.layers[1]
    assert layer.mixer.kind == "paged_attention" and layer.mixer.params["num_kv_heads"] == 1
    assert layer.feed_forward.params["intermediate_size"] == 320
    assert layer.norms["pre_mixer"].params["eps"] == 1e-6
    assert spec.head.params["weight"] == "lm_head.weight"
    assert build_model_spec(config_from_dict(TINY_A)).head.params["weight"] is None  # tied


def test_run_order_is_checked():
    spec = build_model_spec(config_from_dict(TINY_A))
    import dataclasses

    bad = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(5)))
    with pytest.raises(ValueError, match="layer 5"):
        bad.validate()
    bad = dataclasses.replace(spec, schedule=(ScheduleEntry(0, cache_from=0),))
    with pytest.raises(ValueError, match="earlier"):
        bad.validate()
    dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                                        ScheduleEntry(1, cache_from=1))).validate()


def test_registering_another_architecture():
    from dataclasses import dataclass

    @dataclass(frozen=True)
    class ToyConfig:
        architecture: str
        width: int

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["architectures"][0], raw["width"])

    def toy_spec(cfg):
        base = build_model_spec(config_from_dict({**TINY_A, "hidden_size": cfg.width}))
        import dataclasses

        return dataclasses.replace(base, architecture=cfg.architecture)

    register_architecture("ToyForTests", ToyConfig, toy_spec, replace=True)
    assert "ToyForTests" in supported_architectures()
    cfg = config_from_dict({"architectures": ["ToyForTests"], "width": 128})
    assert build_model_spec(cfg).hidden_size == 128
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("ToyForTests", ToyConfig, toy_spec)
