from .engine_config import EngineConfig
from .model_config import (
    ConfigError,
    LlamaConfig,
    RopeScaling,
    architecture_name,
    estimate_param_count,
    kv_bytes_per_token,
    load_stop_token_ids,
    max_kv_tokens,
    read_config_dict,
)
from .registry import (
    Architecture,
    build_model_spec,
    config_from_dict,
    get_architecture,
    load_config,
    register_architecture,
    supported_architectures,
)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = [
    "Architecture", "ConfigError", "EngineConfig", "LayerSpec", "LlamaConfig", "ModelSpec",
    "PartSpec", "RopeScaling", "ScheduleEntry", "architecture_name", "build_model_spec",
    "config_from_dict", "estimate_param_count", "get_architecture", "kv_bytes_per_token",
    "load_config", "load_stop_token_ids", "max_kv_tokens", "read_config_dict",
    "register_architecture", "supported_architectures",
]
