from .engine_config import EngineConfig
from .model_config import (
    ConfigError,
    Footprint,
    architecture_name,
    load_stop_token_ids,
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
    "Architecture", "ConfigError", "EngineConfig", "Footprint", "LayerSpec", "ModelSpec",
    "PartSpec", "ScheduleEntry", "architecture_name", "build_model_spec", "config_from_dict",
    "get_architecture", "load_config", "load_stop_token_ids", "read_config_dict",
    "register_architecture", "supported_architectures",
]
