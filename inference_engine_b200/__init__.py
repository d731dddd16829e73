"""A small, whole LLM inference engine for one NVIDIA B200: from a model folder to tokens.

    from inference_engine_b200 import LLMEngine, SamplingParams
    engine = LLMEngine.from_model_dir("model_dir")            # or LLMEngine.from_random(cfg)
    tokens = engine.generate({"a": [1, 2, 3]}, SamplingParams(temperature=0, max_tokens=16))
"""

from .config import EngineConfig, load_config, register_architecture
from .sampling.params import SamplingParams

__version__ = "0.1.0"


def __getattr__(name: str):
    # torch-dependent parts are imported on first use so that `engine info` needs no torch
    if name == "LLMEngine":
        from .engine.llm_engine import LLMEngine

        return LLMEngine
    if name == "generate":
        from .engine.generate import generate

        return generate
    if name in ("load_model", "random_model"):
        from .engine import loading

        return getattr(loading, name)
    raise AttributeError(name)


__all__ = ["EngineConfig", "LLMEngine", "SamplingParams", "generate",
           "load_config", "load_model", "random_model", "register_architecture"]
