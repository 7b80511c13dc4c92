"""mini_engine_b200: a small, whole LLM inference engine for one B200 (sm_100a)."""
from .config import EngineConfig, load_model_config, register_architecture
from .sampling import SamplingParams

__all__ = ["LLM", "SamplingParams", "EngineConfig", "load_model_config", "register_architecture"]


def __getattr__(name):
    if name == "LLM":                     # imported lazily: the engine pulls in the kernels' loader
        from .llm import LLM
        return LLM
    raise AttributeError(name)
