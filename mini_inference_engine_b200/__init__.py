"""A small, whole, single-GPU inference engine for the Llama dense decoder on B200 (sm_100a).

Exports are lazy, as in inference_engine/__init__.py:1-9, so that importing a subpackage (the
kernels, the cache manager) does not pull in the engine."""

__all__ = ["LLMEngine", "SamplingParams", "EngineConfig", "RequestOutput"]


def __getattr__(name):
    if name in ("LLMEngine", "RequestOutput"):
        from .engine import engine
        return getattr(engine, name)
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    if name == "EngineConfig":
        from .config.engine_config import EngineConfig
        return EngineConfig
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
