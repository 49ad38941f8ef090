from .generate import GenerationError, GenerationStats, generate_ids

__all__ = ["GenerationError", "GenerationStats", "generate_ids", "Engine", "Entry", "StepError", "EngineBackend"]


def __getattr__(name):
    if name in ("Engine", "Entry", "StepError"):
        from . import step
        return getattr(step, name)
    if name == "EngineBackend":
        from .backend import EngineBackend
        return EngineBackend
    raise AttributeError(name)
