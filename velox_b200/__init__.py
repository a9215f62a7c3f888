"""velox_b200: a small, whole LLM inference engine for one NVIDIA B200.

    from velox_b200 import LLM, SamplingParams
    llm = LLM("<model folder>", dtype="bfloat16")
    ids = llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=16))
"""
__version__ = "0.1.0"

_EXPORTS = {
    "LLM": ("velox_b200.engine.engine", "LLM"),
    "Engine": ("velox_b200.engine.engine", "Engine"),
    "EngineConfig": ("velox_b200.config", "EngineConfig"),
    "Request": ("velox_b200.engine.request", "Request"),
    "SamplingParams": ("velox_b200.sampling.params", "SamplingParams"),
}

__all__ = sorted(_EXPORTS)


def __getattr__(name):
    # Resolved on first use, so that importing the package stays cheap (no torch yet).
    try:
        module, attribute = _EXPORTS[name]
    except KeyError:
        raise AttributeError(f"module 'velox_b200' has no attribute {name!r}") from None
    import importlib

    value = getattr(importlib.import_module(module), attribute)
    globals()[name] = value
    return value
