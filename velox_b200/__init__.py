"""velox_b200: a small, whole LLM inference engine for one NVIDIA B200."""
__version__ = "0.1.0"
