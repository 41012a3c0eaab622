"""A small, whole LLM inference engine for one NVIDIA B200 (sm_100a): Qwen3 dense."""
__version__ = "0.1.0"
