"""A small, whole LLM inference engine for one NVIDIA B200 (sm_100a): Qwen3 dense.

    from mini_inference_b200 import LLM, SamplingParams
    llm = LLM("model_dir", dtype="bfloat16")
    out = llm.generate([[1, 2, 3]], SamplingParams(max_new_tokens=16))
"""
__version__ = "0.1.0"

from .config.engine_args import EngineArgs  # noqa: E402
from .engine.llm import LLM, create_engine  # noqa: E402
from .engine.request import SamplingParams  # noqa: E402

__all__ = ["LLM", "SamplingParams", "EngineArgs", "create_engine"]
