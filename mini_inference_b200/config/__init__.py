from .engine_args import EngineArgs
from .model_config import ConfigError, Qwen3Config, read_config_json
from .registry import load_config, register_architecture, resolve, supported_architectures
from .spec import ExecStep, LayerSpec, ModelSpec, PartSpec

__all__ = ["EngineArgs", "ConfigError", "Qwen3Config", "read_config_json", "load_config",
           "register_architecture", "resolve", "supported_architectures",
           "ExecStep", "LayerSpec", "ModelSpec", "PartSpec"]
