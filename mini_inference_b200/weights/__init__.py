from .random_init import init_random_on_device, write_random_model
from .safetensors_io import SafetensorsFile, open_model_tensors, write_safetensors
from .store import WeightError, load_into, runtime_dtype

__all__ = ["write_random_model", "init_random_on_device", "SafetensorsFile", "open_model_tensors", "write_safetensors",
           "WeightError", "load_into", "runtime_dtype"]
