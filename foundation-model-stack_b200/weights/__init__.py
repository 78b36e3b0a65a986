from .adapters import extend_adapter, get_adapted, list_sources, register_adapter, register_adapter_step
from .loader import WeightError, checkpoint_dtype, kept_dtype, load_weights
from .random_init import write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, find_checkpoint_files, write_safetensors
from .sources import FileSource, RandomSource, TensorLayout

__all__ = ["extend_adapter", "checkpoint_dtype", "get_adapted", "list_sources", "register_adapter", "register_adapter_step", "WeightError",
           "kept_dtype", "load_weights", "write_random_model", "SafetensorsError", "SafetensorsFile",
           "find_checkpoint_files", "write_safetensors", "FileSource", "RandomSource", "TensorLayout"]
