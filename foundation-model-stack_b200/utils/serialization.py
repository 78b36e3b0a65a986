"""``from fms_b200.utils.serialization import get_adapted, register_adapter, ...`` — the reference's import path
for its adapter registry and checkpoint reading (fms/utils/serialization.py:27-160 register_adapter_step,
register_adapter, extend_adapter, list_sources; :292-316 get_adapted; :339-450 load_state_dict).  The functions live in
``fms_b200.weights``; ``load_state_dict`` here opens a folder, file or glob of safetensors lazily, by tensor name."""
from .. import models as _models  # noqa: F401  (importing the architectures registers their adapters)
from ..weights import (FileSource, WeightError, extend_adapter, find_checkpoint_files, get_adapted, list_sources,
                       register_adapter, register_adapter_step)

__all__ = ["extend_adapter", "get_adapted", "list_sources", "load_state_dict", "register_adapter", "register_adapter_step",
           "WeightError"]


def load_state_dict(model_path: str) -> FileSource:
    """The tensors of a checkpoint (safetensors; a folder, one file or a glob, shards included) as a lazy mapping:
    ``keys()``, ``spec(name)`` (dtype, shape) and ``get(name)``; nothing is read before it is asked for."""
    if not find_checkpoint_files(model_path):
        raise FileNotFoundError(f"no safetensors at {model_path!r}")
    return FileSource(model_path)
