"""Registry from an architecture's name and variant to its model, and ``get_model``
(fms/models/__init__.py:28-69 for the registry, :298-503 for get_model).

    model = get_model("llama", "3-8b", device_type="cuda", data_type="bf16")           # random weights
    model = get_model("llama", model_path="/folder", source="hf")                       # config.json + safetensors
    model = get_model("hf_pretrained", model_path="/folder")                            # architecture from config.json
"""
from __future__ import annotations

import json
import logging
import os
from typing import Callable, Dict, List, Optional, Union

import torch

from .base import Model

logger = logging.getLogger(__name__)

_models: Dict[str, Dict[str, Callable[..., Model]]] = {}
_architectures: Dict[str, type] = {}
_hf_architectures: Dict[str, str] = {}


def register_architecture(architecture: str, model_class: type, config_json_names=()) -> None:
    """``config_json_names``: values of config.json's ``architectures[0]`` that mean this architecture."""
    if architecture in _architectures:
        raise KeyError(f"architecture {architecture} is already registered")
    _architectures[architecture] = model_class
    for n in config_json_names:
        _hf_architectures[n] = architecture


def register_model(architecture: str, variant: str, factory: Callable[..., Model]) -> None:
    variants = _models.setdefault(architecture, {})
    if variant in variants:
        raise KeyError(f"Variant {variant} already registered for architecture {architecture}")
    variants[variant] = factory


def list_models() -> List[str]:
    return list(_models.keys())


def list_variants(architecture: str) -> List[str]:
    if architecture not in _models:
        raise KeyError(f"{architecture} is not registered. See `models.list_models()` for available architectures")
    return list(_models[architecture].keys())


_DTYPES = {
    "bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32,
    torch.bfloat16: torch.bfloat16, torch.float32: torch.float32,
}


def _dtype(data_type) -> torch.dtype:
    if data_type not in _DTYPES:
        raise ValueError(f"data_type {data_type!r} is not supported: bf16 and fp32 are")
    return _DTYPES[data_type]


def read_config_json(model_path: str) -> dict:
    path = os.path.join(model_path, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {model_path}")
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


def get_model(architecture: str, variant: Optional[str] = None, model_path: Optional[str] = None,
              source: Optional[str] = None, device_type: str = "cuda", data_type: Union[str, torch.dtype, None] = None,
              distributed_strategy: Optional[str] = None, checkpoint_sharding: Optional[str] = None, group=None,
              seed: int = 0, init: str = "baseline", **kwargs) -> Model:
    """Builds a model and fills its weights.

    architecture: a registered name, or "hf_pretrained" to take it from ``model_path``'s config.json.
    variant: a registered configuration; None with a ``model_path`` folder means its config.json.
    model_path: folder (or file, or glob) of safetensors; None means random weights from ``seed``.
    source: the checkpoint's naming ("hf" by default; "fms" for the engine's own names).
    data_type: "bf16" or "fp32": the compute dtype; float32 uses no reduced-precision product.  None: the dtype
        in which the checkpoint stores its matrices (fms/utils/serialization.py:679-687), which must be one of
        the two, else an error asks for ``data_type``; bfloat16 for random weights.
    init: how random weights are drawn: "baseline" (matrices and embedding ~ N(0, 0.02), gains 1 + U(-0.1, 0.1)) or
        "fms" (the reference's ``reset_parameters``: fms/models/llama.py:231-235, :387-393;
        fms/modules/attention.py:689-692; fms/modules/feedforward.py:269-283; gains 1).
    distributed_strategy, checkpoint_sharding, group: the reference's parameters for several devices
        (fms/models/__init__.py:298-308); this library runs on one GPU and refuses anything but None.
    kwargs: overrides of configuration fields, as in the reference.
    """
    if distributed_strategy is not None or checkpoint_sharding is not None or group is not None:
        raise NotImplementedError("this library runs a model on one GPU: distributed_strategy, checkpoint_sharding "
                                  "and group must be None")
    from ..weights.sources import FileSource, RandomSource

    config = None
    if architecture == "hf_pretrained" or (variant is None and model_path is not None and os.path.isdir(model_path)
                                            and os.path.isfile(os.path.join(model_path, "config.json"))):
        if model_path is None:
            raise ValueError("hf_pretrained needs a model_path with a config.json")
        values = read_config_json(model_path)
        if architecture == "hf_pretrained":
            names = values.get("architectures") or [None]
            if names[0] not in _hf_architectures:
                raise KeyError(f"config.json names architecture {names[0]!r}; known: {sorted(_hf_architectures)}")
            architecture = _hf_architectures[names[0]]
            source = source or _architectures[architecture].default_source
        if architecture not in _architectures:
            raise KeyError(f"{architecture} is not registered. See `models.list_models()` for available architectures")
        config = _architectures[architecture].config_from_json(values)
        model = _architectures[architecture](config, **kwargs)
    else:
        if architecture not in _models:
            raise KeyError(f"{architecture} is not registered. See `models.list_models()` for available architectures")
        if variant not in _models[architecture]:
            raise KeyError(f'{variant} is not a registered variant of {architecture}. See '
                           f'`models.list_variants("{architecture}")` for available variants.')
        model = _models[architecture][variant](**kwargs)

    from ..weights.loader import checkpoint_dtype

    device = torch.device(device_type)
    if model_path is not None:
        src = FileSource(model_path)
        dtype = checkpoint_dtype(src) if data_type is None else _dtype(data_type)
    else:
        # random weights straight on the device, through the same adapter and checks as a file
        src = RandomSource(model.checkpoint_layout(), seed, dtype=torch.bfloat16, device=device, init=init)
        source = model.default_source
        dtype = torch.bfloat16 if data_type is None else _dtype(data_type)
    return model.load(src, source, device, dtype)


from . import llama  # noqa: E402,F401  (registers the architecture and its variants)


def _import_plugins() -> None:
    """Modules named in FMS_B200_PLUGINS (comma-separated, importable names) are imported once the built-in
    architectures are registered: an architecture, part or adapter that lives outside this library registers itself
    there, and the command-line programs (which find the model class through config.json) then know it."""
    import importlib

    for name in filter(None, (n.strip() for n in os.environ.get("FMS_B200_PLUGINS", "").split(","))):
        try:
            importlib.import_module(name)
        except Exception as e:
            raise ImportError(f"FMS_B200_PLUGINS names {name!r}, which cannot be imported: {e}") from e


_import_plugins()

__all__ = ["Model", "get_model", "list_models", "list_variants", "register_architecture", "register_model",
           "read_config_json"]
