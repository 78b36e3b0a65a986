"""Random-weights mode: write a model folder (``config.json`` + ``model.safetensors``) from a
configuration and a seed.  The folder is then a model like any other."""
from __future__ import annotations

import json
import os

import torch

from .safetensors_io import write_safetensors
from .sources import RandomSource


def write_random_model(folder: str, config_json: dict, layout, seed: int, dtype: torch.dtype = torch.bfloat16,
                       gain_dtype: torch.dtype = None, std: float = 0.02) -> str:
    """``config_json``: the architecture's own config.json keys; ``layout``: its checkpoint tensors
    (``TensorLayout``).  Returns the folder."""
    os.makedirs(folder, exist_ok=True)
    src = RandomSource(layout, seed, dtype=dtype, device="cpu", std=std, gain_dtype=gain_dtype)
    tensors = {name: src.get(name) for name in src.keys()}
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_json, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, {"format": "pt", "seed": str(seed)})
    return folder
