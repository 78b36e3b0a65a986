"""Adapters from a checkpoint's tensor names and layouts to the engine's, in the manner of
fms/utils/serialization.py:27-161.

An adapter is a list of named steps; a step maps a dict {name: tensor} to a new dict and may look at
keyword arguments that the loader passes on (``config``: the architecture's configuration).  Steps are
registered per architecture, adapters per (architecture, source).  A step must work on tensors of the
``meta`` device too (shapes only): the loader first runs the adapter on shapes to check the whole
checkpoint before it reads any data.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Mapping

import torch

AdapterStep = Callable[..., Dict[str, torch.Tensor]]

_steps: Dict[str, Dict[str, AdapterStep]] = {}
_adapters: Dict[str, Dict[str, List[str]]] = {}


def register_adapter_step(architecture: str, name: str, step: AdapterStep) -> None:
    steps = _steps.setdefault(architecture, {})
    if name in steps:
        raise KeyError(f"adapter step {name} is already registered for architecture {architecture}")
    steps[name] = step


def register_adapter(architecture: str, source: str, step_names: List[str]) -> None:
    sources = _adapters.setdefault(architecture, {})
    if source in sources:
        raise KeyError(f"source {source} is already registered for architecture {architecture}")
    for s in step_names:
        if s not in _steps.get(architecture, {}):
            raise KeyError(f"adapter step {s} is not registered for architecture {architecture}")
    sources[source] = list(step_names)


def extend_adapter(architecture: str, source: str, adapter_steps: List[str]) -> None:
    """Appends registered steps to the adapter of a source that exists already
    (fms/utils/serialization.py:104-148).  The other sources of the architecture stay as they are."""
    if source not in _adapters.get(architecture, {}):
        raise KeyError(f"Source {source} must already be registered for architecture {architecture}")
    for s in adapter_steps:
        if s not in _steps.get(architecture, {}):
            raise KeyError(f"adapter step {s} is not registered for architecture {architecture}")
    _adapters[architecture][source] = _adapters[architecture][source] + list(adapter_steps)


def list_sources(architecture: str) -> List[str]:
    return list(_adapters.get(architecture, {}))


def get_adapted(architecture: str, source: str, tensors: Mapping[str, torch.Tensor],
                **kwargs) -> Dict[str, torch.Tensor]:
    """Runs the adapter's steps.  An unknown architecture or source leaves the names as they are
    (fms/utils/serialization.py:129-161)."""
    out = dict(tensors)
    for name in _adapters.get(architecture, {}).get(source, []):
        out = _steps[architecture][name](out, **kwargs)
    return out
