"""Base class of every architecture's typed configuration.

Behaviour follows ``fms.utils.config.ModelConfig`` (fms/utils/config.py:14-88): JSON load and save, keys
that the dataclass does not know are ignored on load, ``updated(**kw)`` returns a deep copy with
overrides and reports unknown names.
"""
from __future__ import annotations

import copy
import dataclasses
import json
import logging
import os
from typing import Any, Dict, TypeVar, Union

logger = logging.getLogger(__name__)

T = TypeVar("T", bound="ModelConfig")


@dataclasses.dataclass
class ModelConfig:
    @classmethod
    def load(cls, json_file: Union[str, os.PathLike]):
        with open(json_file, "r", encoding="utf-8") as reader:
            return cls.from_dict(json.load(reader))

    @classmethod
    def from_dict(cls, values: Dict[str, Any]):
        known = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in values.items() if k in known})

    def as_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    def save(self, file_path: Union[str, os.PathLike]) -> None:
        with open(file_path, "w", encoding="utf-8") as f:
            json.dump(self.as_dict(), f)

    def updated(self: T, **kwargs) -> T:
        clone = copy.deepcopy(self)
        unknown = []
        for k, v in kwargs.items():
            if hasattr(clone, k):
                setattr(clone, k, v)
            else:
                unknown.append(k)
        if unknown:
            logger.info("unknown parameters while updating the configuration: %s", unknown)
        post = getattr(clone, "__post_init__", None)
        if post is not None:
            post()
        return clone
