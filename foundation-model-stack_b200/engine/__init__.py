from .batch import Batch
from .decoder import Decoder
from .step import Engine

__all__ = ["Batch", "Decoder", "Engine"]
