from .cache import BLOCK_TOKENS, Cache, KVGroup, KVLayerView, StateGroup, StateLayerView
from .requests import KVRequest, StateRequest
from .slots import BlockPool, CacheFull, SlotAllocator

__all__ = ["BLOCK_TOKENS", "Cache", "KVGroup", "KVLayerView", "StateGroup", "StateLayerView", "KVRequest",
           "StateRequest", "BlockPool", "CacheFull", "SlotAllocator"]
