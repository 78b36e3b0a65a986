from .model_config import ModelConfig
from .specs import BlockSpec, DecoderSpec, FeedForwardSpec, LayerCall, MixerSpec, NormSpec, PositionSpec

__all__ = ["ModelConfig", "BlockSpec", "DecoderSpec", "FeedForwardSpec", "LayerCall", "MixerSpec", "NormSpec",
           "PositionSpec"]
