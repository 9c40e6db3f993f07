from .llama import LlamaConfig, RopeScaling
from .plan import (BlockSpec, ConnectionSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, MixerSpec,
                   ModelPlan, NormSpec, PositionSpec)
from .reader import KeyReader, read_json_file

__all__ = ["LlamaConfig", "RopeScaling", "BlockSpec", "ConnectionSpec", "EmbeddingSpec", "FeedForwardSpec", "HeadSpec",
           "LayerRun", "MixerSpec", "ModelPlan", "NormSpec", "PositionSpec", "KeyReader", "read_json_file"]
