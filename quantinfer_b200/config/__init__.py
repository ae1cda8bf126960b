from .qwen3 import Qwen3Config
from .registry import (architectures, config_class_for, config_from_dict, load_config,
                       register_architecture)
from .bebuvik import BebuvikConfig
from .kiruvik import KiruvikConfig
from .dulotar import DulotarConfig
from .lemotar import LemotarConfig
from .spec import (AttentionSpec, BigramEmbeddingSpec, DenseFeedForwardSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec,
                   LatentAttentionSpec, LayerCall, LayerSpec, ModelSpec, NormSpec, ParallelLayerSpec, PositionSpec,
                   RotarySpec, ShortConvSpec, ClampedGLUSpec, GatedAttentionSpec, MoESpec, ReentrySpec, SandwichLayerSpec,
                   StateSpaceSpec, ConvPreNormLayerSpec, LightningAttentionSpec, MinGRUSpec, ParallelMixersSpec, TimeMixSpec,
                   GatedDeltaSpec, PostNormLayerSpec)

__all__ = [
    "Qwen3Config", "architectures", "config_class_for", "config_from_dict", "load_config",
    "register_architecture", "AttentionSpec", "EmbeddingSpec", "FeedForwardSpec", "HeadSpec",
    "LayerCall", "LayerSpec", "ModelSpec", "NormSpec", "PositionSpec", "BebuvikConfig", "BigramEmbeddingSpec",
    "DenseFeedForwardSpec", "LatentAttentionSpec", "ParallelLayerSpec", "RotarySpec", "ShortConvSpec",
    "KiruvikConfig", "ClampedGLUSpec", "GatedAttentionSpec", "MoESpec", "ReentrySpec", "SandwichLayerSpec", "StateSpaceSpec",
    "DulotarConfig", "ConvPreNormLayerSpec", "LightningAttentionSpec", "MinGRUSpec", "ParallelMixersSpec", "TimeMixSpec",
    "LemotarConfig", "GatedDeltaSpec", "PostNormLayerSpec",
]
