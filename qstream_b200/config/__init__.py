"""Typed configuration and the architecture registry."""
from .specs import (AttentionSpec, BlockSpec, DecayAttentionSpec, EmbeddingSpec, GatedDeltaSpec, GatedMlpSpec, GlaSpec, HeadSpec,
                    HyperConnectionSpec, LatentAttentionSpec, LayerRun, MlpSpec, MlstmSpec, ModelSpec, NormedEmbeddingSpec,
                    NormSpec, PairEmbeddingSpec, PairMixerSpec, PositionHalfSpec, PositionSpec, RmsNormSpec, RotaryHalfSpec,
                    RoutedExpertsSpec, StreamNormSpec, StreamSumNormSpec, WkvSpec)
from .registry import (architecture_names, config_class_for, config_from_dict, load_config,
                       register_architecture)
from .gptj import GptjConfig
from .lutelorn import LutelornConfig
from .fofinex import FofinexConfig
from .sefuvik import SefuvikConfig
from .nutatar import NutatarConfig

register_architecture(GptjConfig, GptjConfig.model_type)
register_architecture(LutelornConfig, LutelornConfig.model_type)
register_architecture(FofinexConfig, FofinexConfig.model_type)
register_architecture(SefuvikConfig, SefuvikConfig.model_type)
register_architecture(NutatarConfig, NutatarConfig.model_type)

__all__ = ["AttentionSpec", "BlockSpec", "DecayAttentionSpec", "EmbeddingSpec", "GatedMlpSpec", "HeadSpec",
           "LatentAttentionSpec", "LayerRun", "MlpSpec", "MlstmSpec", "ModelSpec", "NormedEmbeddingSpec", "NormSpec",
           "PairEmbeddingSpec", "PositionSpec", "RmsNormSpec", "RotaryHalfSpec", "RoutedExpertsSpec", "StreamNormSpec",
           "WkvSpec", "GatedDeltaSpec", "HyperConnectionSpec", "PairMixerSpec", "PositionHalfSpec", "StreamSumNormSpec",
           "GlaSpec", "GptjConfig", "LutelornConfig", "FofinexConfig", "SefuvikConfig", "NutatarConfig", "architecture_names",
           "config_class_for", "config_from_dict", "load_config", "register_architecture"]
