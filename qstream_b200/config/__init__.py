"""Typed configuration and the architecture registry."""
from .specs import (AttentionSpec, BlockSpec, EmbeddingSpec, HeadSpec, LayerRun, MlpSpec,
                    ModelSpec, NormSpec, PositionSpec)
from .registry import (architecture_names, config_class_for, config_from_dict, load_config,
                       register_architecture)
from .gptj import GptjConfig

register_architecture(GptjConfig, GptjConfig.model_type)

__all__ = ["AttentionSpec", "BlockSpec", "EmbeddingSpec", "HeadSpec", "LayerRun", "MlpSpec",
           "ModelSpec", "NormSpec", "PositionSpec", "GptjConfig", "architecture_names",
           "config_class_for", "config_from_dict", "load_config", "register_architecture"]
