"""Typed configuration, read from config.json, and the architecture registry."""

from .registry import (ConfigError, ModelConfig, TensorNames, architecture_names, config_from_dict, load_config,
                       register_architecture, save_config)
from .specs import (ActMLPSpec, AttentionSpec, BiasedAttentionSpec, BlockSpec, BranchNormSpec, CausalConvSpec, PostNormBlockSpec,
                    SinusoidSpec, TalkingAttentionSpec, DiffAttentionSpec, GatedMLPSpec, GLASpec, GroupedNormSpec,
                    LatentAttentionSpec, ModelSpec, MoESpec, NormSpec, PairRopeSpec, ParallelBlockSpec, RopeSpec,
                    ScaledHalfRopeSpec, StreamBlockSpec, StreamNormSpec, WKVSpec, KeyValueAttentionSpec, MLSTMSpec, PairMixerSpec,
                    SandwichBlockSpec, LoopSpec)

__all__ = ["ConfigError", "ModelConfig", "TensorNames", "architecture_names", "config_from_dict", "load_config",
           "register_architecture", "save_config", "AttentionSpec", "BlockSpec", "GatedMLPSpec", "ModelSpec",
           "NormSpec", "RopeSpec", "BiasedAttentionSpec", "GroupedNormSpec", "LatentAttentionSpec", "PairRopeSpec",
           "ParallelBlockSpec", "WKVSpec", "DiffAttentionSpec", "GLASpec", "MoESpec", "ScaledHalfRopeSpec", "StreamBlockSpec",
           "StreamNormSpec", "ActMLPSpec", "BranchNormSpec", "CausalConvSpec", "PostNormBlockSpec", "SinusoidSpec",
           "TalkingAttentionSpec", "KeyValueAttentionSpec", "MLSTMSpec", "PairMixerSpec", "SandwichBlockSpec", "LoopSpec"]
