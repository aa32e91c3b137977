"""Configuration: architecture-neutral specs, family configs, and the architecture registry."""
from .specs import (AttentionSpec, ConfigError, ConvWindowAttentionSpec, GatedDeltaRuleSpec,
                    GatedMLPSpec, LatentAttentionSpec, LayerSpec, Mamba2Spec, MixerBranch, MLSTMSpec,
                    ModelSpec, MoESpec, NameLayout, NormSpec, ParallelMixersSpec, PassStart,
                    PooledWindowAttentionSpec, RampScaling, RetentionSpec, RopeSpec,
                    ScheduleEntry, ScoreSpec, WavelengthScaling)
from .qwen3 import Qwen3Config
from .gukidra import GukidraConfig
from .fikotar import FikotarConfig
from .ketopel import KetopelConfig
from .folivik import FolivikConfig
from .registry import (family_for, load_config, parse_config, read_config_json,
                       register_architecture, registered_architectures)

__all__ = [
    "AttentionSpec", "ConfigError", "GatedMLPSpec", "LayerSpec", "ModelSpec", "NameLayout",
    "NormSpec", "RopeSpec", "ScheduleEntry", "ScoreSpec", "Qwen3Config",
    "GukidraConfig", "FikotarConfig", "KetopelConfig", "FolivikConfig", "Mamba2Spec", "GatedDeltaRuleSpec",
    "LatentAttentionSpec", "PassStart", "RampScaling", "ConvWindowAttentionSpec", "RetentionSpec", "MixerBranch",
    "ParallelMixersSpec", "MoESpec", "WavelengthScaling", "MLSTMSpec", "PooledWindowAttentionSpec", "family_for", "load_config",
    "parse_config", "read_config_json", "register_architecture", "registered_architectures",
]
