"""Configuration: typed specifications, the MiniCPM/FM9G config, the architecture registry."""
from .specs import (AttentionSpec, BlockSpec, ConfigError, ConvAttentionSpec, FrequencyRampSpec, GLUSpec, LatentAttentionSpec,
                    DeltaRuleSpec, StepVectorSpec, LayerNormSpec, LinearAttentionSpec, MLPSpec, ModelSpec, PairRotarySpec, ParallelMixerSpec, PostNormBlockSpec, ReinjectSpec, RMSNormSpec,
                    RopeSpec, RoutedExpertsSpec, RunEntry, SandwichBlockSpec, SelectiveScanSpec, SwiGLUSpec, default_order)
from .minicpm import MiniCPMConfig
from .sitelorn import SitelornConfig
from .vunelix import VunelixConfig
from .vipovik import VipovikConfig
from .fapenex import FapenexConfig
from .presets import PRESETS, Preset
from .registry import (architecture_names, config_class_for, read_config,
                       register_architecture)

# The names the reference's loader accepts for this decoder (scripts/jiuge.py:422, :437).
for _name in ("minicpm", "fm9g", "llama", "MiniCPMForCausalLM", "LlamaForCausalLM"):
    register_architecture(_name, MiniCPMConfig)

register_architecture("sitelorn", SitelornConfig)
register_architecture("vunelix", VunelixConfig)
register_architecture("vipovik", VipovikConfig)
register_architecture("fapenex", FapenexConfig)

__all__ = [
    "DeltaRuleSpec", "StepVectorSpec", "FapenexConfig",
    "MLPSpec", "ParallelMixerSpec", "VipovikConfig",
    "FrequencyRampSpec", "LatentAttentionSpec", "ReinjectSpec", "RoutedExpertsSpec", "SandwichBlockSpec", "SelectiveScanSpec", "VunelixConfig",
    "ConvAttentionSpec", "GLUSpec", "LayerNormSpec", "LinearAttentionSpec", "PairRotarySpec", "PostNormBlockSpec", "SitelornConfig",
    "AttentionSpec", "BlockSpec", "ConfigError", "ModelSpec", "RMSNormSpec", "RopeSpec",
    "RunEntry", "SwiGLUSpec", "default_order", "MiniCPMConfig", "architecture_names",
    "config_class_for", "read_config", "register_architecture", "PRESETS", "Preset",
]
