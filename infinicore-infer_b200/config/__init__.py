"""Configuration: typed specifications, the MiniCPM/FM9G config, the architecture registry."""
from .specs import (AttentionSpec, BlockSpec, ConfigError, ModelSpec, RMSNormSpec, RopeSpec,
                    RunEntry, SwiGLUSpec, default_order)
from .minicpm import MiniCPMConfig
from .presets import PRESETS, Preset
from .registry import (architecture_names, config_class_for, read_config,
                       register_architecture)

# The names the reference's loader accepts for this decoder (scripts/jiuge.py:422, :437).
for _name in ("minicpm", "fm9g", "llama", "MiniCPMForCausalLM", "LlamaForCausalLM"):
    register_architecture(_name, MiniCPMConfig)

__all__ = [
    "AttentionSpec", "BlockSpec", "ConfigError", "ModelSpec", "RMSNormSpec", "RopeSpec",
    "RunEntry", "SwiGLUSpec", "default_order", "MiniCPMConfig", "architecture_names",
    "config_class_for", "read_config", "register_architecture", "PRESETS", "Preset",
]
