"""Configuration: part specs, the Qwen3 config, engine settings and the registry."""

from .engine import EngineConfig, SchedulerConfig
from .nuvivik import NuvivikConfig
from .qwen3 import Qwen3Config
from .registry import (
    Architecture,
    architecture_of,
    known_architectures,
    read_model_config,
    register_architecture,
)
from .specs import (
    AttentionSpec,
    DenseMLPSpec,
    DifferentialSpec,
    GatedMLPSpec,
    GatedRecurrenceSpec,
    LatentAttentionSpec,
    LayerNormSpec,
    LayerSpec,
    LinearRecurrenceSpec,
    ModelSpec,
    NoPositionSpec,
    NormSpec,
    OutputNormSpec,
    RotarySpec,
    RoutedMLPSpec,
    RunSpec,
    SandwichConvSpec,
    StreamMixSpec,
)
from .tekilorn import TekilornConfig
from .zabutar import ZabutarConfig
from .zofadra import ZofadraConfig

register_architecture(
    Architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, Qwen3Config.to_model_spec),
    replace=True,
)
register_architecture(
    Architecture("Zofadra", ZofadraConfig.from_dict, ZofadraConfig.to_model_spec),
    replace=True,
)
register_architecture(
    Architecture("Tekilorn", TekilornConfig.from_dict, TekilornConfig.to_model_spec),
    replace=True,
)

register_architecture(
    Architecture("Zabutar", ZabutarConfig.from_dict, ZabutarConfig.to_model_spec),
    replace=True,
)

register_architecture(
    Architecture("Nuvivik", NuvivikConfig.from_dict, NuvivikConfig.to_model_spec),
    replace=True,
)

__all__ = [
    "Architecture",
    "AttentionSpec",
    "DenseMLPSpec",
    "DifferentialSpec",
    "EngineConfig",
    "GatedMLPSpec",
    "GatedRecurrenceSpec",
    "LatentAttentionSpec",
    "LayerNormSpec",
    "LayerSpec",
    "LinearRecurrenceSpec",
    "ModelSpec",
    "NoPositionSpec",
    "NormSpec",
    "NuvivikConfig",
    "OutputNormSpec",
    "Qwen3Config",
    "RotarySpec",
    "RoutedMLPSpec",
    "RunSpec",
    "SandwichConvSpec",
    "SchedulerConfig",
    "StreamMixSpec",
    "TekilornConfig",
    "ZabutarConfig",
    "ZofadraConfig",
    "architecture_of",
    "known_architectures",
    "read_model_config",
    "register_architecture",
]
