from tinyserve_llm_b200.config.duduvik import DuduvikConfig, duduvik_model_spec
from tinyserve_llm_b200.config.llama import ConfigError, LlamaConfig, llama_model_spec
from tinyserve_llm_b200.config.registry import (
    ARCHITECTURES,
    Architecture,
    load_model_spec,
    read_config_json,
    register_architecture,
    resolve_architecture,
)
from tinyserve_llm_b200.config.spec import (
    AttentionSpec,
    BlockSpec,
    GatedMLPSpec,
    InlineRotarySpec,
    LatentAttentionSpec,
    LinearRecurrenceSpec,
    Llama3Scaling,
    ModelSpec,
    PartSpec,
    RMSNormSpec,
    RotarySpec,
    RoutedExpertsSpec,
    RunEntry,
    StreamRMSNormSpec,
)

__all__ = [
    "ARCHITECTURES", "Architecture", "AttentionSpec", "BlockSpec", "ConfigError", "GatedMLPSpec",
    "DuduvikConfig", "InlineRotarySpec", "LatentAttentionSpec", "LinearRecurrenceSpec", "RoutedExpertsSpec",
    "StreamRMSNormSpec", "duduvik_model_spec", "Llama3Scaling", "LlamaConfig", "ModelSpec", "PartSpec", "RMSNormSpec", "RotarySpec", "RunEntry",
    "llama_model_spec", "load_model_spec", "read_config_json", "register_architecture",
    "resolve_architecture",
]
