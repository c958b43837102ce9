from .engine_config import EngineConfig, parse_dtype
from .model_spec import AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec, RopeSpec

__all__ = ["EngineConfig", "parse_dtype", "AttentionSpec", "GatedMLPSpec", "LayerSpec", "ModelSpec", "NormSpec",
           "RopeSpec"]
