from .base import ConfigError, architecture_of, load_model_config, make_model_config, read_config_json, require
from .specs import (AttentionSpec, BlockSpec, DenseMLPSpec, GLASpec, GatedMLPSpec, LatentAttentionSpec, Mamba2Spec, MixerSlot,
                    ModelSpec, NormSpec, PostNormBlockSpec, RopeSpec, RoutedMLPSpec, ScheduleEntry, ClampedGLUSpec, MinGRUSpec,
                    PooledWindowAttentionSpec, StreamBlockSpec, TokenSideSpec)
from .falcon_h1 import FalconH1Config
from .dudurax import DuduraxConfig
from .kuvazen import KuvazenConfig
from .pupopel import PupopelConfig
from .zarisun import ZarisunConfig

__all__ = [
    "ConfigError", "architecture_of", "load_model_config", "make_model_config", "read_config_json", "require",
    "AttentionSpec", "BlockSpec", "GatedMLPSpec", "Mamba2Spec", "MixerSlot", "ModelSpec", "NormSpec",
    "RopeSpec", "ScheduleEntry", "FalconH1Config", "DuduraxConfig", "DenseMLPSpec", "GLASpec", "LatentAttentionSpec",
    "PostNormBlockSpec", "RoutedMLPSpec", "KuvazenConfig", "ClampedGLUSpec", "MinGRUSpec", "PooledWindowAttentionSpec",
    "StreamBlockSpec", "TokenSideSpec", "PupopelConfig", "ZarisunConfig",
]
