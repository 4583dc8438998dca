from .specs import (BigramSpec, BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ShortConvSpec)
from .registry import (ArchitectureEntry, UnknownArchitecture, lookup_architecture,
                       read_config_json, register_architecture, registered_architectures)
from .qwen2 import ConfigError, Qwen2Config
from .vunovik import VunovikConfig
from .gisirax import GisiraxConfig
from .lipizen import LipizenConfig
from .netezen import NetezenConfig
from . import shapes

__all__ = ["BlockSpec", "FeedForwardSpec", "MixerSpec", "ModelSpec", "NormSpec", "PositionSpec",
           "ArchitectureEntry", "UnknownArchitecture", "lookup_architecture", "read_config_json",
           "register_architecture", "registered_architectures", "ConfigError", "Qwen2Config", "VunovikConfig", "GisiraxConfig", "LipizenConfig", "NetezenConfig", "ShortConvSpec", "BigramSpec"]
