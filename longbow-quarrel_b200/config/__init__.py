from .base import ConfigError, read_config_json
from .fetorax import FetoraxConfig, FetoraxLayer, Rotation
from .lavutar import LavutarConfig, LavutarLayer
from .llama import LlamaConfig, RopeScaling, FULL_ATTENTION, SLIDING_ATTENTION
from .raritar import RaritarConfig, RaritarLayer
from .zoporax import ZoporaxConfig, ZoporaxLayer
from .registry import (Architecture, architecture_of, load_config, register_architecture,
                       registered_architectures)

__all__ = ["ConfigError", "read_config_json", "LlamaConfig", "FetoraxConfig", "FetoraxLayer", "Rotation", "ZoporaxConfig", "ZoporaxLayer", "RaritarConfig", "RaritarLayer", "LavutarConfig", "LavutarLayer", "RopeScaling", "FULL_ATTENTION",
           "SLIDING_ATTENTION", "Architecture", "architecture_of", "load_config",
           "register_architecture", "registered_architectures"]
