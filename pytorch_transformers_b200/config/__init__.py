from .base import ConfigError, ModelConfig
from .falcon import FalconConfig
from .generation import GenerationConfig
from .pafevik import PafevikConfig
from .zalunex import ZalunexConfig
from .pogezen import PogezenConfig
from .figudra import FigudraConfig
from .registry import AutoConfig, Architecture, lookup, lookup_config, register_architecture, registered
