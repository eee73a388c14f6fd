from .base import (ConfigReader, LayerCall, LayerSpec, ModelConfig, ModelPlan, PartSpec,  # noqa: F401
                   read_config_json)
from .gemma2 import Gemma2Config  # noqa: F401
