from .base import (ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry,
                   read_config_json)
from .kolorax import KoloraxConfig
from .pepolorn import PepolornConfig
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "LayerSpec", "ModelConfig", "ModelSpec", "PartSpec", "ScheduleEntry",
           "KoloraxConfig", "PepolornConfig", "Qwen3Config", "read_config_json"]
