from .model_config import ConfigError, Qwen2Config, parse_qwen2_config, read_config_json
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

__all__ = ["ConfigError", "Qwen2Config", "parse_qwen2_config", "read_config_json", "LayerSpec", "ModelSpec",
           "PartSpec", "ScheduleEntry", "TensorSpec"]
