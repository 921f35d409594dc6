from .model import GPTConfig
from .training import TrainingConfig, build_resume_config, default_linear_config
from .presets import PRESETS, apply_overrides, get_preset

__all__ = ["GPTConfig", "TrainingConfig", "build_resume_config", "default_linear_config",
           "PRESETS", "apply_overrides", "get_preset"]
