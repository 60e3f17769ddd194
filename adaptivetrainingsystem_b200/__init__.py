"""adaptivetrainingsystem_b200 -- a Blackwell-native (sm_100a) sparse-transformer training and inference framework."""
__version__ = "0.1.0"
from .config import Config, ConfigPresets, ConfigManager, ModelConfig, DeepSeekConfig
