from .model_config import ModelConfig, NiduvikConfig, Qwen3Config, SatedraConfig
from .runtime_config import RuntimeConfig

__all__ = ["ModelConfig", "NiduvikConfig", "Qwen3Config", "RuntimeConfig", "SatedraConfig"]
