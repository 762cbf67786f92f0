from .model_config import ModelConfig, NiduvikConfig, Qwen3Config
from .runtime_config import RuntimeConfig

__all__ = ["ModelConfig", "NiduvikConfig", "Qwen3Config", "RuntimeConfig"]
