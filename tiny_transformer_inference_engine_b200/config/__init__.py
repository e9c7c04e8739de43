from .model_config import ModelConfig, ConfigError, DEFAULT_ARCHITECTURE
from .engine_config import CacheConfig, SchedulerConfig, EngineConfig, COMPUTE_DTYPES

__all__ = ["ModelConfig", "ConfigError", "DEFAULT_ARCHITECTURE", "CacheConfig", "SchedulerConfig",
           "EngineConfig", "COMPUTE_DTYPES"]
