"""A single-GPU inference engine for the Llama-style multi-query GPT, written for B200 (sm_100a)."""
from .config import ModelConfig, EngineConfig, CacheConfig, SchedulerConfig
from .sampling import SamplingParams
from .engine import Engine, load_model, generate_ids, StepEntry
from .weights import write_random_model, WeightError
from .registry import register_model, register_part

__all__ = ["ModelConfig", "EngineConfig", "CacheConfig", "SchedulerConfig", "SamplingParams", "Engine",
           "load_model", "generate_ids", "StepEntry", "write_random_model", "WeightError",
           "register_model", "register_part"]
