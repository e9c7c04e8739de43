from .batch import StepEntry, BatchPacker
from .step import Stepper
from .scheduler import Scheduler, Request
from .engine import Engine, load_model, generate_ids

__all__ = ["StepEntry", "BatchPacker", "Stepper", "Scheduler", "Request", "Engine", "load_model", "generate_ids"]
