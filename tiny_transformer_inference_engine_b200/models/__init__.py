"""Architectures (as data) and the generic model.  Importing registers the built-in one."""
from .model import Model
from . import mqa_gpt  # noqa: F401  (registration)
