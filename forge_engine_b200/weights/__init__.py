"""Checkpoint reading and seeded random weights."""

from .loader import load_checkpoint
from .random_init import random_tensors, write_model_folder

__all__ = ["load_checkpoint", "random_tensors", "write_model_folder"]
