"""Checkpoint reading and seeded random weights."""

from .loader import CheckpointTensors, load_checkpoint, open_checkpoint
from .random_init import RandomTensors, random_tensors, write_model_folder

__all__ = ["CheckpointTensors", "RandomTensors", "load_checkpoint", "open_checkpoint", "random_tensors",
           "write_model_folder"]
