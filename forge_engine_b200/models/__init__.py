"""Model assembly from specs."""

from .decoder import DecoderModel, expected_tensors

__all__ = ["DecoderModel", "expected_tensors"]
