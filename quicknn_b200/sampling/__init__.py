"""Sampling: options in the reference's names, and the device-side sampler."""
from .options import GenerationOptions, OptionsError, seed_state
from .sampler import NonFiniteLogits, Sampler

__all__ = ["GenerationOptions", "OptionsError", "seed_state", "NonFiniteLogits", "Sampler"]
