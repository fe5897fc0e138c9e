"""Greedy and temperature sampling."""

from .sampler import Sampler

__all__ = ["Sampler"]
