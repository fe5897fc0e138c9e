"""The generic decoder; architectures differ only in the ModelSpec their configuration yields."""

from .decoder import Decoder

__all__ = ["Decoder"]
