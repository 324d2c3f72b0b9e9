"""Plan builders; importing this package registers the architectures."""
from . import dense_decoder
from .dense_decoder import build_dense_decoder_plan

__all__ = ["build_dense_decoder_plan", "dense_decoder"]
