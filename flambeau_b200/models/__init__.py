"""Architectures: import the built-in ones so that they are registered."""
from . import mistral  # noqa: F401
from .decoder import DecoderModel  # noqa: F401
