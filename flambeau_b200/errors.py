"""The error classes that a user's input can cause (a bad model folder, configuration, weight file, step record
or option), gathered for the command line programs, which print them in one line instead of a stack trace.
Everything else (a kernel that flagged a fault, a failed build) keeps its trace."""
from __future__ import annotations

from .cache.pages import PageError
from .config.base import ConfigError
from .engine.batch import BatchError
from .engine.runtime import NoDeviceError
from .weights.loader import WeightError
from .weights.safetensors_io import SafetensorsError

USER_ERRORS = (ConfigError, WeightError, SafetensorsError, BatchError, PageError, NoDeviceError, FileNotFoundError,
               ValueError)

__all__ = ["USER_ERRORS"]
