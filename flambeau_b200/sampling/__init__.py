from .params import SamplingParams, uniform_for  # noqa: F401
