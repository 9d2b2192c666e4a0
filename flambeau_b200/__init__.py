"""flambeau_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

    from flambeau_b200 import generate
    tokens = generate("model_dir", [[1, 2, 3]], max_tokens=16)
"""
from . import models  # noqa: F401  (registers the built-in architectures)
from .config.registry import known_architectures, load_config, register_architecture  # noqa: F401
from .sampling.params import SamplingParams  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    # the engine pulls in the CUDA library; import it only when asked for
    if name in ("generate", "Generator"):
        from .engine import generate as _g
        return getattr(_g, name)
    if name in ("Engine", "EngineOptions"):
        from .engine import step as _s
        return getattr(_s, name)
    raise AttributeError(name)
