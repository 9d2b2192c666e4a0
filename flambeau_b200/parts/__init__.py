"""Parts: import the built-in ones so that they are registered."""
from . import attention, block, embedding, feedforward, norms, positions  # noqa: F401
from .base import (FeedForward, KVRequirement, Mixer, Norm, Part, PositionEncoding, StateRequirement,  # noqa: F401
                   TensorSpec)
from .spec import (LayerCall, ModelSpec, PartSpec, build_part, part_class, register_part,  # noqa: F401
                   unregister_part)
