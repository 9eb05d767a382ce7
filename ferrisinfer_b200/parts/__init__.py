"""Parts of a layer (mixer, feed-forward, norm, position encoding, block) and the model built from them."""

from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the built-in kinds)
from .base import (FeedForward, FixedState, LayerCache, Mixer, Norm, PagedKV, PagedMeta, Part, PositionEncoding,
                   SeqInfo, StepContext)
from .model import DecoderModel, build_model
from .plan import (LayerPlan, ModelPlan, PartSpec, RunStep, TensorSpec, build_part, register_part,
                   registered_parts)
