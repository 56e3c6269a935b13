from . import attention, block, embedding, layernorm, mlp, positions  # noqa: F401  (register)
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS,
                   POSITION_ENCODINGS, FeedForward, Mixer, Norm, Part, PositionEncoding,
                   register_arrangement, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position_encoding)
from .context import HostBatch, StepContext, StepPlan
from .model import DecoderModel
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec, TensorSpec, pre_norm_layer

__all__ = [n for n in dir() if not n.startswith("_")]
