from .base import (Block, Embedding, EntryInfo, FeedForward, Head, LayerCache, Mixer, Norm, Part, PositionEncoding,
                   Runtime, StepContext)
from .model import DecoderModel, LayerRun, LayerSpec, ModelSpec, declared_tensors
