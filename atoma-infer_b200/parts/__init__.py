from .base import (Block, EntryInfo, FeedForward, LayerCache, Mixer, Norm, Part, PositionEncoding, Runtime,
                   StepContext)
from .model import DecoderModel, LayerRun, LayerSpec, ModelSpec, declared_tensors
