from .spec import PartSpec, LayerSpec, ModelSpec
from .base import (Part, Norm, PositionEncoding, Mixer, FeedForward, PagedKVSpec, SlotStateSpec,
                   register_part, unregister_part, build_part)
from .context import StepContext, GroupView, LayerCache
from .model import Model, Layer, expected_params

__all__ = ["PartSpec", "LayerSpec", "ModelSpec", "Part", "Norm", "PositionEncoding", "Mixer", "FeedForward",
           "PagedKVSpec", "SlotStateSpec", "register_part", "unregister_part", "build_part",
           "StepContext", "GroupView", "LayerCache", "Model", "Layer", "expected_params"]
