"""Parts a layer is made of.  Importing this package registers the built-in parts."""
from . import norm, position, attention, mlp, block  # noqa: F401  (registration)
from .base import (Part, Norm, PositionEncoding, Mixer, FeedForward, Block, LayerContext,
                   WeightSpec, KVNeed, StateNeed, MATRIX, VECTOR, INT_TABLE)
from .description import PartSpec, LayerSpec, ScheduleEntry, ModelDescription
from .model import Model, CacheBinding, build_part
