"""Parts that models are assembled from; importing the package registers the built-in ones."""
from . import attention, basic, blocks, feed_forward  # noqa: F401
from .registry import (PartError, part_class, register_arrangement, register_feed_forward, register_mixer,
                       register_norm, register_part, register_position)
from .spec import (AttentionSpec, GatedDenseSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry,
                   SubLayerSpec, TensorDecl, default_schedule, pre_norm_layer)
