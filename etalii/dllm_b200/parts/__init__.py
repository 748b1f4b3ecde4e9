from . import (attention, block, differential_attention, embedding, feed_forward, linear_attention, mixture, norm,  # noqa: F401
               parallel, position, reentry)  # (register the built-in parts)
from .registry import build_part, part_factory, register_part, unregister_part  # noqa: F401
from .spec import LayerSpec, ModelSpec, ParamSpec, PartSpec, ScheduleEntry  # noqa: F401
