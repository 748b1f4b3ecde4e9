from . import attention, block, embedding, feed_forward, linear_attention, norm, parallel, position, reentry  # noqa: F401  (register the built-in parts)
from .registry import build_part, part_factory, register_part, unregister_part  # noqa: F401
from .spec import LayerSpec, ModelSpec, ParamSpec, PartSpec, ScheduleEntry  # noqa: F401
