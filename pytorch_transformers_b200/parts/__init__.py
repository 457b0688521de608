from .base import (BuildContext, CacheNeed, DeferredSum, resolve, ModelSpec, ParamDecl, Part, PartSpec, ScheduleEntry, StateNeed,
                   make_part, part_class, register_part)
from . import attention, block, feedforward, norm, position  # noqa: F401  (registers the built-in parts)
