from .base import (BuildContext, CacheNeed, DeferredSum, NormedStream, resolve, ModelSpec, ParamDecl, Part, PartSpec, ScheduleEntry, StateNeed,
                   make_part, part_class, register_part)
from . import (attention, block, experts, feedforward, gated_attention, gla, input_conv, latent_attention, linear_attention,  # noqa: F401
               mlstm, norm, pair, position, recurrent)  # noqa: F401  (registers the built-in parts)
