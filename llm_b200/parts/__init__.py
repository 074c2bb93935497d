from . import (attention, block, diff_attention, embedding, feed_forward, gla, hyper, latent_attention, norm, position, recurrent,  # noqa: F401
               routed)  # noqa: F401 (register kinds)
from .base import (CacheNeed, ParamInfo, Part, ResidualStream, StateNeed, build_part, part_class,
                   register_part)

__all__ = ["CacheNeed", "ParamInfo", "Part", "ResidualStream", "StateNeed", "build_part", "part_class",
           "register_part"]
