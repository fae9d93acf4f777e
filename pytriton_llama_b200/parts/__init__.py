"""Parts of a decoder layer.  Importing this package registers the built-in kinds."""
from .base import (CacheNeed, Part, PartSpec, Runtime, TensorSpec, build_part, part_kinds,  # noqa: F401
                   register_part)
from . import (attention, block, chunk_attention, clamped_glu, delta_rule, depth_average, gated_side, gelu_mlp, general_delta, gla, hyper,  # noqa: F401
               latent_attention, layernorm, parallel, retention, rmsnorm, rope, routed_experts, scan, swiglu, window_attention)
