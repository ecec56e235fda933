from .registry import (BuildContext, CacheNeed, Mixer, Part, build_part, register_part, registered_parts, to_compute)
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep, spec_param_specs
from . import (attention, block, delta_rule, diff_attention, embedding, feed_forward, gla, latent_attention, mamba2,
               masked_attention, norm, rotary, routed_ff, selective_scan, side_by_side)  # noqa: F401  (register the kinds)

__all__ = ["BuildContext", "CacheNeed", "Mixer", "Part", "build_part", "register_part", "registered_parts",
           "to_compute", "LayerSpec", "ModelSpec", "PartSpec", "RunStep", "spec_param_specs"]
