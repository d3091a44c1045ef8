"""Meta-format Llama checkpoints (`consolidated.*.pth`, sharded by tensor parallelism)."""

from ..checkpoint_maps import decoder_weight_maps, fuse_projections, unfuse_projections

weight_maps = decoder_weight_maps("meta")
to_halite_postprocess = fuse_projections
from_halite_preprocess = unfuse_projections
