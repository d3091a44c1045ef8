"""Hugging Face Qwen3 checkpoints (safetensors; q/k RMSNorm inside attention)."""

from ..checkpoint_maps import decoder_weight_maps, fuse_projections, unfuse_projections

weight_maps = decoder_weight_maps("hf", qk_norm=True)
to_halite_postprocess = fuse_projections
from_halite_preprocess = unfuse_projections
