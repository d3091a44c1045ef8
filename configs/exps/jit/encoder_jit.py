"""Encoder-JiT-L/16 on ImageNet 256x256: six conditional JiT blocks on a SigLIP2-large encoder
(first four blocks unconditioned), same diffusion objective and schedule as the plain JiT run
(reference: configs/exps/jit/encoder_jit.py)."""

from functools import partial

from halite_b200.conf import call
from halite_b200.models.models.jit import encoder_jit_block_iterator
from halite_b200.parallel.parallelize import parallelize
from halite_b200.projects.common.config import load_model

from ...models.encoder_jit import encoder_jit
from .jit import conf

conf.training.freeze_encoder = False
conf.output.output_dir = "/data/runs/encoder_jit"


def encoder_jit_l_16(encoder_checkpoint="/data/halite/siglip2_large_patch16_256"):
    conf.model = load_model(encoder_checkpoint)
    conf.model.wrapper = call[encoder_jit](
        image_size=256, patch_size=16, n_labels=1000, dim=1024, patch_dim=128, n_heads=16, head_dim=1024 // 16,
        n_layers=6, intermediate_size=int(4096 * 2 / 3), in_context_len=32, qk_norm=True, cond_start_id=4)
    conf.model.parallelize = partial(parallelize, param_dtype="bfloat16", reduce_dtype="float32",
                                     activation_checkpointing=False, reshard_after_forward=True,
                                     block_iterator=encoder_jit_block_iterator)
    return conf
