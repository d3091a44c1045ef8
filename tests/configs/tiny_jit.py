"""Miniature JiT diffusion run on synthetic colour blobs for the entry-point tests."""

import os
from functools import partial

from torch import optim

from halite_b200.conf import call, field
from halite_b200.conf.loader import load_module
from halite_b200.optim import lr_scheduler
from halite_b200.parallel.parallelize import parallelize
from halite_b200.projects.dit.dataset import SyntheticImages
from halite_b200.projects.dit.diffusion import Diffusion

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_jit = load_module(os.path.join(_ROOT, "configs/models/jit.py"))

conf = field()
conf.model = field(
    model=call[_jit.jit](image_size=16, patch_size=4, n_labels=10, dim=32, patch_dim=16, n_heads=2, head_dim=16,
                         n_layers=3, intermediate_size=64, in_context_len=2, in_context_start=1, qk_norm=True),
    parallelize=partial(parallelize, param_dtype="float32", reduce_dtype="float32"))
conf.data = field(train=SyntheticImages(64, 16, n_labels=10))
conf.training = field(
    train_batch_size=16, eval_batch_size=4, n_epochs=3, max_iter=10,
    optimizer=partial(optim.AdamW, lr=2e-3, betas=(0.9, 0.95), weight_decay=0),
    scheduler=partial(lr_scheduler.cycle_scheduler, lr=2e-3, initial_multiplier=1e-2, final_multiplier=1, warmup=0,
                      decay=("linear", "cos")),
    criterion=Diffusion(input_shape=(3, 16, 16), n_labels=10, steps=3, guidance_scale=2.0, guidance_interval=(0.1, 1.0)),
    ema=0.9, data_parallel_shard=int(os.environ.get("WORLD_SIZE", "1")))
conf.output = field(log_step=2, output_dir=os.environ.get("HB_TEST_OUT"), name="tiny", sampling_step=5, save_step=5)
