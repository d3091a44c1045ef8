"""The tiny pre-training experiment with Shampoo on replicated data parallelism (whole weight
matrices on every rank, gradients all-reduced over the replicate dimension)."""

import os
from functools import partial

from halite_b200.conf.loader import load_module
from halite_b200.optim.shampoo import AdamGraftingConfig, Shampoo
from halite_b200.parallel import parallelize

conf = load_module(os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_lm.py")).conf
conf.model.wrapper = partial(parallelize, param_dtype="float32", reduce_dtype="float32", data_parallel="ddp")
conf.training.optimizer = partial(Shampoo, lr=3e-3, betas=(0.9, 0.95), precondition_frequency=3, inv_root_override=2,
                                  grafting_config=AdamGraftingConfig(beta2=0.95, epsilon=1e-8))
conf.training.data_parallel_shard = 1
conf.training.data_parallel_replicate = int(os.environ.get("WORLD_SIZE", "1"))
