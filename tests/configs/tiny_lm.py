"""Experiment configuration used by the entry-point tests: a 2-layer Llama-style model on a
byte-tokenised record-file corpus."""

import os
from functools import partial

from torch import nn, optim

from halite_b200.conf import field
from halite_b200.conf.loader import load_module
from halite_b200.data import preprocess
from halite_b200.data.tokenizers import ByteTokenizer
from halite_b200.nn.loss import CrossEntropyLoss
from halite_b200.optim import lr_scheduler
from halite_b200.parallel import parallelize

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_zoo = load_module(os.path.join(_ROOT, "configs/models/transformer.py"))

conf = field()

conf.model = field(
    model=_zoo.transformer(vocab_size=260, dim=64, n_heads=4, head_dim=16, n_layers=2, intermediate_size=176,
                           context_len=64, n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=True,
                           gated_ff_split=True, init=partial(nn.init.normal_, std=0.02)),
    wrapper=partial(parallelize, param_dtype="float32", reduce_dtype="float32"),
)

_data_root = os.environ.get("HB_TEST_DATA", "/nonexistent")
_spec = field(root=_data_root, ratios={"a": 0.8, "b": 0.2},
              shards={"a": {"s0.hbrec": 200}, "b": {"s0.hbrec": 50}})
conf.data = field(
    train=_spec, eval=_spec, train_ratio=0.9, eval_ratio=0.1,
    preprocess=[preprocess.ParseFeatures(),
                preprocess.Tokenize(ByteTokenizer(), bos=True, eos=True),
                preprocess.SequencePacking(33),
                preprocess.AutoregressiveSample()],
    collate_fn=preprocess.Collator(keys=("input", "target")),
)

conf.training = field(
    train_batch_size=8, eval_batch_size=8, max_iter=12,
    optimizer=partial(optim.AdamW, lr=3e-3, betas=(0.9, 0.95)),
    scheduler=partial(lr_scheduler.cycle_scheduler, lr=3e-3, warmup=2, decay=("linear", "cos")),
    criterion=CrossEntropyLoss(),
    weight_decay=0.1, clip_grad_norm=1.0, eval_step=6, n_epochs=4,
    data_parallel_shard=int(os.environ.get("WORLD_SIZE", "1")),
)

conf.output = field(log_step=3, save_step=6, output_dir=os.environ.get("HB_TEST_OUT"))
