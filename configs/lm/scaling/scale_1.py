"""Scaling series, smallest point: dim 96, 4 heads, 3 layers, 1024-token rows, Llama-3
vocabulary; 50k steps of batch 64 at learning rate 3e-4 with decoupled weight decay 1e-4 / lr."""

from functools import partial

from torch import optim

from halite_b200.conf import call
from halite_b200.data import preprocess
from halite_b200.data.tokenizers.llama3 import Llama3Tokenizer
from halite_b200.nn.loss import CrossEntropyLoss

from ...models.scaling.base import transformer
from ..base import pretrain

lr = 3e-4
rows = 1024
tokenizer = Llama3Tokenizer("/data/halite/llama3-tokenizer.model")

conf = call[pretrain](call[transformer](
    vocab_size=128256, dim=96, n_heads=4, head_dim=24, n_layers=3, intermediate_size=call[int](96 * 3.5),
    max_position_embeddings=rows, rms_norm_epsilon=1e-6), lr=lr, weight_decay=1e-4 / lr, batch_size=64,
    optimizer=partial(optim.AdamW, lr=lr), activation_checkpointing=False)
conf.data.preprocess = [preprocess.ParseFeatures(), preprocess.Tokenize(tokenizer, bos=True, eos=True),
                        preprocess.SequencePacking(rows + 1), preprocess.AutoregressiveSample()]
conf.data.train_ratio, conf.data.eval_ratio = 0.9999, 0.0001
conf.training.criterion = CrossEntropyLoss()
