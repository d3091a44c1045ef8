"""Shared skeleton of the pre-training experiments: DCLM text, sentencepiece tokenizer, packed
2048-token rows, AdamW (0.9, 0.95), linear warm-up + cosine decay, z-loss 1e-4, batch 320,
50k steps (reference: configs/lm/dense_662m.py:25-81 and siblings)."""

from functools import partial

from torch import optim

from halite_b200.conf import config_fn, field
from halite_b200.data import preprocess
from halite_b200.data.tokenizers.sentencepiece import SentencePieceTokenizer
from halite_b200.nn.loss import CrossEntropyLoss
from halite_b200.optim import lr_scheduler
from halite_b200.parallel.parallelize import parallelize

from ..data.dclm_samples import conf as data_conf

n_vocab = 32000
max_length = 2048
tokenizer_path = "/data/halite/llama2-tokenizer.model"


@config_fn
def pretrain(model, lr=1e-3, weight_decay=0.1, warmup=5000, batch_size=320, max_iter=50000, optimizer=None,
             postprocess=None, activation_checkpointing=True, output_dir="/data/runs/lm"):
    tokenizer = SentencePieceTokenizer(tokenizer_path)
    conf = field()
    conf.model = field(
        model=model,
        wrapper=partial(parallelize, param_dtype="bfloat16", reduce_dtype="float32",
                        activation_checkpointing=activation_checkpointing,
                        activation_checkpointing_config={"mode": "full"}))
    conf.data = field(
        train=data_conf, train_ratio=0.9998, eval=data_conf, eval_ratio=0.0002,
        preprocess=[preprocess.ReadRawText(), preprocess.Tokenize(tokenizer, bos=True, eos=True),
                    preprocess.SequencePacking(max_length + 1), preprocess.AutoregressiveSample()],
        collate_fn=preprocess.Collator(keys=("input", "target")))
    conf.training = field(
        train_batch_size=batch_size, eval_batch_size=batch_size, max_iter=max_iter, gradient_checkpointing=False,
        optimizer=optimizer if optimizer is not None else partial(optim.AdamW, lr=lr, betas=(0.9, 0.95)),
        scheduler=partial(lr_scheduler.cycle_scheduler, lr=lr, initial_multiplier=1e-6, warmup=warmup,
                          decay=("linear", "cos")),
        criterion=CrossEntropyLoss(z_loss=1e-4, fast=True), weight_decay=weight_decay, clip_grad_norm=1.0,
        n_epochs=1, postprocess=postprocess)
    conf.output = field(log_step=10, output_dir=output_dir)
    return conf
