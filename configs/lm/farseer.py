"""Data-quality scaling runs on the five Nemotron-CC tiers: a 202M decoder whose embedding is
initialised at dim**-1.5 and multiplied by dim**0.5, trained on a chosen mixture of the tiers;
the run name is derived from the hyper-parameters (reference: configs/lm/farseer.py:22-161).

Everything an experiment varies lives in `conf.hparams`; the rest of the tree refers to it, so
`hparams.lr=...` or `hparams.data_ratios.high=...` on the command line changes every dependent
value."""

from functools import partial

from torch import nn, optim

from halite_b200.conf import call, field
from halite_b200.data import preprocess
from halite_b200.data.tokenizers.sentencepiece import SentencePieceTokenizer
from halite_b200.models.embedding import TextEmbedding
from halite_b200.nn.loss import CrossEntropyLoss
from halite_b200.optim import lr_scheduler
from halite_b200.parallel.parallelize import parallelize
from halite_b200.projects.common.logging import hparam_to_name

from ..data import nemotron_cc
from ..models.transformer import transformer, use_fused_linear_cross_entropy

conf = field()
conf.hparams = field(
    lr=2 ** (-0.5 * 14), dim=1024, n_layers=16, intermediate_size=2752, weight_decay=0.1, n_vocab=32000,
    batch_size=16, tokenizer_path="/data/halite/llama2-tokenizer.model", max_length=2048,
    max_tokens=8192 * (10 ** 6), model_size="202m", data_setting="uniform",
    data_ratios={t: 0.2 for t in nemotron_cc.TIERS},
)
hp = conf.hparams.ref
tokenizer = SentencePieceTokenizer(hp.tokenizer_path)

conf.model = field(
    model=call[transformer](
        vocab_size=conf.hparams.n_vocab, dim=conf.hparams.dim, n_heads=8, head_dim=conf.hparams.dim // 8,
        n_layers=conf.hparams.n_layers, intermediate_size=conf.hparams.intermediate_size,
        context_len=conf.hparams.max_length, post_norm=False, attention_processor="torch",
        embedding=TextEmbedding(nn.Embedding(conf.hparams.n_vocab, conf.hparams.dim), 0,
                                embed_init=partial(nn.init.normal_, std=conf.hparams.dim ** -1.5),
                                multiplier=conf.hparams.dim ** 0.5)),
    wrapper=partial(parallelize, param_dtype="bfloat16", reduce_dtype="float32",
                    tensor_parallel_config={"enable_async_tp": True}, activation_checkpointing=True,
                    activation_checkpointing_config={"mode": "full", "selective": "op"}, force_fsdp=True),
)

conf.data = field(
    train=field(root=nemotron_cc.root, ratios=hp.data_ratios, shards=nemotron_cc.uniform.shards),
    train_ratio=0.9998,
    eval=nemotron_cc.uniform,
    eval_ratio=0.0002,
    preprocess=[preprocess.ReadRawText(), preprocess.Tokenize(tokenizer, bos=True, eos=True),
                preprocess.SequencePacking(hp.max_length + 1), preprocess.AutoregressiveSample()],
    collate_fn=preprocess.Collator(keys=("input", "target")),
)

conf.training = field(
    train_batch_size=hp.batch_size, eval_batch_size=256,
    max_iter=hp.max_tokens // hp.max_length // hp.batch_size,
    gradient_checkpointing=False,
    optimizer=partial(optim.AdamW, lr=hp.lr, betas=(0.9, 0.95)),
    scheduler=partial(lr_scheduler.cycle_scheduler, lr=hp.lr, initial_multiplier=1e-6,
                      final_multiplier=1e-6 / hp.lr, warmup=2000, decay=("linear", "cos")),
    criterion=CrossEntropyLoss(z_loss=1e-4, fast=True), weight_decay=hp.weight_decay, clip_grad_norm=1.0,
    n_epochs=1,
)

conf.output = field(
    log_step=10, output_dir="/data/runs/farseer",
    name=partial(hparam_to_name,
                 format="{model_size}@lr-{lr:.5f}_batch-{batch_size}_max_tokens-{max_tokens:.3e}_data-{data_setting}"),
)


def scale_202m():
    conf.model.model = use_fused_linear_cross_entropy(conf.model.model, z_loss=1e-4)
    conf.training.calc_loss_in_model = True
    return conf
