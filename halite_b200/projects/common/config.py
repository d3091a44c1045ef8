"""Typed sections shared by every entry point's configuration, and the model-folder format
(`config.json` + tokenizer files) that sits beside checkpoints
(reference: projects/common/config.py:14-268; field names are kept so existing experiment
configurations validate unchanged).
"""

from __future__ import annotations

import copy
import dataclasses
import json
import os
import shutil
from typing import Any

from pydantic import BaseModel, StrictBool, StrictInt, StrictStr

from halite_b200.conf import Config, Instance, deserialize, exempt, field
from halite_b200.models.config import TransformerConfig

# sections of config.json that describe how to rebuild a model
_MODEL_SECTIONS = ("model", "model_infer", "tokenizer", "parallelize", "parallelize_infer")
# files that make up a Hugging Face tokenizer folder
_HF_TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json", "vocab.json", "merges.txt")
_TOKENIZER_CONF = "halite_tokenizer_config.json"


def check_tokenizer_exists(checkpoint_path: str):
    """Path to hand to the tokenizer constructor: the sentencepiece file itself, or the folder
    for a `tokenizer.json`; None when the folder has no tokenizer."""
    spm = os.path.join(checkpoint_path, "tokenizer.model")
    if os.path.exists(spm):
        return spm
    if os.path.exists(os.path.join(checkpoint_path, "tokenizer.json")):
        return checkpoint_path
    return None


def get_tokenizer_files(checkpoint_path: str):
    if checkpoint_path is None:
        return []
    if os.path.isfile(checkpoint_path):
        return [checkpoint_path]
    spm = os.path.join(checkpoint_path, "tokenizer.model")
    if os.path.exists(spm):
        return [spm]
    return [os.path.join(checkpoint_path, n) for n in _HF_TOKENIZER_FILES
            if os.path.exists(os.path.join(checkpoint_path, n))]


def _plain(section):
    if section is None or isinstance(section, (str, int, float, bool)):
        return section
    if dataclasses.is_dataclass(section):
        return dataclasses.asdict(section)
    if isinstance(section, BaseModel):
        return section.model_dump()
    if hasattr(section, "to_dict"):
        return section.to_dict()
    return section


def save_model(model_config, checkpoint_path):
    """Write `config.json`, copy the tokenizer's files and store how to construct it."""
    os.makedirs(checkpoint_path, exist_ok=True)
    doc = {name: _plain(getattr(model_config, name, None)) for name in _MODEL_SECTIONS}
    doc["model_conf"] = _plain(getattr(model_config, "model_conf", None))
    with open(os.path.join(checkpoint_path, "config.json"), "w") as f:
        json.dump(doc, f, indent=2)
    tok = getattr(model_config, "tokenizer", None)
    if tok is None:
        return
    source = tok.get("model_path") if hasattr(tok, "get") else getattr(tok, "model_path", None)
    for path in get_tokenizer_files(source):
        dst = os.path.join(checkpoint_path, os.path.basename(path))
        if os.path.abspath(path) != os.path.abspath(dst):
            shutil.copy(path, dst)
    with open(os.path.join(checkpoint_path, _TOKENIZER_CONF), "w") as f:
        json.dump(_plain(tok), f, indent=2)


class Model(Config):
    model_conf: TransformerConfig | None = None
    model: Instance | None = None
    model_infer: Instance | None = None
    tokenizer: Instance | None = None
    parallelize: Instance | None = None
    parallelize_infer: Instance | None = None
    wrapper: Instance | None = None
    policy: dict[str, Any] | None = None
    checkpoint_path: StrictStr | None = None

    def model_post_init(self, __context):
        """With only `checkpoint_path` given, take everything else from its `config.json`."""
        if self.checkpoint_path is None or self.model is not None:
            return
        with open(os.path.join(self.checkpoint_path, "config.json")) as f:
            doc = json.load(f)
        for name in _MODEL_SECTIONS:
            if doc.get(name) is not None:
                setattr(self, name, Instance(doc[name]))
        tok_path = check_tokenizer_exists(self.checkpoint_path)
        if tok_path is not None and self.tokenizer is not None:
            self.tokenizer["model_path"] = tok_path
        if doc.get("model_conf") is not None:
            self.model_conf = TransformerConfig(**doc["model_conf"])

    def save(self, checkpoint_path):
        save_model(self, checkpoint_path)


@exempt
def load_model(checkpoint_path):
    """Config-file helper: `model=load_model("/path")` yields the `Model` section of a saved
    model folder."""
    doc = deserialize(os.path.join(checkpoint_path, "config.json"))
    conf = field()
    for name in _MODEL_SECTIONS:
        if name in doc and doc[name] is not None:
            conf[name] = doc[name]
    tok_path = check_tokenizer_exists(checkpoint_path)
    if tok_path is not None and "tokenizer" in conf:
        conf["tokenizer"]["model_path"] = tok_path
    if doc.get("model_conf") is not None:
        conf["model_conf"] = doc["model_conf"]
    conf["checkpoint_path"] = checkpoint_path
    return conf


def get_tokenizer(model):
    """Tokenizer `Instance` of a model section: its own, else the one stored in its folder."""
    get = model.get if hasattr(model, "get") else lambda k, d=None: getattr(model, k, d)
    ckpt = get("checkpoint_path")
    if get("tokenizer") is not None:
        tok = Instance(copy.deepcopy(_plain(get("tokenizer"))))
        if ckpt is not None and check_tokenizer_exists(ckpt) is not None:
            tok["model_path"] = check_tokenizer_exists(ckpt)
        return tok
    if ckpt is None:
        raise ValueError("tokenizer or checkpoint is not specified")
    with open(os.path.join(ckpt, _TOKENIZER_CONF)) as f:
        tok = Instance(json.load(f))
    tok["model_path"] = check_tokenizer_exists(ckpt)
    return tok


class Training(Config):
    train_batch_size: StrictInt | None = None
    eval_batch_size: StrictInt | None = None
    max_iter: StrictInt | None = None
    gradient_checkpointing: StrictBool = False
    optimizer: Instance
    scheduler: Instance
    criterion: Instance | None = None
    model_initializer: Instance | None = None
    postprocess: Instance | None = None
    weight_decay: float = 0.0
    clip_grad_norm: float | None = None
    n_epochs: int = 1
    eval_step: int = 1000
    seed: int = 42
    train_step_fn: Instance | None = None
    eval_step_fn: Instance | None = None
    data_parallel_replicate: StrictInt = 1
    data_parallel_shard: StrictInt = 1
    tensor_parallel: StrictInt = 1
    pipeline_parallel: StrictInt = 1
    calc_loss_in_model: StrictBool = False


class Dataset(Config):
    root: str
    ratios: dict[str, float]
    shards: dict[str, dict[str, int]]


class Data(Config):
    train: Dataset | Instance | None = None
    eval: Dataset | Instance | None = None
    train_ratio: float = 1.0
    eval_ratio: float = 1.0
    preprocess: list[Instance] | None = None
    preprocess_eval: list[Instance] | None = None
    collate_fn: Instance | None = None
    collate_fn_eval: Instance | None = None


class Output(Config):
    log_step: StrictInt                       # console / tracker logging period
    save_step: StrictInt | None = None        # checkpoint period
    output_dir: StrictStr | None = None
    wandb_log_step: StrictInt | None = None   # defaults to log_step
    project: StrictStr | None = None
    name: StrictStr | Instance | None = None

    def model_post_init(self, __context):
        if self.wandb_log_step is None:
            self.wandb_log_step = self.log_step


class Experiment(Config):
    conf: dict[str, Any] | None = None
    tags: dict[str, Any] | None = None
