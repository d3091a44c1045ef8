"""Convert Meta / Hugging Face checkpoints into a model folder this package loads: a
`torch.distributed.checkpoint` directory with top-level key `model`, `config.json` and tokenizer
files (counterpart of the reference's scripts/tools/convert_checkpoint.py).

    python scripts/tools/convert_checkpoint.py --conf configs/models/qwen3/qwen3_0_6b.py \
        --tokenizer_type hf --tokenizer /path/to/hf_dir --out /path/out "/path/to/hf_dir/*.safetensors"

With `--reverse` the direction flips: a model folder is exported to foreign keys as
`--shards` tensor-parallel `.pth` files.
"""

import argparse
import json
import os
import shutil
from glob import glob

import torch
import torch.distributed.checkpoint as dcp

from halite_b200.conf import load_config
from halite_b200.logging import logger
from halite_b200.models.convert import convert_checkpoint

try:
    from safetensors import safe_open
except ImportError:  # pragma: no cover
    safe_open = None

_HF_FILES = ("tokenizer.json", "tokenizer_config.json", "vocab.json", "merges.txt")


def read_checkpoint(path):
    if path.endswith(".safetensors"):
        if safe_open is None:
            raise RuntimeError("safetensors is not installed")
        with safe_open(path, framework="pt", device="cpu") as f:
            return {k: f.get_tensor(k) for k in f.keys()}
    return torch.load(path, map_location="cpu", weights_only=True)


def to_plain(conf):
    return conf.to_dict() if hasattr(conf, "to_dict") else conf


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--conf", required=True)
    ap.add_argument("--conf_name", default=None)
    ap.add_argument("--tokenizer_type", default="sentencepiece", choices=["sentencepiece", "hf"])
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--out", required=True)
    ap.add_argument("--reverse", action="store_true")
    ap.add_argument("--shards", type=int, default=1)
    ap.add_argument("checkpoint_pattern")
    args = ap.parse_args(argv)

    conf = load_config(args.conf, config_name=args.conf_name)
    os.makedirs(args.out, exist_ok=True)
    if args.reverse:
        from halite_b200.conf import instantiate

        with torch.device("meta"):
            model = instantiate(conf.model)
        model.to_empty(device="cpu")
        sd = {"model": {k: v for k, v in model.state_dict().items()}}
        dcp.load(sd, checkpoint_id=args.checkpoint_pattern)
        outs = convert_checkpoint(sd["model"], conf.model_conf, conf.policy, mode="from_halite", n_shards=args.shards)
        outs = outs if isinstance(outs, list) else [outs]
        for i, shard in enumerate(outs):
            torch.save(shard, os.path.join(args.out, f"consolidated.{i:02d}.pth"))
        logger.info(f"wrote {len(outs)} shard(s) to {args.out}")
        return

    files = sorted(glob(args.checkpoint_pattern))
    logger.info(f"loading {len(files)} checkpoints")
    converted = convert_checkpoint([read_checkpoint(f) for f in files], conf.model_conf, conf.policy, mode="to_halite")
    with open(os.path.join(args.out, "config.json"), "w") as f:
        json.dump(to_plain(conf), f, indent=2)
    logger.info("saving checkpoints")
    dcp.save({"model": converted}, storage_writer=dcp.FileSystemWriter(args.out, thread_count=8))
    if conf.get("tokenizer") is not None:
        with open(os.path.join(args.out, "halite_tokenizer_config.json"), "w") as f:
            json.dump(to_plain(conf["tokenizer"]), f, indent=2)
    if args.tokenizer is not None:
        if args.tokenizer_type == "sentencepiece":
            shutil.copy(args.tokenizer, os.path.join(args.out, "tokenizer.model"))
        else:
            for name in _HF_FILES:
                src = os.path.join(args.tokenizer, name)
                if os.path.exists(src):
                    shutil.copy(src, os.path.join(args.out, name))
    logger.info(f"wrote {len(converted)} tensors to {args.out}")


if __name__ == "__main__":
    main()
