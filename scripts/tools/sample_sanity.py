"""Print a few batches exactly as the trainer would see them (datasets, preprocessing, collate),
decoded back to text when the config has a tokenizer (counterpart of the reference's
scripts/tools/sample_sanity.py).

    python scripts/tools/sample_sanity.py --conf configs/lm/dense_662m.py --n_batch 2
"""

import argparse
import json

import torch

from halite_b200.conf import instantiate, load_config
from halite_b200.data.dataloader import DataLoader
from halite_b200.data.dataset import WeightedIterableDataset, build_dataset_from_spec


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--conf", required=True)
    ap.add_argument("--conf_name", default=None)
    ap.add_argument("--n_batch", type=int, default=1)
    ap.add_argument("--batch_size", type=int, default=2)
    ap.add_argument("--output", default=None)
    ap.add_argument("opts", nargs="*")
    args = ap.parse_args(argv)

    conf = load_config(args.conf, config_name=args.conf_name, overrides=args.opts)
    data = conf["data"]
    ops = [instantiate(op) for op in (data.get("preprocess") or [])]
    collate = instantiate(data["collate_fn"]) if data.get("collate_fn") is not None else None
    sources, ratios, names = build_dataset_from_spec(data["train"], "train", data.get("train_ratio", 1.0))
    ds = WeightedIterableDataset(sources, ratios, names, operations=ops)
    print(ds.summary())
    tokenizer = None
    model = conf.get("model")
    if model is not None and model.get("tokenizer") is not None:
        tokenizer = instantiate(model["tokenizer"])
    dumped = []
    for i, batch in enumerate(DataLoader(ds, batch_size=args.batch_size, collate_fn=collate, num_workers=0)):
        if i >= args.n_batch:
            break
        entry = {}
        for key, val in batch.items():
            if isinstance(val, torch.Tensor):
                entry[key] = {"shape": list(val.shape), "dtype": str(val.dtype), "head": val.flatten()[:16].tolist()}
                if tokenizer is not None and val.dtype == torch.int64 and val.dim() == 2 and key in ("input", "target"):
                    entry[key]["text"] = [tokenizer.decode([t for t in row.tolist() if t >= 0]) for row in val[:2]]
            elif key == "_meta_":
                entry[key] = {k: v for k, v in val.items() if k != "samples_meta"}
            else:
                entry[key] = val if isinstance(val, (str, int, float, list)) else str(val)
        dumped.append(entry)
        print(f"--- batch {i}")
        print(json.dumps(entry, indent=2, default=str)[:4000])
    if args.output:
        with open(args.output, "w") as f:
            json.dump(dumped, f, indent=2, default=str)
    return dumped


if __name__ == "__main__":
    main()
