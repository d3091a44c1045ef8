"""Scan a directory of record files and print the `{root, ratios, shards}` specification the
training configs consume (counterpart of the reference's scripts/tools/gather_dataset.py).
Ratios default to each dataset's share of the total record count.

    python scripts/tools/gather_dataset.py --ext hbrec --depth 1 --output spec.json /data/corpus
"""

import argparse
import json
import os
from glob import glob

from halite_b200.data.sources import FileInstruction, open_source


def record_count(path):
    return len(open_source([FileInstruction(path, 0, None, None)]))


def gather(path, ext="hbrec", depth=0):
    files = sorted(glob(os.path.join(path, f"**/*.{ext}"), recursive=True))
    shards = {}
    for file in files:
        folder = os.path.dirname(file)
        rel = os.path.relpath(folder, path)
        if depth:
            rel = os.sep.join(os.path.normpath(rel).split(os.sep)[:depth])
            folder = os.path.join(path, rel)
        shards.setdefault(rel, {})[os.path.relpath(file, folder)] = record_count(file)
    totals = {name: sum(s.values()) for name, s in shards.items()}
    grand = sum(totals.values()) or 1
    return {"root": path, "ratios": {n: t / grand for n, t in totals.items()}, "shards": shards}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--depth", type=int, default=0, help="directory levels that name a dataset (0 = full path)")
    ap.add_argument("--output", default=None)
    ap.add_argument("--ext", default="hbrec")
    ap.add_argument("path")
    args = ap.parse_args(argv)
    spec = gather(args.path, args.ext, args.depth)
    text = json.dumps(spec, indent=4)
    print(text)
    if args.output:
        with open(args.output, "w") as f:
            f.write(text)
    return spec


if __name__ == "__main__":
    main()
