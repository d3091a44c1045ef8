"""Convert text corpora into record-file shards (`.hbrec`) that the data pipeline reads
(counterpart of the reference's convert_to_arrayrecord.py / hf_to_arrayrecord.py /
hf_parquet_to_arrayrecord.py, for this package's own container format).

    python scripts/tools/convert_to_records.py --output out/dclm --shard_size 100000 "raw/**/*.jsonl"
    python scripts/tools/convert_to_records.py --output out/math --source hf --split train EleutherAI/hendrycks_math
    python scripts/tools/convert_to_records.py --output out/fw --source parquet --shuffle "fineweb/*.parquet"

Every record is one JSON object (bytes). Shards are named `<name>-<split>-<i>-of-<n>.hbrec`.
"""

import argparse
import glob
import json
import os
import random

from halite_b200.data.sources import RecordFileWriter


def iter_jsonl(paths):
    for path in paths:
        with open(path, "rb") as f:
            for line in f:
                line = line.strip()
                if line:
                    yield line


def iter_text(paths, key="text"):
    for path in paths:
        with open(path, encoding="utf-8") as f:
            yield json.dumps({key: f.read()}).encode()


def iter_parquet(paths):
    import pyarrow.parquet as pq

    for path in paths:
        table = pq.ParquetFile(path)
        for batch in table.iter_batches(batch_size=1024):
            for row in batch.to_pylist():
                yield json.dumps(row, default=str).encode()


def iter_hf(dataset, name, split, trust_remote_code=False):
    import datasets

    ds = datasets.load_dataset(dataset, name, split=split, trust_remote_code=trust_remote_code)
    for row in ds:
        yield json.dumps(row, default=str).encode()


def write_shards(records, out_dir, stem, shard_size, n_shards=None):
    """Round-robin into `n_shards` files when given, else cut a new file every `shard_size`."""
    os.makedirs(out_dir, exist_ok=True)
    counts = {}
    if n_shards:
        names = [f"{stem}-{i + 1}-of-{n_shards}.hbrec" for i in range(n_shards)]
        writers = [RecordFileWriter(os.path.join(out_dir, n)) for n in names]
        for i, rec in enumerate(records):
            writers[i % n_shards].write(rec)
            counts[names[i % n_shards]] = counts.get(names[i % n_shards], 0) + 1
        for w in writers:
            w.close()
        return counts
    tmp, writer, n = [], None, 0
    for rec in records:
        if writer is None:
            tmp.append(os.path.join(out_dir, f"{stem}-part{len(tmp):05d}.tmp"))
            writer, n = RecordFileWriter(tmp[-1]), 0
        writer.write(rec)
        n += 1
        if n >= shard_size:
            writer.close()
            counts[tmp[-1]] = n
            writer = None
    if writer is not None:
        writer.close()
        counts[tmp[-1]] = n
    final = {}
    for i, path in enumerate(tmp):
        name = f"{stem}-{i + 1}-of-{len(tmp)}.hbrec"
        os.replace(path, os.path.join(out_dir, name))
        final[name] = counts[path]
    return final


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--output", required=True)
    ap.add_argument("--source", default="jsonl", choices=["jsonl", "text", "parquet", "hf"])
    ap.add_argument("--shard_size", type=int, default=1_000_000, help="records per shard")
    ap.add_argument("--n_shards", type=int, default=None)
    ap.add_argument("--split", default="train")
    ap.add_argument("--names", default=None, help="hf: comma list of configuration names")
    ap.add_argument("--shuffle", action="store_true", help="shuffle records in memory before writing")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--trust_remote_code", action="store_true")
    ap.add_argument("input")
    args = ap.parse_args(argv)

    spec = {}
    if args.source == "hf":
        for name in (args.names.split(",") if args.names else [None]):
            recs = iter_hf(args.input, name, args.split, args.trust_remote_code)
            stem = f"{name or 'data'}-{args.split}"
            spec.update(write_shards(recs, args.output, stem, args.shard_size, args.n_shards))
    else:
        paths = sorted(glob.glob(args.input, recursive=True))
        if not paths:
            raise SystemExit(f"no input files match {args.input}")
        recs = {"jsonl": iter_jsonl, "text": iter_text, "parquet": iter_parquet}[args.source](paths)
        if args.shuffle:
            recs = list(recs)
            random.Random(args.seed).shuffle(recs)
        spec.update(write_shards(recs, args.output, f"data-{args.split}", args.shard_size, args.n_shards))
    print(json.dumps({os.path.basename(os.path.normpath(args.output)): spec}, indent=2))
    return spec


if __name__ == "__main__":
    main()
