"""Data pipeline: record files, ratio mixing with deterministic shuffling, sequence packing, and
the break / state_dict / resume equality check (pattern of the reference's
test/stateful_dataloader.py)."""

import json
import os

import pytest
import torch

from halite_b200.data import DataLoader, WeightedIterableDataset, build_dataset_from_spec
from halite_b200.data import preprocess as P
from halite_b200.data.index_shuffle import index_shuffle
from halite_b200.data.record import Record
from halite_b200.data.sources import RecordFile, RecordFileWriter
from halite_b200.data.tokenizers import ByteTokenizer


def make_spec(tmp_path, sizes=(("a", 200), ("b", 50))):
    shards, ratios = {}, {}
    for name, n in sizes:
        d = tmp_path / name
        d.mkdir()
        with RecordFileWriter(str(d / "s0.hbrec")) as w:
            for i in range(n):
                w.write(json.dumps({"text": f"{name}-{i} " + "x" * (i % 17), "idx": i}))
        shards[name] = {"s0.hbrec": n}
        ratios[name] = 0.8 if name == "a" else 0.2
    return {"root": str(tmp_path), "ratios": ratios, "shards": shards}


def test_record_file_roundtrip(tmp_path):
    p = str(tmp_path / "x.hbrec")
    with RecordFileWriter(p) as w:
        for i in range(100):
            w.write(b"r%d" % i * (i % 5 + 1))
    r = RecordFile(p)
    assert len(r) == 100 and r[0] == b"r0" and r[7] == b"r7r7r7" and r[99] == b"r99" * 5
    with pytest.raises(IndexError):
        r[100]


def test_index_shuffle_is_a_permutation():
    for n in (1, 2, 17, 1000, 4097):
        seen = sorted(index_shuffle(i, n - 1, 42) for i in range(n))
        assert seen == list(range(n))
    assert [index_shuffle(i, 999, 1) for i in range(10)] != [index_shuffle(i, 999, 2) for i in range(10)]


def test_split_and_ratio_mixing(tmp_path):
    spec = make_spec(tmp_path)
    # train reads the tail share of each shard, eval the head share
    train, ratios, names = build_dataset_from_spec(spec, "train", 0.9)
    evals, _, _ = build_dataset_from_spec(spec, "eval", 0.1)
    assert [len(s) for s in train] == [180, 45] and [len(s) for s in evals] == [20, 5]
    assert json.loads(train[0][0])["idx"] == 20 and json.loads(train[0][179])["idx"] == 199
    assert json.loads(evals[0][0])["idx"] == 0 and json.loads(evals[0][19])["idx"] == 19
    assert len(build_dataset_from_spec(spec, "train", 0)[0][0]) == 200
    ds = WeightedIterableDataset(train, ratios, names, operations=[P.ParseFeatures()], seed=3)
    counts = {"a": 0, "b": 0}
    seen = set()
    for rec in ds:
        counts[rec["_meta_"]["dataset_name"]] += 1
        seen.add((rec["_meta_"]["dataset_name"], rec["idx"]))
    assert counts["a"] / counts["b"] == pytest.approx(4.0, rel=0.05)
    assert len(seen) == counts["a"] + counts["b"]           # no repeats below one epoch
    # two ranks see disjoint halves
    halves = [set(), set()]
    for r in range(2):
        d = WeightedIterableDataset(train, ratios, names, operations=[P.ParseFeatures()], seed=3,
                                    num_replicas=2, rank=r)
        halves[r] = {(x["_meta_"]["dataset_name"], x["idx"]) for x in d}
    assert not (halves[0] & halves[1])


def build_loader(spec, workers, rank=0):
    train, ratios, names = build_dataset_from_spec(spec, "train", 0)
    ops = [P.ParseFeatures(), P.Tokenize(ByteTokenizer(), bos=True, eos=True), P.SequencePacking(33),
           P.AutoregressiveSample()]
    ds = WeightedIterableDataset(train, ratios, names, operations=ops, seed=7, num_replicas=1, rank=rank)
    return DataLoader(ds, batch_size=4, rank=rank, num_workers=workers, collate_fn=P.Collator(keys=("input", "target")))


@pytest.mark.parametrize("workers", [0, 2])
def test_break_and_resume_reproduces_the_stream(tmp_path, workers):
    spec = make_spec(tmp_path)
    full = [b["input"] for b in build_loader(spec, workers)]
    assert len(full) > 12 and full[0].shape == (4, 32)
    loader = build_loader(spec, workers)
    head, state = [], None
    for i, b in enumerate(loader):
        head.append(b["input"])
        if i == 5:
            state = loader.state_dict()
            break
    resumed = build_loader(spec, workers)
    resumed.load_state_dict(state)
    tail = [b["input"] for b in resumed]
    got = head + tail
    assert len(got) == len(full)
    for a, b in zip(got, full):
        assert torch.equal(a, b)


def test_packing_meta_and_collator():
    recs = [Record(text=list(range(i * 10, i * 10 + 7)), _meta_={"dataset_id": 0, "sample_id": i}) for i in range(5)]
    packed = list(P.AutoregressiveSample()(P.SequencePacking(10, rewind=0)(iter(recs))))
    assert len(packed) == 3 and packed[0]["text"] == [0, 1, 2, 3, 4, 5, 6, 10, 11, 12]
    assert packed[0]["_meta_"]["sample_ids"] == [0, 1] and packed[1]["_meta_"]["sample_ids"] == [1, 2]
    batch = P.Collator(keys=("input", "target"))(packed)
    assert batch["input"].shape == (3, 9) and torch.equal(batch["input"][:, 1:], batch["target"][:, :-1])
    assert len(batch["_meta_"]["samples_meta"]) == 3
    rows = batch.unbind(["input"])
    assert len(rows) == 3 and rows[1]["input"].shape == (9,)


def test_sft_sample_masks_prompt_and_packing_pads_rows():
    from halite_b200.projects.sft.preprocess import (SFTSample, SFTSequencePacking, collate_offsets,
                                                     length_to_offsets)

    tok = ByteTokenizer()
    sample = SFTSample("q", "a", tok, prompt_tokenizer_kwargs={"bos": True}, response_tokenizer_kwargs={"eos": True})
    rec = sample.process(Record(q="ab", a="xyz", _meta_={"dataset_id": 0, "sample_id": 5}))
    assert rec["input"].tolist() == [tok.bos_id, 97, 98, 120, 121, 122, tok.eos_id]
    # prompt positions ignored; position of the last prompt token predicts the first response token
    assert rec["target"].tolist() == [-100, -100, 120, 121, 122, tok.eos_id, -100]

    def recs(lengths):
        for i, n in enumerate(lengths):
            yield Record(input=torch.arange(n) + 100 * i, target=torch.arange(n) + 100 * i + 1,
                         _meta_={"dataset_id": 0, "sample_id": i})

    pack = SFTSequencePacking(8, use_position_ids=True, use_document_offsets=True)
    rows = list(pack(recs([3, 4, 5, 8, 11, 2])))
    assert all(len(r["input"]) == 8 and len(r["target"]) == 8 for r in rows)
    assert rows[0]["input"].tolist() == [0, 1, 2, 100, 101, 102, 103, 0]          # 3 + 4, one pad
    assert rows[0]["target"].tolist()[-1] == -100
    assert rows[0]["document_offsets"].tolist() == [0, 3, 7, 8]
    assert rows[0]["position_ids"].tolist() == [0, 1, 2, 0, 1, 2, 3, 0]
    assert rows[0]["_meta_"]["sample_ids"] == [0, 1]
    assert rows[1]["input"].tolist()[:5] == [200, 201, 202, 203, 204] and rows[2]["_meta_"]["sample_ids"] == [3]
    assert rows[3]["input"].tolist() == list(range(400, 408))                      # long sample truncated
    assert rows[4]["_meta_"]["sample_ids"] == [5] and len(rows) == 5
    keep = SFTSequencePacking(8, use_rest_of_long_sequence=True)
    rows2 = list(keep(recs([11])))
    assert [r["input"].tolist()[:3] for r in rows2] == [[0, 1, 2], [8, 9, 10]]
    assert length_to_offsets([2, 4, 3]).tolist() == [0, 2, 6, 9]
    assert collate_offsets([torch.tensor([0, 3, 8]), torch.tensor([0, 8])], 4).tolist() == [[0, 3, 8, 8], [0, 8, 8, 8]]
    # state round trip in the middle of a stream
    a = SFTSequencePacking(8)
    it = a(recs([3, 4, 5, 2, 6]))
    first = next(it)
    b = SFTSequencePacking(8)
    b.load_state_dict(a.state_dict())
    assert len(b.state_dict()["input_ids"]) == len(a._pending) and first["input"].shape == (8,)


def test_tools_convert_gather_and_sanity(tmp_path, capsys):
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "scripts/tools"))
    import convert_to_records
    import gather_dataset
    import sample_sanity

    raw = tmp_path / "raw"
    raw.mkdir()
    for part in range(2):
        with open(raw / f"p{part}.jsonl", "w") as f:
            for i in range(25):
                f.write(json.dumps({"text": f"doc {part}-{i} " + "lorem ipsum " * 8}) + "\n")
    out = tmp_path / "corpus" / "web"
    spec = convert_to_records.main(["--output", str(out), "--shard_size", "20", str(raw / "*.jsonl")])
    assert sorted(spec.values()) == [10, 20, 20] and all(n.endswith("-of-3.hbrec") for n in spec)
    rr = convert_to_records.main(["--output", str(tmp_path / "corpus" / "rr"), "--n_shards", "2", "--shuffle",
                                  str(raw / "*.jsonl")])
    assert sorted(rr.values()) == [25, 25]
    gathered = gather_dataset.main(["--ext", "hbrec", str(tmp_path / "corpus")])
    assert set(gathered["shards"]) == {"web", "rr"} and gathered["ratios"]["web"] == pytest.approx(0.5)
    assert gathered["shards"]["web"] == spec
    conf = tmp_path / "configs" / "exp.py"
    conf.parent.mkdir()
    conf.write_text(f'''
from halite_b200.conf import field
from halite_b200.data import preprocess
from halite_b200.data.tokenizers import ByteTokenizer
conf = field()
conf.model = field(tokenizer=ByteTokenizer())
conf.data = field(train={json.dumps(gathered)}, train_ratio=1.0,
    preprocess=[preprocess.ParseFeatures(), preprocess.Tokenize(ByteTokenizer(), bos=True, eos=True),
                preprocess.SequencePacking(33), preprocess.AutoregressiveSample()],
    collate_fn=preprocess.Collator(keys=("input", "target")))
''')
    dumped = sample_sanity.main(["--conf", str(conf), "--n_batch", "2", "--output", str(tmp_path / "dump.json")])
    assert len(dumped) == 2 and dumped[0]["input"]["shape"] == [2, 32] and "doc" in dumped[0]["input"]["text"][0] + dumped[1]["input"]["text"][0]
    assert (tmp_path / "dump.json").exists()
