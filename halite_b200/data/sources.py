"""Record sources: random-access containers of byte payloads.

`RecordFile` is this package's own container (`.hbrec`): a 32-byte header, the payloads back to
back, and a trailing table of uint64 offsets; reads go through one memory map, so a worker
touches only the pages it needs. Third-party containers the reference reads (ArrayRecord,
FFRecord, Bagz; data/dataset.py:31-149) are supported when their libraries are importable.
"""

from __future__ import annotations

import bisect
import dataclasses
import itertools
import mmap
import struct

_MAGIC = b"HBREC001"


@dataclasses.dataclass
class FileInstruction:
    filename: str
    skip: int = 0
    take: int | None = None
    examples_in_shard: int | None = None


class RecordFileWriter:
    def __init__(self, path):
        self.f = open(path, "wb")
        self.f.write(_MAGIC + struct.pack("<QQQ", 0, 0, 0))
        self.offsets = [32]

    def write(self, payload: bytes):
        if isinstance(payload, str):
            payload = payload.encode("utf-8")
        self.f.write(payload)
        self.offsets.append(self.offsets[-1] + len(payload))

    def close(self):
        table_at = self.offsets[-1]
        self.f.write(struct.pack(f"<{len(self.offsets)}Q", *self.offsets))
        self.f.seek(8)
        self.f.write(struct.pack("<QQQ", len(self.offsets) - 1, table_at, 0))
        self.f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class RecordFile:
    def __init__(self, path):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if self._mm[:8] != _MAGIC:
            raise ValueError(f"{path} is not a record file")
        self.n, self.table_at, _ = struct.unpack_from("<QQQ", self._mm, 8)

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        if not 0 <= i < self.n:
            raise IndexError(i)
        a, b = struct.unpack_from("<QQ", self._mm, self.table_at + 8 * i)
        return bytes(self._mm[a:b])

    def __getstate__(self):
        return {"path": self.path}

    def __setstate__(self, state):
        self.__init__(state["path"])


class ShardedSource:
    """Several shard files seen as one sequence, each restricted to [skip, skip + take)."""

    def __init__(self, file_instructions):
        self.readers, counts = [], []
        for ins in file_instructions:
            reader = self._open(ins.filename)
            self.readers.append(reader)
            counts.append(ins.take if ins.take is not None else len(reader) - ins.skip)
        self.skips = [ins.skip for ins in file_instructions]
        self.cumsum = list(itertools.accumulate(counts))
        self.length = self.cumsum[-1] if counts else 0

    def _open(self, filename):
        return RecordFile(filename)

    def _read(self, reader, index):
        return reader[index]

    def __len__(self):
        return self.length

    def __getitem__(self, index):
        if not 0 <= index < self.length:
            raise IndexError(index)
        shard = bisect.bisect_right(self.cumsum, index)
        local = index - (self.cumsum[shard - 1] if shard else 0)
        return self._read(self.readers[shard], local + self.skips[shard])


class RecordFileDataSource(ShardedSource):
    pass


class FFRecordDataSource(ShardedSource):
    def _open(self, filename):
        from ffrecord import FileReader

        return FileReader(filename, check_data=False)

    def _read(self, reader, index):
        return reader.read_one(index).tobytes()


class BagzDataSource(ShardedSource):
    def _open(self, filename):
        import bagz

        return bagz.Reader(filename)


class JsonlDataSource:
    """Lines of a .jsonl / .txt file as payloads (line offsets indexed once at open)."""

    def __init__(self, file_instructions):
        self.files = []
        counts = []
        for ins in file_instructions:
            offsets = [0]
            with open(ins.filename, "rb") as f:
                for line in f:
                    offsets.append(offsets[-1] + len(line))
            n = len(offsets) - 1
            take = ins.take if ins.take is not None else n - ins.skip
            self.files.append((ins.filename, offsets, ins.skip))
            counts.append(take)
        self.cumsum = list(itertools.accumulate(counts))
        self.length = self.cumsum[-1] if counts else 0
        self._handles = {}

    def __len__(self):
        return self.length

    def __getitem__(self, index):
        shard = bisect.bisect_right(self.cumsum, index)
        local = index - (self.cumsum[shard - 1] if shard else 0)
        name, offsets, skip = self.files[shard]
        f = self._handles.get(name)
        if f is None:
            f = self._handles[name] = open(name, "rb")
        i = local + skip
        f.seek(offsets[i])
        return f.read(offsets[i + 1] - offsets[i]).rstrip(b"\n")

    def __getstate__(self):
        d = dict(self.__dict__)
        d["_handles"] = {}
        return d


def open_source(instructions):
    name = instructions[0].filename
    if name.endswith(".hbrec"):
        return RecordFileDataSource(instructions)
    if name.endswith(".ffr"):
        return FFRecordDataSource(instructions)
    if name.endswith((".bag", ".bagz")):
        return BagzDataSource(instructions)
    if name.endswith((".jsonl", ".txt")):
        return JsonlDataSource(instructions)
    if name.endswith(".arrayrecord"):
        import array_record.python.array_record_data_source as array_record

        return array_record.ArrayRecordDataSource(instructions)
    raise ValueError(f"unsupported record file extension: {name}")
