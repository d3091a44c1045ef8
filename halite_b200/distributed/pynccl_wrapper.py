"""ctypes binding of `libnccl.so.2` (reference: distributed/pynccl_wrapper.py:11-470): lets a
process create NCCL communicators of its own, outside `torch.distributed`'s global group. Used
for weight broadcast between a trainer job and separately launched generator processes."""

from __future__ import annotations

import ctypes
import glob
import os
from dataclasses import dataclass

import torch

ncclResult_t = ctypes.c_int
ncclComm_t = ctypes.c_void_p
cudaStream_t = ctypes.c_void_p
buffer_t = ctypes.c_void_p


class ncclUniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


class ncclDataTypeEnum:
    ncclInt8, ncclUint8, ncclInt32, ncclUint32, ncclInt64, ncclUint64 = 0, 1, 2, 3, 4, 5
    ncclFloat16, ncclFloat32, ncclFloat64, ncclBfloat16 = 6, 7, 8, 9
    _MAP = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
            torch.float64: 8, torch.bfloat16: 9}

    @classmethod
    def from_torch(cls, dtype: torch.dtype) -> int:
        try:
            return cls._MAP[dtype]
        except KeyError:
            raise ValueError(f"unsupported dtype for NCCL: {dtype}") from None


class ncclRedOpTypeEnum:
    ncclSum, ncclProd, ncclMax, ncclMin, ncclAvg = 0, 1, 2, 3, 4

    @classmethod
    def from_torch(cls, op) -> int:
        from torch.distributed import ReduceOp

        table = {ReduceOp.SUM: 0, ReduceOp.PRODUCT: 1, ReduceOp.MAX: 2, ReduceOp.MIN: 3, ReduceOp.AVG: 4}
        try:
            return table[op]
        except KeyError:
            raise ValueError(f"unsupported reduce op for NCCL: {op}") from None


def find_nccl_library() -> str:
    """`HALITE_NCCL_SO_PATH` if set, else the libnccl bundled with torch, else the system one."""
    env = os.environ.get("HALITE_NCCL_SO_PATH")
    if env:
        return env
    site = os.path.dirname(os.path.dirname(torch.__file__))
    for pattern in ("nvidia/nccl/lib/libnccl.so.2", "torch/lib/libnccl.so*"):
        hits = sorted(glob.glob(os.path.join(site, pattern)))
        if hits:
            return hits[0]
    return "libnccl.so.2"


@dataclass
class Function:
    name: str
    restype: object
    argtypes: list


class NCCLLibrary:
    functions = [
        Function("ncclGetErrorString", ctypes.c_char_p, [ncclResult_t]),
        Function("ncclGetVersion", ncclResult_t, [ctypes.POINTER(ctypes.c_int)]),
        Function("ncclGetUniqueId", ncclResult_t, [ctypes.POINTER(ncclUniqueId)]),
        Function("ncclCommInitRank", ncclResult_t, [ctypes.POINTER(ncclComm_t), ctypes.c_int, ncclUniqueId, ctypes.c_int]),
        Function("ncclAllReduce", ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                                 ncclComm_t, cudaStream_t]),
        Function("ncclReduce", ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_int, ncclComm_t, cudaStream_t]),
        Function("ncclAllGather", ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ncclComm_t,
                                                 cudaStream_t]),
        Function("ncclReduceScatter", ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                                     ncclComm_t, cudaStream_t]),
        Function("ncclSend", ncclResult_t, [buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t,
                                            cudaStream_t]),
        Function("ncclRecv", ncclResult_t, [buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t,
                                            cudaStream_t]),
        Function("ncclBroadcast", ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                                 ncclComm_t, cudaStream_t]),
        Function("ncclCommDestroy", ncclResult_t, [ncclComm_t]),
        Function("ncclGroupStart", ncclResult_t, []),
        Function("ncclGroupEnd", ncclResult_t, []),
    ]
    _cache: dict = {}

    def __init__(self, so_file: str | None = None):
        so_file = so_file or find_nccl_library()
        if so_file not in NCCLLibrary._cache:
            lib = ctypes.CDLL(so_file)
            funcs = {}
            for f in self.functions:
                fn = getattr(lib, f.name)
                fn.restype, fn.argtypes = f.restype, f.argtypes
                funcs[f.name] = fn
            NCCLLibrary._cache[so_file] = (lib, funcs)
        self.lib, self._funcs = NCCLLibrary._cache[so_file]
        self.so_file = so_file

    def check(self, result):
        if result != 0:
            raise RuntimeError(f"NCCL error: {self._funcs['ncclGetErrorString'](result).decode()}")

    def ncclGetVersion(self) -> str:
        v = ctypes.c_int()
        self.check(self._funcs["ncclGetVersion"](ctypes.byref(v)))
        s = str(v.value)
        return f"{int(s[:-4] or 0)}.{int(s[-4:-2])}.{int(s[-2:])}" if v.value >= 10000 else s

    def ncclGetUniqueId(self) -> ncclUniqueId:
        uid = ncclUniqueId()
        self.check(self._funcs["ncclGetUniqueId"](ctypes.byref(uid)))
        return uid

    def unique_id_from_bytes(self, data: bytes) -> ncclUniqueId:
        uid = ncclUniqueId()
        ctypes.memmove(ctypes.addressof(uid.internal), data, 128)
        return uid

    def ncclCommInitRank(self, world_size, unique_id, rank) -> ncclComm_t:
        comm = ncclComm_t()
        self.check(self._funcs["ncclCommInitRank"](ctypes.byref(comm), world_size, unique_id, rank))
        return comm

    def __getattr__(self, name):
        funcs = self.__dict__.get("_funcs", {})
        if name in funcs:
            fn = funcs[name]
            return lambda *a: self.check(fn(*a))
        raise AttributeError(name)
