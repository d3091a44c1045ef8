"""Small shared helpers (reference: utils/__init__.py:23-39)."""

from __future__ import annotations

import torch

_DTYPES = {
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float64": torch.float64, "fp64": torch.float64, "double": torch.float64,
    "int32": torch.int32, "int64": torch.int64, "int8": torch.int8, "uint8": torch.uint8,
    "bool": torch.bool,
}


def get_torch_dtype(dtype):
    """'bfloat16' / 'torch.bfloat16' / torch.bfloat16 -> torch.bfloat16; None passes through."""
    if dtype is None or isinstance(dtype, torch.dtype):
        return dtype
    name = str(dtype).replace("torch.", "").lower()
    if name not in _DTYPES:
        raise ValueError(f"unknown dtype {dtype!r}")
    return _DTYPES[name]


def dtype_name(dtype) -> str:
    return str(dtype).replace("torch.", "")
