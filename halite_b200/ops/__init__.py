"""Op front-ends. Every op has two implementations and nothing else:

* `sm100`: the hand-written CUDA kernels in `halite_b200/csrc` (bf16 tensors on a CUDA device);
* `reference`: plain PyTorch in fp32, used on CPU and as the oracle in tests.

On a GPU a bf16 tensor runs the sm_100a kernel, and a missing extension raises. The one
exception is a matrix product with a dimension that is not a multiple of 8 (TMA needs 16-byte
rows): it goes to the library GEMM and `ops/linear.py` logs that once per shape. Set
`HALITE_B200_FORCE_REFERENCE=1` to run the PyTorch path on purpose (tests do, to compare the two).
"""

from __future__ import annotations

import os

import torch

_ext = None
_status = {}


def ext():
    """The compiled extension module (builds it in-tree on first use when stale)."""
    global _ext
    if _ext is None:
        from halite_b200.csrc import build

        _ext = build.load()
    return _ext


def force_reference() -> bool:
    return os.environ.get("HALITE_B200_FORCE_REFERENCE", "0") == "1"


def use_sm100(*tensors) -> bool:
    """True when the tensors live on a CUDA device in bf16 and the kernels should run."""
    if force_reference():
        return False
    t = tensors[0]
    if not t.is_cuda:
        return False
    return t.dtype == torch.bfloat16


def status_word(device) -> torch.Tensor:
    """Per-device int32 that kernels set when a bounded wait gives up (0 = healthy)."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device=None):
    """Read the status word (synchronises) and raise if any kernel recorded a timeout."""
    if not _status:
        return
    for key, t in _status.items():
        code = int(t.item())
        if code != 0:
            t.zero_()
            what = "read a page id outside the KV pool" if code == 8 else "gave up a bounded wait"
            raise RuntimeError(f"halite_b200 kernel on cuda:{key} {what} (code {code})")


from .linear import linear, gemm, matmul_nt  # noqa: E402
from .norm import rms_norm, rms_norm_reference  # noqa: E402
from .rope import apply_rope, rope_tables, apply_rope_reference  # noqa: E402
from .activation import gated_act, swiglu, geglu_tanh  # noqa: E402
from .loss import (cross_entropy_rows, cross_entropy_rows_reference, fused_linear_cross_entropy,  # noqa: E402
                   logprob_entropy)
from .optim import fused_adamw_step, grad_sumsq  # noqa: E402
from .rl import gae, gae_reference  # noqa: E402
