"""Engine B: a manager that schedules several forwards ahead of the device and a model worker
that executes mixed prefill + decode batches on the paged kernels, optionally in a separate
process (reference: transformers/tokainfer/*, the Tokasaurus-style engine)."""

from .inference_engine import InferenceEngine
from .types import ServerConfig

__all__ = ["InferenceEngine", "ServerConfig"]
