from .parallel_dims import ParallelDims
from .fsdp import apply_ddp, apply_fsdp
from .parallelize import parallelize
