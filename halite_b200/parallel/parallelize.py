"""`parallelize(model, mesh, parallel_dims, ...)`: apply tensor parallelism, activation
checkpointing and data-parallel sharding to a model, in that order (reference:
transformers/parallelize.py:12-127). The `compile` knob of the reference is accepted and
ignored: the hot path here is hand-written kernels, not a tracing compiler. Every other knob
does what its name says or raises.
"""

from __future__ import annotations


from halite_b200.parallel.fsdp import apply_ddp, apply_fsdp
from halite_b200.utils import get_torch_dtype


def parallelize(model, mesh=None, parallel_dims=None, param_dtype="bfloat16", reduce_dtype="float32",
                tensor_parallel_config=None, activation_checkpointing=False,
                activation_checkpointing_config=None, compile=False, compile_config=None,
                reshard_after_forward=False, data_parallel="fsdp", force_fsdp=False, device=None,
                loss_parallel=False, block_iterator=None, fused_all_gather=None,
                fused_reduce_scatter=None, **unknown):
    if unknown:
        raise TypeError(f"parallelize() got options it does not implement: {sorted(unknown)}")
    pd = parallel_dims if parallel_dims is not None else mesh
    param_dtype = get_torch_dtype(param_dtype)
    reduce_dtype = get_torch_dtype(reduce_dtype)

    if pd is not None and pd.tp_enabled:
        from halite_b200.parallel.tensor_parallel import apply_tp

        apply_tp(model, pd, loss_parallel=loss_parallel, **(tensor_parallel_config or {}))

    if activation_checkpointing:
        cfg = dict(activation_checkpointing_config or {})
        mode = cfg.get("mode", "full")
        if mode == "full":
            model.gradient_checkpointing_enable(int(cfg.get("every", 1)))
        elif mode == "selective":
            # "op": keep the attention half, recompute the feed-forward half of every block;
            # an integer k: recompute every k-th block, keep the others' activations
            selective = str(cfg.get("selective", "1"))
            if selective == "op":
                model.gradient_checkpointing_enable(0, ops=True)
            else:
                model.gradient_checkpointing_enable(1, stride=int(selective))
        else:
            raise ValueError(f"activation checkpointing mode must be 'full' or 'selective', got {mode!r}")

    if data_parallel == "ddp" or (pd is not None and not pd.dp_shard_enabled and pd.dp_replicate_enabled
                                  and not force_fsdp):
        return apply_ddp(model, pd, param_dtype=param_dtype, reduce_dtype=reduce_dtype, device=device)
    return apply_fsdp(model, pd, param_dtype=param_dtype, reduce_dtype=reduce_dtype,
                      reshard_after_forward=reshard_after_forward, device=device, block_iterator=block_iterator,
                      fused_all_gather=fused_all_gather, fused_reduce_scatter=fused_reduce_scatter)
