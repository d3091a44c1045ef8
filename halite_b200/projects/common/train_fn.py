"""Step functions.

`basic_train_step(data, model, criterion) -> (loss, loss_dict)` is the pluggable forward + loss
that experiment configurations name as `train_step_fn` / `eval_step_fn`
(reference: projects/common/train_fn.py:18-34).

`optimization_step(...)` is a whole update (the hot loop of the reference's scripts/lm.py:56-143):
forward, loss, backward, gradient clipping, scheduler and optimizer step. It returns device
tensors only; the caller decides when to read them."""

from __future__ import annotations

from collections.abc import Mapping


from halite_b200.optim.sharded_adamw import clip_grad_norm_


def get_fields(record, fields):
    """{name: value} for one field name or several, from a mapping or an object."""
    names = [fields] if isinstance(fields, str) else list(fields)
    if isinstance(record, Mapping):
        return {n: record[n] for n in names}
    return {n: getattr(record, n) for n in names}


_MODEL_INPUTS = (("input", "input_ids"), ("position_ids", "position_ids"),
                 ("document_offsets", "document_offsets"))


def basic_train_step(data, model, criterion):
    kwargs = {dst: data[src] for src, dst in _MODEL_INPUTS if src in data}
    out = model(**kwargs)
    return criterion(out.logits, data["target"])


def optimization_step(model, batch, optimizer, scheduler=None, criterion=None, clip_grad_norm=None,
                     calc_loss_in_model=False, grad_accum_steps=1, input_key="input", target_key="target",
                     aux_loss_weight=1.0):
    """`batch` maps `input_key` / `target_key` to [B, S] token tensors (already on the device).
    With `calc_loss_in_model` the head computes the loss (fused linear + cross entropy);
    otherwise `criterion(logits, target)` does."""
    inputs, targets = batch[input_key], batch[target_key]
    extra = {k: v for k, v in batch.items() if k in ("position_ids", "document_offsets", "attention_mask")}
    if calc_loss_in_model:
        out = model(inputs, target=targets, **extra)
        loss, loss_dict = out.loss, dict(out.loss_dict or {})
    else:
        out = model(inputs, **extra)
        loss, loss_dict = criterion(out.logits, targets)
        loss_dict = dict(loss_dict)
    for aux in out.aux_outputs or []:
        if isinstance(aux, dict):
            for k, v in aux.items():
                if k.endswith("loss"):
                    loss = loss + aux_loss_weight * v
                    loss_dict[k] = loss_dict.get(k, 0) + v.detach()
    if grad_accum_steps > 1:
        loss = loss / grad_accum_steps
    loss.backward()
    fsdp = getattr(model, "_hb_fsdp", None)
    if fsdp is not None:
        fsdp.finish_backward()
    grad_norm = None
    if clip_grad_norm:
        grad_norm = clip_grad_norm_(model, clip_grad_norm, optimizer)
    if scheduler is not None:
        scheduler.step()
    optimizer.step()
    optimizer.zero_grad(set_to_none=True)
    return {"loss": loss.detach(), "grad_norm": grad_norm, "loss_dict": loss_dict}
