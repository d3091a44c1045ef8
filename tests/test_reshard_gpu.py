"""The one-launch trainer -> engine reshard kernel on one GPU: flat buffers cut into 1, 3 and 8
shards that live in separate allocations (standing in for the ranks' memories; the kernel only
sees base pointers), uneven padding, whole tensors, row slices, column slices and separately cut
blocks of packed matrices, against gather-then-slice with torch."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _segments(flat_off, shape, es, plan, tp_rank, tp_size):
    numel = 1
    for s in shape:
        numel *= s
    rows_full = shape[0] if len(shape) > 1 else 1
    cols = numel // rows_full
    if plan is None:
        return [(flat_off, 1, numel, numel)]
    if plan[1] == 0:
        parts = plan[2] if plan[0] == "shard_parts" else [rows_full]
        out, at = [], 0
        for n in parts:
            step = n // tp_size
            out.append((flat_off + (at + tp_rank * step) * cols, 1, step * cols, step * cols))
            at += n
        return out
    step = cols // tp_size
    return [(flat_off + tp_rank * step, rows_full, step, cols)]


@pytest.mark.parametrize("n_shards", [1, 3, 8])
@pytest.mark.parametrize("tp_size", [1, 2, 4])
def test_reshard_kernel_matches_gather_then_slice(n_shards, tp_size):
    import halite_b200.ops as ops

    C = ops.ext()
    g = torch.Generator(device="cuda").manual_seed(n_shards * 10 + tp_size)
    tensors = {"qkv": ((5120, 256), ("shard_parts", 0, [3072, 1024, 1024])), "out": ((256, 3072), ("shard", 1)),
               "up": ((1024, 256), ("shard", 0)), "norm": ((256,), None), "embed": ((1000, 256), None)}
    es = 2
    entries, off = {}, 0
    for name, (shape, _) in tensors.items():
        off = (off + 7) // 8 * 8
        n = 1
        for s in shape:
            n *= s
        entries[name] = off
        off += n
    chunk = n_shards * 128
    padded = (off + chunk - 1) // chunk * chunk + (chunk if n_shards == 3 else 0)      # uneven tail padding
    flat = torch.randn(padded, device="cuda", generator=g).bfloat16()
    shard = padded // n_shards
    shards = [flat[r * shard:(r + 1) * shard].clone() for r in range(n_shards)]        # separate allocations
    for tp_rank in range(tp_size):
        rows, dsts, wants = [], {}, {}
        for name, (shape, plan) in tensors.items():
            plan_here = plan if tp_size > 1 else None
            segs = _segments(entries[name], shape, es, plan_here, tp_rank, tp_size)
            numel = sum(r * n for _, r, n, _ in segs)
            dst = torch.full((numel,), float("nan"), device="cuda", dtype=torch.bfloat16)
            dsts[name] = dst
            n_all = 1
            for s in shape:
                n_all *= s
            full = flat[entries[name]:entries[name] + n_all].view(shape)
            if plan_here is None:
                wants[name] = full.reshape(-1)
            elif plan_here[0] == "shard_parts":
                pieces, at = [], 0
                for n in plan_here[2]:
                    step = n // tp_size
                    pieces.append(full[at + tp_rank * step: at + (tp_rank + 1) * step])
                    at += n
                wants[name] = torch.cat(pieces, 0).reshape(-1)
            else:
                dim = plan_here[1]
                step = full.shape[dim] // tp_size
                wants[name] = full.narrow(dim, tp_rank * step, step).reshape(-1)
            at = 0
            for e0, r, n, pitch in segs:
                bases = [s.data_ptr() for s in shards] + [0] * (8 - n_shards)
                rows.append([dst.data_ptr() + at] + bases + [e0 * es, pitch * es, shard * es, n * es, r])
                at += r * n * es
        table = torch.tensor(rows, dtype=torch.int64).cuda()
        C.reshard_copy(table)
        torch.cuda.synchronize()
        for name in tensors:
            assert torch.equal(dsts[name], wants[name]), (name, n_shards, tp_size, tp_rank)


def test_fused_resharder_fills_a_tensor_parallel_engine_from_a_sharded_model():
    """End to end on one GPU: training model in flat unit buffers -> engine model cut for tp rank
    0 and 1 of 2, every engine tensor equal to the slice of the training parameter."""
    import os
    from functools import partial

    from halite_b200.conf import instantiate
    from halite_b200.conf.loader import load_module
    from halite_b200.infer.tensor_parallel import apply_infer_tp
    from halite_b200.parallel import parallelize
    from halite_b200.parallel.reshard import FusedResharder
    from halite_b200.distributed.state_dict import reshard_state_dict
    from tests.helpers import ROOT

    zoo = load_module(os.path.join(ROOT, "configs/models/transformer.py"))
    kw = dict(vocab_size=1024, dim=256, n_heads=4, head_dim=64, n_layers=2, intermediate_size=512, context_len=256,
              n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=False, gated_ff_split=True,
              init=partial(torch.nn.init.normal_, std=0.02))
    cfg = zoo.transformer(**kw)
    with torch.device("meta"):
        model = instantiate(cfg)
    model = parallelize(model, None, None, device=torch.device("cuda", 0))
    torch.manual_seed(0)
    model.init_weights(torch.device("cuda", 0))
    for tp_rank in range(2):
        with torch.device("meta"):
            imodel = instantiate(instantiate(zoo.transformer_infer(**kw, infer="paged"))(cfg))
        plan = apply_infer_tp(imodel, tp_rank, 2, None)
        target = {k: torch.full(v.shape, float("nan"), device="cuda", dtype=torch.bfloat16)
                  for k, v in imodel.state_dict().items()}
        rs = FusedResharder(model, target, tp_rank, 2, plan)
        assert not rs.fallback
        rs.run()
        torch.cuda.synchronize()
        want = reshard_state_dict(model.state_dict(), imodel.state_dict(), device="cuda", tp_rank=tp_rank, tp_size=2,
                                  tp_plan=plan)
        for k in target:
            assert torch.equal(target[k], want[k]), k
