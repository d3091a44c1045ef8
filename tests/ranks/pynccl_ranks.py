"""Rank script (one process per GPU): the ctypes NCCL communicator, created outside
torch.distributed, against known answers."""

import os
import sys

import torch

from halite_b200.distributed.process_group import stateless_init_process_group

rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
port = int(sys.argv[1])
torch.cuda.set_device(rank)
comm = stateless_init_process_group("127.0.0.1", port, rank, ws, torch.device("cuda", rank))
x = torch.full((1024,), float(rank + 1), device="cuda", dtype=torch.bfloat16)
assert comm.all_reduce(x).float().mean().item() == sum(range(1, ws + 1))
g = torch.empty(ws * 8, device="cuda")
comm.all_gather(g, torch.full((8,), float(rank), device="cuda"))
assert g.view(ws, 8)[:, 0].tolist() == list(map(float, range(ws)))
sizes = [r + 1 for r in range(ws)]
gv = torch.empty(sum(sizes), 4, device="cuda")
comm.all_gatherv(gv, torch.full((rank + 1, 4), float(rank), device="cuda"), sizes)
want = torch.cat([torch.full((r + 1,), float(r)) for r in range(ws)])
assert gv[:, 0].cpu().tolist() == want.tolist()
rs = torch.empty(4, device="cuda")
comm.reduce_scatter(rs, torch.arange(ws * 4, device="cuda", dtype=torch.float32))
assert rs.cpu().tolist() == [ws * (rank * 4 + i) for i in range(4)]
rv = torch.empty(rank + 1, 4, device="cuda")
comm.reduce_scatterv(rv, torch.ones(sum(sizes), 4, device="cuda"), sizes)
assert rv.cpu().eq(ws).all()
b = torch.arange(16, device="cuda", dtype=torch.float32) if rank == 0 else torch.zeros(16, device="cuda")
comm.broadcast(b, src=0)
assert b.cpu().tolist() == list(map(float, range(16)))
if ws >= 2:
    if rank == 0:
        comm.send(torch.full((5,), 7.0, device="cuda"), dst=1)
    elif rank == 1:
        r = torch.zeros(5, device="cuda")
        comm.recv(r, src=0)
        assert r.cpu().eq(7).all()
torch.cuda.synchronize()
comm.group.barrier(timeout=30)
comm.destroy()
print(f"RESULT rank={rank} nccl {comm.nccl.ncclGetVersion()}")
