"""Rank script: StatelessProcessGroup objects and barrier over a TCPStore; rank 2 (when
present) skips the second barrier so the others see the timeout error instead of hanging."""

import os
import sys

from halite_b200.distributed.process_group import StatelessProcessGroup

rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
port = int(sys.argv[1])
pg = StatelessProcessGroup.create("127.0.0.1", port, rank, ws)
got = pg.all_gather_obj({"rank": rank, "payload": list(range(rank + 1))})
assert [g["rank"] for g in got] == list(range(ws))
assert pg.broadcast_obj("hello" if rank == 1 else None, src=1) == "hello"
pg.send_obj(("to", (rank + 1) % ws, "from", rank), dst=(rank + 1) % ws)
msg = pg.recv_obj(src=(rank - 1) % ws)
assert msg == ("to", rank, "from", (rank - 1) % ws)
pg.barrier(timeout=20)
status = "ok"
if ws >= 3:
    if rank == 2:
        status = "absent"          # never joins the second barrier
    else:
        try:
            pg.barrier(timeout=1.0)
            status = "no-timeout"
        except RuntimeError as e:
            status = "timeout:" + str(e)[-12:]
print(f"RESULT rank={rank} {status}")
if rank == 0:
    import time
    time.sleep(1.5)                # keep the store alive until the others have finished
