"""Row-sharded driver on two CPU ranks over gloo; the per-rank forward is the oracle."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import dlrnet_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, out_dir):
    import sys
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [here, os.path.join(here, "ml-dlr-lock_b200")]
    from dlr_lock_b200.sharding import RowShardedForward
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    p, x = O.seeded_case(64, 16, 6, M, seed=5, alpha=0.5)
    p32 = p.to(torch.float32)
    drv = RowShardedForward(lambda xb: O.forward_fp32(xb, p32), tile=4)
    y = drv(x.float())
    a, b = drv.local_rows(M)
    torch.save({"y": y, "rows": (a, b)}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _run(M, tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, M, str(tmp_path)), nprocs=world, join=True)
    p, x = O.seeded_case(64, 16, 6, M, seed=5, alpha=0.5)
    want = O.forward_fp32(x.float(), p.to(torch.float32))
    got = [torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(world)]
    for g in got:
        assert g["y"].shape == want.shape
        assert torch.allclose(g["y"], want, atol=1e-5)
    rows = [g["rows"] for g in got]
    assert rows[0][0] == 0 and rows[0][1] == rows[1][0] and rows[1][1] == M


def test_two_ranks_ragged(tmp_path):
    _run(11, tmp_path)     # 3 tiles of 4: ranks get 8 and 3 rows


def test_fewer_rows_than_a_tile(tmp_path):
    _run(3, tmp_path)      # rank 1 gets nothing and still takes part in the gather
