"""The multi-rank statistics gather on CPU ranks (gloo, world size 2)."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, lanes, queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    entry.load_package()
    from gradoom_b200 import stats

    owned = stats.lane_slice(rank, world, lanes)
    sb = torch.zeros((lanes, 27))
    sb[:, 0] = torch.tensor([float(g) for g in owned])          # killcount = global lane id
    sb[:, 17] = 100.0 + rank
    sb[:, 26] = torch.tensor([2.0 * g for g in owned])
    gathered = stats.gather_lane_stats(sb)
    queue.put((rank, gathered.clone()))
    dist.barrier()
    dist.destroy_process_group()


def test_all_gather_orders_lanes_globally():
    world, lanes = 2, 5
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, lanes, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank in range(world):
        g = results[rank]
        assert g.shape == (world * lanes, 4)
        assert g[:, 0].tolist() == [float(i) for i in range(world * lanes)]
        assert g[:, 1].tolist() == [100.0] * lanes + [101.0] * lanes
        assert g[:, 3].tolist() == [2.0 * i for i in range(world * lanes)]
