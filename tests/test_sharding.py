"""Utterance sharding (one process per GPU, no data-path collective): the plan is deterministic and balanced, and two
gloo ranks on CPU agree on it and reduce their timings the way bench.py does (max over ranks)."""
import os
import socket
import zlib

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lokinfer_b200 import sharding


def test_assign_is_a_balanced_partition():
    r = np.random.default_rng(0)
    lengths = r.integers(120, 801, 64).tolist()
    for ws in (1, 2, 4, 8):
        plan = sharding.assign(lengths, ws)
        flat = sorted(i for p in plan for i in p)
        assert flat == list(range(64))
        ld = sharding.loads(lengths, plan)
        assert max(ld) - min(ld) <= max(lengths)
        assert max(ld) <= 1.05 * sum(lengths) / ws + max(lengths) / 2
    assert sharding.assign([], 2) == [[], []]
    assert abs(sharding.audio_seconds([2080]) - 26.0) < 1e-12


def _worker(rank, world, port, lengths, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    plan = sharding.assign(lengths, world)
    mine = plan[rank]
    # every rank derives the same plan; check it by exchanging a hash of the whole plan
    h = torch.tensor([zlib.crc32(str(plan).encode())], dtype=torch.int64)
    hs = [torch.zeros_like(h) for _ in range(world)]
    dist.all_gather(hs, h)
    same = all(int(x) == int(h) for x in hs)
    # the benchmark's reduction: time = max over ranks, units = sum over ranks
    t = torch.tensor([float(sum(lengths[i] for i in mine))], dtype=torch.float64)
    units = t.clone()
    dist.barrier()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(units, op=dist.ReduceOp.SUM)
    if rank == 0:
        out.put((same, float(t), float(units), [len(p) for p in plan]))
    dist.destroy_process_group()


def test_two_gloo_ranks_agree_on_the_plan():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    lengths = np.random.default_rng(1).integers(120, 801, 16).tolist()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, lengths, q)) for r in range(2)]
    for p in procs:
        p.start()
    same, tmax, units, counts = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same and sum(counts) == 16
    assert units == float(sum(lengths))
    assert tmax == float(max(sharding.loads(lengths, sharding.assign(lengths, 2))))
